// Host entry points of the rows kernel family (defined in rows_conv.cu / rows_filter.cu).
// Each returns ROWS_SERVED after enqueueing its kernel, or ROWS_DECLINED without launching
// anything when the geometry, dtype or alignment is outside what the family covers.
#pragma once

#include "common.cuh"

namespace dwb {

// ROWS_SERVED_DW: served, and the kernel finished the filter gradient itself (no second pass).
enum { ROWS_DECLINED = 0, ROWS_SERVED = 1, ROWS_SERVED_DW = 2 };

template <typename T> int rows_forward(const T *x, const T *w, T *y, const Shape &s, cudaStream_t st);
// The forward with a fused epilogue (rows_conv_epi.cu); 3x3 / 5x5 / 7x7 only.
template <typename T>
int rows_forward_epilogue(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep,
                          cudaStream_t st);
template <typename T>
int rows_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st);
// Batch/row slices per channel the first pass would use (0: declines); sizes the workspace.
template <typename T> int rows_backward_filter_slices(const Shape &s);
template <typename T>
int rows_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                         cudaStream_t st, int *slices_out);

// Fused backward: dx and the first pass of dW (partial sums, as rows_backward_filter) from one
// read of dy.  With `dw_direct` the kernel may finish dW itself (thread-block clusters over the
// slices, small problems) and then returns ROWS_SERVED_DW.
template <typename T> int rows_backward_slices(const Shape &s);
template <typename T>
int rows_backward(const T *x, const T *dy, const T *w, T *dx, typename Elem<T>::acc_t *partial,
                  const Shape &s, cudaStream_t st, int *slices_out, T *dw_direct);

// Tiles family (tiles.cu): any padding, any map size; 3x3 / 5x5 / 7x7; fp32, fp16, bf16.
template <typename T>
int tiles_forward(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep, cudaStream_t st);
template <typename T>
int tiles_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st);
// Upper bound of the slices per channel the tiles family's filter-gradient first pass uses
// (0: the family does not serve the shape); sizes the workspace.
int tiles_filter_slices(const Shape &s);
// `slices` is that bound; *slices_used (<= slices) is what the launch wrote.
template <typename T>
int tiles_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                          int slices, cudaStream_t st, int *slices_used);

// Channels-last (NHWC) operators (nhwc.cu): 3x3 / 5x5 / 7x7, stride 1 or 2, any padding; fp32,
// fp16, bf16.
int nhwc_filter_slices(const Shape &s);
template <typename T>
int nhwc_forward(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep, cudaStream_t st);
template <typename T>
int nhwc_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st);
template <typename T>
int nhwc_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                         cudaStream_t st, int *slices_out);
// Both gradients from one pass over dy where the channels-last tensor-copy kernels can (stride 1,
// 3x3 / 5x5); ROWS_DECLINED otherwise.
template <typename T>
int nhwc_backward(const T *x, const T *dy, const T *w, T *dx, typename Elem<T>::acc_t *partial,
                  const Shape &s, cudaStream_t st, int *slices_out);

// Reads and clears the flags kernels raise when a bounded wait expires (synchronises the
// device).  Bit 0: forward/backward-input kernels, bit 1: backward-filter kernels.
int rows_take_device_error();
// Variant and tiling a call would use, as 24 ints (0 returned: the family declines):
// VI, VO, U, mask, LW, G, NRT, TH, NRB, RBH, PS, ZT, ZBF, TAPB, DPL, DYOFF, ntiles|TPC, SL, mode.
int rows_debug_conv_plan(int op, int esize, const Shape &s, int a16, int *out);
int rows_debug_filter_plan(int esize, const Shape &s, int a16, int *out);
int rows_debug_backward_plan(int esize, const Shape &s, int a16, int *out);
int rows_conv_take_error();
int rows_filter_take_error();
int rows_backward_take_error();

}  // namespace dwb
