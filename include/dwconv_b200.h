/*
 * dwconv_b200 -- depthwise conv2d (forward, backward-input, backward-filter)
 * for NVIDIA B200 (sm_100a).  C ABI of libdwconv_b200.so.
 *
 * The library is the device side of a drop-in for the `torch_dwconv` extension
 * of rosinality/depthwise-conv-pytorch.  That extension exports four functions
 * from a pybind11 module (torch_dwconv/dwconv.cpp:60-67); each of them has a
 * counterpart below that takes raw device pointers, sizes and a stream instead
 * of torch tensors.  The operators never allocate: the caller owns inputs,
 * outputs and the backward workspace.  (The one allocating entry point is
 * dwconv_b200_exchange_create, which makes the buffer that peers' GPUs write
 * into for the multi-GPU sum; it is not on the per-call path.)
 *
 * Conventions
 *   - activations are contiguous NCHW, filters contiguous [C,1,kh,kw];
 *   - every pointer is a device pointer of the CURRENT device, aligned to the
 *     element size (faster kernels are chosen when it is 16-byte aligned);
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); every
 *     call is asynchronous on it and never synchronises;
 *   - every call returns a dwconv_b200_status; nothing is launched unless the
 *     arguments validated, and every launch is followed by an error check;
 *   - fp16 data is accumulated in fp32 and rounded once; fp32 in fp32; fp64 in
 *     fp64.  Forward and backward-input add the taps in row-major order into
 *     a single accumulator with one fused multiply-add per tap, which is the
 *     order of the reference kernels (torch_dwconv/dwconv_kernel.cu:164-172),
 *     so fp32 results are bit-identical to it.  Backward-filter is a
 *     deterministic two-pass tree reduction (the reference uses atomics,
 *     dwconv_kernel.cu:303-305,:583).
 *   - the library is re-entrant; it keeps no state besides once-only kernel
 *     attribute set-up.
 */
#ifndef DWCONV_B200_H_
#define DWCONV_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DWCONV_B200_API __attribute__((visibility("default")))
#else
#define DWCONV_B200_API
#endif

#define DWCONV_B200_VERSION 200 /* major*10000 + minor*100 + patch */

typedef enum dwconv_b200_dtype {
  DWCONV_B200_F32 = 0,
  DWCONV_B200_F16 = 1,  /* accumulates in fp32 (the reference accumulates in half) */
  DWCONV_B200_F64 = 2,
  DWCONV_B200_BF16 = 3  /* not in the reference; fp32 accumulation; general-purpose kernels only */
} dwconv_b200_dtype;

typedef enum dwconv_b200_status {
  DWCONV_B200_OK = 0,
  DWCONV_B200_BAD_ARGUMENT = 1,       /* null pointer, non-positive extent, an exchange object of another layer */
  DWCONV_B200_UNSUPPORTED_DTYPE = 2,
  DWCONV_B200_MISALIGNED = 3,         /* pointer not aligned to its element size */
  DWCONV_B200_WORKSPACE_TOO_SMALL = 4,
  DWCONV_B200_CUDA_ERROR = 5,         /* a launch failed; see dwconv_b200_last_cuda_error */
  DWCONV_B200_UNSUPPORTED_SHAPE = 6,  /* a forced kernel family cannot serve this shape */
  DWCONV_B200_TOO_LARGE = 7           /* an extent exceeds what the entry point accepts */
} dwconv_b200_status;

/* Kernel families, for dwconv_b200_set_path / dwconv_b200_last_path. */
typedef enum dwconv_b200_path {
  DWCONV_B200_PATH_AUTO = 0,    /* choose per shape (default) */
  DWCONV_B200_PATH_DIRECT = 1,  /* one thread per output, any shape / dtype */
  DWCONV_B200_PATH_ROWS = 2,    /* bulk-copy staged row tiles, lane-per-column warps */
  DWCONV_B200_PATH_TILES = 3    /* shared-memory tiles, any padding and map size (3x3/5x5/7x7) */
} dwconv_b200_path;

/* Geometry of one depthwise convolution in forward terms.
 * Ho = floor((H + 2*ph - kh)/sh) + 1 for symmetric padding; a caller with a
 * different bottom/right padding passes the Ho/Wo it wants (any value with
 * 1 <= Ho and (Ho-1)*sh - ph + kh <= H + "bottom padding" is meaningful: rows
 * outside the input read as zero). */
typedef struct dwconv_b200_shape {
  int N, C, H, W; /* input  [N,C,H,W]  */
  int kh, kw;     /* filter [C,1,kh,kw] */
  int sh, sw;     /* stride */
  int ph, pw;     /* top / left zero padding */
  int Ho, Wo;     /* output [N,C,Ho,Wo] */
} dwconv_b200_shape;

DWCONV_B200_API int dwconv_b200_version(void);
DWCONV_B200_API const char *dwconv_b200_status_string(int status);
/* cudaError_t of the most recent failed launch on the calling thread (0 if none). */
DWCONV_B200_API int dwconv_b200_last_cuda_error(void);

/* Every wait inside a kernel (on a bulk copy landing in shared memory) is bounded; a kernel
 * whose wait expires raises a flag, finishes without hanging and leaves wrong output.
 * This call synchronises the device, returns the flags raised since the last call (0 = none;
 * bit 0 forward/backward-input kernels, bit 1 backward-filter kernels, bit 2 the exchange between
 * GPUs) and clears them.
 * Diagnostic: not needed on the hot path.  No counterpart in the reference. */
DWCONV_B200_API int dwconv_b200_device_status(void);

/* Host-only: the kernel variant and tiling the rows family would use for an operator
 * (op 0 forward, 1 backward-input, 2 backward-filter, 3 fused backward), as 24 ints; returns 0 if that family
 * declines the problem.  For tests that model the kernels' index arithmetic on the CPU.
 * No counterpart in the reference. */
DWCONV_B200_API int dwconv_b200_debug_plan(int op, int dtype, const dwconv_b200_shape *shape,
                                           int aligned16, int *out24);

/* Force a kernel family (testing / profiling).  Process-wide; returns the previous value. */
DWCONV_B200_API int dwconv_b200_set_path(int path);
/* Kernel family that served the calling thread's most recent call. */
DWCONV_B200_API int dwconv_b200_last_path(void);

/* Output extent of up/pad/correlate/decimate:
 * (in*up + pad0 + pad1 - k + down) / down.
 * Replaces make_conv2d_params, torch_dwconv/dwconv_kernel.cu:612-615. */
DWCONV_B200_API int dwconv_b200_out_size(int in, int up, int pad0, int pad1, int k, int down);

/* ------------------------------------------------------------------------
 * Natural-form entry points (what the Python autograd function calls).
 * ---------------------------------------------------------------------- */

/* y = depthwise cross-correlation of x with w.
 * Replaces dwconv2d(..., forward=true) and dwconv2d_small(..., forward=true),
 * torch_dwconv/dwconv.cpp:27-46, as called at torch_dwconv/dwconv.py:28-35. */
DWCONV_B200_API int dwconv_b200_forward(const void *x, const void *w, void *y, int dtype,
                        const dwconv_b200_shape *shape, void *stream);

/* dx = gradient of the forward w.r.t. x, given dy [N,C,Ho,Wo]; dx is [N,C,H,W]
 * and every element of it is written (rows/columns no window reaches get 0).
 * Replaces dwconv2d(..., forward=false) and dwconv2d_small(..., forward=false),
 * torch_dwconv/dwconv.cpp:27-46, as called at torch_dwconv/dwconv.py:56-64. */
DWCONV_B200_API int dwconv_b200_backward_input(const void *dy, const void *w, void *dx, int dtype,
                               const dwconv_b200_shape *shape, void *stream);

/* Scratch bytes dwconv_b200_backward_filter needs for this geometry (>= 16). */
DWCONV_B200_API size_t dwconv_b200_backward_filter_workspace_bytes(int dtype, const dwconv_b200_shape *shape);

/* dw [C,1,kh,kw] = gradient w.r.t. the filter.  `workspace` is caller-owned
 * device scratch of at least the size reported above, 16-byte aligned; it is
 * fully overwritten, never read before being written.
 * Replaces dwconv2d_backward_kernel, torch_dwconv/dwconv.cpp:48-58, as called
 * at torch_dwconv/dwconv.py:66-68 (which also zero-fills dW first,
 * dwconv_kernel.cu:1026-1027; not needed here). */
DWCONV_B200_API int dwconv_b200_backward_filter(const void *x, const void *dy, void *dw, void *workspace,
                                size_t workspace_bytes, int dtype,
                                const dwconv_b200_shape *shape, void *stream);

/* ------------------------------------------------------------------------
 * Forward with a fused epilogue (opt-in; no counterpart in the reference, which
 * rejects a bias outright, torch_dwconv/dwconv.py:108-109).
 *   y = act(conv(x, w) * scale[c] + bias[c])
 * applied to the accumulator (fp32; fp64 for f64 data) before the one rounding to
 * the storage type.  `scale` and `bias` are [C] arrays of the tensors' element
 * type on the device, each may be NULL (1 resp. 0).  This is what follows a
 * depthwise convolution in the blocks that use one (folded batch-norm scale and
 * shift, then ReLU6 / SiLU / hard-swish); done separately it costs another read
 * and write of the output map.  Every shape and dtype dwconv_b200_forward
 * serves is served.  A NULL `epilogue`, or one with no scale, no bias and no
 * activation, is the plain forward.
 * ---------------------------------------------------------------------- */
typedef enum dwconv_b200_activation {
  DWCONV_B200_ACT_NONE = 0,
  DWCONV_B200_ACT_RELU = 1,
  DWCONV_B200_ACT_RELU6 = 2,
  DWCONV_B200_ACT_SILU = 3,      /* v * sigmoid(v) */
  DWCONV_B200_ACT_HARDSWISH = 4  /* v * relu6(v + 3) / 6 */
} dwconv_b200_activation;

typedef struct dwconv_b200_epilogue {
  const void *scale; /* [C] or NULL */
  const void *bias;  /* [C] or NULL */
  int activation;    /* dwconv_b200_activation */
} dwconv_b200_epilogue;

DWCONV_B200_API int dwconv_b200_forward_epilogue(const void *x, const void *w, void *y, int dtype,
                                                 const dwconv_b200_shape *shape,
                                                 const dwconv_b200_epilogue *epilogue, void *stream);

/* ------------------------------------------------------------------------
 * Channels-last (NHWC) operators: activations laid out x[n][h][w][c]
 * (torch.channels_last), filters [C,1,kh,kw] as everywhere.  The reference makes
 * every operand contiguous NCHW first (torch_dwconv/dwconv_kernel.cu:741-742,
 * 855-856,1023-1024), which costs a channels-last caller an extra read and write
 * of each map; these read and write NHWC in place.  `shape` has the same meaning
 * as for the NCHW entry points.  Served: square 3x3 / 5x5 / 7x7 filters, equal
 * strides 1 or 2, any padding, f32 / f16 / bf16; anything else returns
 * DWCONV_B200_UNSUPPORTED_SHAPE (make the maps contiguous NCHW and use the
 * entry points above).  Same summation order as the NCHW kernels: the same
 * values give the same bits.  forward_nhwc takes the optional epilogue of
 * dwconv_b200_forward_epilogue (NULL: none); backward_filter_nhwc takes the
 * workspace of dwconv_b200_backward_filter (same size query).
 * ---------------------------------------------------------------------- */
DWCONV_B200_API int dwconv_b200_forward_nhwc(const void *x, const void *w, void *y, int dtype,
                                             const dwconv_b200_shape *shape,
                                             const dwconv_b200_epilogue *epilogue, void *stream);
DWCONV_B200_API int dwconv_b200_backward_input_nhwc(const void *dy, const void *w, void *dx, int dtype,
                                                    const dwconv_b200_shape *shape, void *stream);
DWCONV_B200_API int dwconv_b200_backward_filter_nhwc(const void *x, const void *dy, void *dw,
                                                     void *workspace, size_t workspace_bytes, int dtype,
                                                     const dwconv_b200_shape *shape, void *stream);
/* Both gradients of channels-last maps in one call (what the reference's backward computes,
 * torch_dwconv/dwconv.py:56-68, for NHWC tensors): dx as dwconv_b200_backward_input_nhwc (bit for
 * bit), dw as dwconv_b200_backward_filter_nhwc to rounding.  At stride 1 with a 3x3 or 5x5 filter
 * both come from ONE pass over dy; other geometries run the two operators.  Workspace as for
 * dwconv_b200_backward_filter. */
DWCONV_B200_API int dwconv_b200_backward_nhwc(const void *x, const void *dy, const void *w, void *dx,
                                              void *dw, void *workspace, size_t workspace_bytes,
                                              int dtype, const dwconv_b200_shape *shape, void *stream);

/* Both gradients from ONE pass over dy: dx as dwconv_b200_backward_input (bit for bit),
 * dw as dwconv_b200_backward_filter (same two-pass reduction; the partial sums are
 * accumulated in another order, so dw agrees to rounding, not bit for bit).  For the
 * shapes the tiled kernels serve (3x3 / 5x5 / 7x7, stride 1 or 2, padding k/2, fp32 and
 * fp16, maps up to 128 columns) the first pass is one kernel that stages the dy rows and
 * the x rows of a group of planes in shared memory and uses every dy window value twice;
 * other shapes run backward-input and backward-filter one after the other.  `workspace`
 * as for dwconv_b200_backward_filter (same size query).
 * Replaces the pair of calls at torch_dwconv/dwconv.py:56-68 (dwconv2d(forward=false)
 * followed by dwconv2d_backward_kernel), which read dy from memory twice. */
DWCONV_B200_API int dwconv_b200_backward(const void *x, const void *dy, const void *w, void *dx, void *dw,
                                         void *workspace, size_t workspace_bytes, int dtype,
                                         const dwconv_b200_shape *shape, void *stream);

/* As dwconv_b200_backward, but the filter gradient goes to an ACCUMULATOR-typed buffer
 * dw_acc [C,1,kh,kw] (float for f32 / f16 / bf16 data, double for f64): dw_acc = sum when
 * `accumulate` is 0, dw_acc += sum otherwise.  For a batch processed in chunks (calls on one
 * stream add in call order: deterministic).  dx (and then w) may be null: filter gradient only.
 * No counterpart in the reference, which zero-fills and adds with atomics inside one call
 * (dwconv_kernel.cu:1026-1027, :303-305). */
DWCONV_B200_API int dwconv_b200_backward_accumulate(const void *x, const void *dy, const void *w, void *dx,
                                                    void *dw_acc, int accumulate, void *workspace,
                                                    size_t workspace_bytes, int dtype,
                                                    const dwconv_b200_shape *shape, void *stream);

/* One asynchronous copy between any two of: device memory, pinned host memory
 * (direction inferred from the pointers), on `stream`.  A bare copy with nothing recorded
 * around it, for pipelines that move maps between pinned host memory and the
 * device (measured: an event recorded after every chunk's copy costs tens of
 * microseconds per chunk while the other direction is busy).  No counterpart in
 * the reference, whose callers copy with torch. */
DWCONV_B200_API int dwconv_b200_copy_async(void *dst, const void *src, size_t bytes, void *stream);

/* ------------------------------------------------------------------------
 * Filter gradient summed over the GPUs of one node, inside the second pass.
 *
 * The reference has no multi-GPU code; a data-parallel caller of it sums dW
 * with a separate all-reduce after dwconv2d_backward_kernel
 * (torch_dwconv/dwconv.py:66-68).  Here the second pass of the reduction
 * stores each rank's sums straight into its peers' exchange buffers (plain
 * peer stores over NVLink, each 32-bit word in one 8-byte store together with
 * its call number) and the receiving side adds the ranks' values in rank
 * order: every rank ends with the same bits, run after run.  A peer store needs
 * several microseconds to become visible, so the exchange is pipelined: call i
 * sends call i's sums and completes call i-1's.
 *
 *   exchange_bytes    size of one rank's exchange buffer for a layer's filter
 *                     (0: bad arguments; world <= 8).
 *   exchange_create   allocates and zeroes that buffer on the current device
 *                     (the one entry point of this library that allocates) for
 *                     ONE layer geometry (dtype, C, kh, kw) and writes its
 *                     64-byte inter-process handle.  Collect every rank's
 *                     handle (rank order) with any host-side all-gather.
 *   exchange_connect  maps the peers' buffers; `handles` = world x 64 bytes.
 *   backward_filter_exchange
 *                     first pass as dwconv_b200_backward_filter; the second
 *                     pass sends this call's sums to every rank and writes the
 *                     PREVIOUS call's world sum to dw_prev (null: not wanted;
 *                     nothing is written on the first call).
 *   backward_exchange the same with the fused backward's first pass
 *                     (dwconv_b200_backward): dx is written too.
 *   backward_filter_allreduce / backward_allreduce
 *                     the same first passes, but the second pass, after
 *                     sending, waits for the other ranks' words of THIS call
 *                     and writes this call's world sum to dw: the whole
 *                     all-reduce inside the kernel that finishes the gradient.
 *                     For a step with nothing left to run behind the gradient
 *                     (the pipelined form plus exchange_finish costs a second
 *                     kernel and starts waiting later).  May be mixed freely
 *                     with the pipelined calls on one object.
 *   exchange_finish   dw = the world sum of the latest call.  Waits for the
 *                     peers' words if they are still in flight.  A step that
 *                     needs its own sum before it ends calls this after the
 *                     kernels that follow the exchange call in the step
 *                     (they hide the stores' flight time).
 *   exchange_destroy  unmaps the peers' buffers and frees this rank's.  A peer's
 *                     kernel stores into this rank's buffer, so destroy only
 *                     when EVERY rank has finished its last call: synchronise
 *                     the device, meet the other ranks at a host barrier, then
 *                     destroy.
 *
 * Every rank must make the same sequence of backward_filter_exchange calls
 * with the same geometry; one exchange object serves one layer, one call at a
 * time (calls on one stream are).  BAD_ARGUMENT if the shape is not the
 * object's.  A kernel that has waited two seconds for its peers' words
 * stops waiting, leaves that output unwritten and raises bit 2 (value 4) of
 * dwconv_b200_device_status.
 * ---------------------------------------------------------------------- */
typedef struct dwconv_b200_exchange dwconv_b200_exchange;
DWCONV_B200_API size_t dwconv_b200_exchange_bytes(int dtype, int C, int kh, int kw, int world);
DWCONV_B200_API int dwconv_b200_exchange_create(int dtype, int C, int kh, int kw, int world, int rank,
                                                dwconv_b200_exchange **out, unsigned char *handle64);
DWCONV_B200_API int dwconv_b200_exchange_connect(dwconv_b200_exchange *ex, const unsigned char *handles);
DWCONV_B200_API int dwconv_b200_exchange_destroy(dwconv_b200_exchange *ex);
DWCONV_B200_API int dwconv_b200_exchange_finish(void *dw, dwconv_b200_exchange *ex, void *stream);
DWCONV_B200_API int dwconv_b200_backward_filter_exchange(const void *x, const void *dy, void *dw_prev,
                                                         void *workspace, size_t workspace_bytes,
                                                         int dtype, const dwconv_b200_shape *shape,
                                                         dwconv_b200_exchange *ex, void *stream);
DWCONV_B200_API int dwconv_b200_backward_exchange(const void *x, const void *dy, const void *w, void *dx,
                                                  void *dw_prev, void *workspace, size_t workspace_bytes,
                                                  int dtype, const dwconv_b200_shape *shape,
                                                  dwconv_b200_exchange *ex, void *stream);
DWCONV_B200_API int dwconv_b200_backward_filter_allreduce(const void *x, const void *dy, void *dw,
                                                          void *workspace, size_t workspace_bytes,
                                                          int dtype, const dwconv_b200_shape *shape,
                                                          dwconv_b200_exchange *ex, void *stream);
DWCONV_B200_API int dwconv_b200_backward_allreduce(const void *x, const void *dy, const void *w, void *dx,
                                                   void *dw, void *workspace, size_t workspace_bytes,
                                                   int dtype, const dwconv_b200_shape *shape,
                                                   dwconv_b200_exchange *ex, void *stream);

/* ------------------------------------------------------------------------
 * Operator-form entry points: one per function of the reference's pybind
 * module, same argument meaning, pointers instead of tensors.
 * ---------------------------------------------------------------------- */

/* Replaces use_dwconv2d_small, torch_dwconv/dwconv.cpp:3-5,61 and
 * dwconv_kernel.cu:652-662.  Pure host logic; returns 0 or 1. */
DWCONV_B200_API int dwconv_b200_use_dwconv2d_small(int in_h, int in_w, int kh, int kw, int up_h, int up_w,
                                   int down_h, int down_w, int pad_h, int pad_w);

/* Replaces dwconv2d, torch_dwconv/dwconv.cpp:27-35.  forward != 0: requires
 * up == 1 and correlates with stride `down`; forward == 0: requires down == 1
 * and computes the transposed operation with stride `up` (flipped filter,
 * dwconv_kernel.cu:107-114).  `out` is [N,C,out_h,out_w] with
 * out = dwconv_b200_out_size(in, up, pad0, pad1, k, down). */
DWCONV_B200_API int dwconv_b200_dwconv2d(const void *in, const void *kernel, void *out, int dtype, int N, int C,
                         int in_h, int in_w, int kh, int kw, int up_h, int up_w, int down_h,
                         int down_w, int pad_h0, int pad_h1, int pad_w0, int pad_w1, int forward,
                         void *stream);

/* Replaces dwconv2d_small, torch_dwconv/dwconv.cpp:37-46 (symmetric padding). */
DWCONV_B200_API int dwconv_b200_dwconv2d_small(const void *in, const void *kernel, void *out, int dtype, int N,
                               int C, int in_h, int in_w, int kh, int kw, int up_h, int up_w,
                               int down_h, int down_w, int pad_h, int pad_w, int forward,
                               void *stream);

/* Replaces dwconv2d_backward_kernel, torch_dwconv/dwconv.cpp:48-58: `up` must
 * be 1, `down` is the forward stride, `pad` the forward padding. */
DWCONV_B200_API int dwconv_b200_dwconv2d_backward_kernel(const void *input, const void *out_grad, void *dkernel,
                                         void *workspace, size_t workspace_bytes, int dtype,
                                         int N, int C, int in_h, int in_w, int out_h, int out_w,
                                         int kh, int kw, int up_h, int up_w, int down_h,
                                         int down_w, int pad_h, int pad_w, void *stream);

/* ------------------------------------------------------------------------
 * Entry point for callers that must not allocate.  It has no counterpart in
 * the reference (whose operators allocate their results and scratch through
 * PyTorch); it exists for hosts that cannot call cudaMalloc on the path where
 * they need the filter gradient: code running under a fixed device-memory
 * budget handed out at start-up, real-time loops that may not block on the
 * allocator, and plugins whose host owns all device memory.
 *
 * Same result as dwconv_b200_backward_filter, but the partial sums of the
 * two-pass reduction live in a fixed array inside the library's device image
 * instead of a caller-supplied workspace.  The array is
 * DWCONV_B200_STATIC_SCRATCH_BYTES long; every GPU that loads the library
 * holds one copy until the process exits.  The call allocates nothing (no
 * cudaMalloc / cudaFree, no allocating library routine) and never synchronises.
 *
 *   - Limit: C * slices * kh * kw accumulators (4 bytes each, 8 for fp64) must
 *     fit the array; the batch split `slices` is reduced down to 1 to make it
 *     fit, and a geometry that still does not fit (C*kh*kw*4 > the array) is
 *     rejected with DWCONV_B200_TOO_LARGE before anything is launched.
 *   - The first call on each device looks up the array's device address (once
 *     per device, with that device current).  Make that first call outside any
 *     CUDA stream capture.
 *   - Every call on a device shares the one array.  Nothing in it needs to
 *     start at zero (each partial sum is written before it is read), so stale
 *     contents from an earlier call are harmless; but two calls whose kernels
 *     overlap on the GPU (different streams, or different host threads on
 *     different streams) race on it.  Serialise them on one stream or with
 *     events.
 * ---------------------------------------------------------------------- */
#define DWCONV_B200_STATIC_SCRATCH_BYTES (4u << 20)

DWCONV_B200_API size_t dwconv_b200_static_scratch_bytes(void);

DWCONV_B200_API int dwconv_b200_backward_filter_static(const void *x, const void *dy, void *dw,
                                                       int dtype, const dwconv_b200_shape *shape,
                                                       void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DWCONV_B200_H_ */
