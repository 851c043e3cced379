// Rows family, forward and backward-input: the operator templates, instantiated per element type
// in translation units of their own (rows_conv.cu: fp32 and the declining fp64; rows_conv_f16.cu;
// rows_conv_bf16.cu) so that they compile side by side.
#pragma once

#include "rows_conv_impl.cuh"

namespace dwb {

template <typename T> int rows_bigk_conv(const RowsParams &p, int K, cudaStream_t st);  // rows_bigk.cu
int rows_bigk_take_error();

template <typename T>
int rows_forward(const T *x, const T *w, T *y, const Shape &s, cudaStream_t st) {
  if constexpr (!RowsDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    const bool big = s.kh > 7;
    if (!conv_shape_ok(s, big)) return ROWS_DECLINED;
    RowsParams p{};
    p.in = x; p.w = w; p.out = y;
    p.NC = s.N * s.C; p.C = s.C;
    p.Hin = s.H; p.Win = s.W; p.Hout = s.Ho; p.Wout = s.Wo;
    p.flip = 0;
    if (big) return t_plan_out ? ROWS_DECLINED : rows_bigk_conv<T>(p, s.kh, st);
    return select_k<T, MODE_FWD, false>(p, s.kh, s.sh, st);
  }
}

template <typename T>
int rows_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st) {
  if constexpr (!RowsDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    const bool big = s.kh > 7;
    if (!conv_shape_ok(s, big)) return ROWS_DECLINED;
    RowsParams p{};
    p.in = dy; p.w = w; p.out = dx;
    p.NC = s.N * s.C; p.C = s.C;
    p.Hin = s.Ho; p.Win = s.Wo; p.Hout = s.H; p.Wout = s.W;
    p.flip = 1;
    if (big) return t_plan_out ? ROWS_DECLINED : rows_bigk_conv<T>(p, s.kh, st);
    // stride 1: the transposed operation is the same correlation with the flipped filter
    return select_k<T, MODE_BWD, false>(p, s.kh, s.sh, st);
  }
}

// Variant and tiling forward (op 0) or backward-input (op 1) would use, for inspection: the
// test-suite models the kernels' index arithmetic on the CPU from these numbers.  Must run in the
// translation unit that holds T's kernels (the plan is handed over in a variable of that unit):
// nothing is launched while it is set.
template <typename T>
int rows_debug_conv_plan_t(int op, const Shape &s, int a16, int *out) {
  // only alignment matters for selection; the pointers are never dereferenced
  const T *fake = reinterpret_cast<const T *>(a16 ? (uintptr_t)0x1000 : (uintptr_t)0x1004);
  t_plan_out = out;
  const int r = op == 0 ? rows_forward<T>(fake, fake, const_cast<T *>(fake), s, nullptr)
                        : rows_backward_input<T>(fake, fake, const_cast<T *>(fake), s, nullptr);
  t_plan_out = nullptr;
  return r == ROWS_SERVED ? 1 : 0;
}

}  // namespace dwb
