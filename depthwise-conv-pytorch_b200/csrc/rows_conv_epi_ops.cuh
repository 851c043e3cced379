// Rows family: the forward with a fused epilogue (scale, bias, activation applied to the
// accumulator before the store).  Same kernels as the plain forward, compiled with EPI; one
// translation unit per element type.
#pragma once

#include "rows_conv_impl.cuh"

namespace dwb {

template <typename T>
int rows_forward_epilogue(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep,
                          cudaStream_t st) {
  if constexpr (!RowsDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (s.kh > 7 || !conv_shape_ok(s, false)) return ROWS_DECLINED;  // large filters: other families
    RowsParams p{};
    p.in = x; p.w = w; p.out = y;
    p.NC = s.N * s.C; p.C = s.C;
    p.Hin = s.H; p.Win = s.W; p.Hout = s.Ho; p.Wout = s.Wo;
    p.flip = 0;
    p.ep = ep;
    return select_k<T, MODE_FWD, true>(p, s.kh, s.sh, st);
  }
}

}  // namespace dwb
