// Rows family: the forward with a fused epilogue (scale, bias, activation applied to the
// accumulator before the store).  Same kernels as the plain forward, compiled with EPI.
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

int rows_conv_epi_take_error() { return conv_take_error_here(); }

template int rows_forward_epilogue<float>(const float *, const float *, float *, const Shape &, const EpilogueArgs &, cudaStream_t);
template int rows_forward_epilogue<__half>(const __half *, const __half *, __half *, const Shape &, const EpilogueArgs &, cudaStream_t);
template int rows_forward_epilogue<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, const Shape &, const EpilogueArgs &, cudaStream_t);
template int rows_forward_epilogue<double>(const double *, const double *, double *, const Shape &, const EpilogueArgs &, cudaStream_t);

}  // namespace dwb
