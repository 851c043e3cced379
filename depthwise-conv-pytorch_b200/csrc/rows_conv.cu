// Rows family, forward and backward-input: the plain operators.
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
// test-suite models the kernels' index arithmetic on the CPU from these numbers.
int rows_debug_conv_plan(int op, int esize, const Shape &s, int a16, int *out) {
  // only alignment matters for selection; the pointers are never dereferenced
  const void *fake = reinterpret_cast<const void *>(a16 ? (uintptr_t)0x1000 : (uintptr_t)0x1004);
  t_plan_out = out;
  int r = ROWS_DECLINED;
  if (esize == 4)
    r = op == 0 ? rows_forward<float>((const float *)fake, (const float *)fake, (float *)fake, s, nullptr)
                : rows_backward_input<float>((const float *)fake, (const float *)fake, (float *)fake, s, nullptr);
  else if (esize == 2)
    r = op == 0 ? rows_forward<__half>((const __half *)fake, (const __half *)fake, (__half *)fake, s, nullptr)
                : rows_backward_input<__half>((const __half *)fake, (const __half *)fake, (__half *)fake, s, nullptr);
  t_plan_out = nullptr;
  return r == ROWS_SERVED ? 1 : 0;
}

int rows_conv_epi_take_error();  // rows_conv_epi.cu
int tiles_tma_take_error();      // tiles_tma.cu
int nhwc_tma_take_error();       // nhwc_tma.cu

int rows_conv_take_error() {
  return conv_take_error_here() | rows_conv_epi_take_error() | rows_bigk_take_error() |
         tiles_tma_take_error() | nhwc_tma_take_error();
}

template int rows_forward<float>(const float *, const float *, float *, const Shape &, cudaStream_t);
template int rows_forward<__half>(const __half *, const __half *, __half *, const Shape &, cudaStream_t);
template int rows_forward<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, const Shape &, cudaStream_t);
template int rows_forward<double>(const double *, const double *, double *, const Shape &, cudaStream_t);
template int rows_backward_input<float>(const float *, const float *, float *, const Shape &, cudaStream_t);
template int rows_backward_input<__half>(const __half *, const __half *, __half *, const Shape &, cudaStream_t);
template int rows_backward_input<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, const Shape &, cudaStream_t);
template int rows_backward_input<double>(const double *, const double *, double *, const Shape &, cudaStream_t);

}  // namespace dwb
