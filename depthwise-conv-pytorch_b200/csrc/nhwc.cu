// Channels-last (NHWC) operators: variant selection and launches (kernels: nhwc_kernels.cuh).
#include "nhwc_kernels.cuh"
#include "rows_api.cuh"

namespace dwb {

// nhwc_tma.cu: the same operators with their tiles brought in by tensor copies.
template <typename T>
int nhwc_tma_conv(const T *in, const T *w, T *out, const NhwcParams &p, int K, int S, cudaStream_t st);
template <typename T>
int nhwc_tma_bwd2(const T *dy, const T *w, T *dx, const NhwcParams &p, int K, cudaStream_t st);
template <typename T>
int nhwc_tma_backward(const T *x, const T *dy, const T *w, T *dx, float *partial, const NhwcFilterParams &p,
                      int K, cudaStream_t st);
template <typename T>
int nhwc_tma_filter(const T *x, const T *dy, float *partial, const NhwcFilterParams &p, int K, int S,
                    cudaStream_t st);

namespace {

template <typename T> struct NhwcDtype { static constexpr bool ok = false; };
template <> struct NhwcDtype<float> { static constexpr bool ok = true; };
template <> struct NhwcDtype<__half> { static constexpr bool ok = true; };
template <> struct NhwcDtype<__nv_bfloat16> { static constexpr bool ok = true; };

inline bool nhwc_filter_ok(const Shape &s) {
  return s.kh == s.kw && (s.kh == 3 || s.kh == 5 || s.kh == 7) && s.sh == s.sw &&
         (s.sh == 1 || s.sh == 2);
}

template <typename T, int K, int S, int UP>
void launch_conv(const T *in, const T *w, T *out, NhwcParams p, cudaStream_t st) {
  using G = NhwcGeo<K, S>;
  p.tiles_x = ceil_div(p.Wout, G::TW);
  p.tiles_y = ceil_div(p.Hout, G::R);
  p.cblocks = ceil_div(p.C, NHWC_CB);
  p.ntiles = (long long)p.N * p.tiles_x * p.tiles_y * p.cblocks;
  const long long cap = 148ll * 16;  // grid-stride beyond this
  const int grid = (int)(p.ntiles < cap ? p.ntiles : cap);
  nhwc_conv_kernel<T, K, S, UP><<<grid, G::THREADS, 0, st>>>(in, w, out, p);
}

template <typename T, int K, int S>
void launch_filter(const T *x, const T *dy, float *partial, NhwcFilterParams p, cudaStream_t st) {
  using G = NhwcGeo<K, S, true>;
  p.tiles_x = ceil_div(p.Wo, G::TW);
  p.tiles_y = ceil_div(p.Ho, G::R);
  p.cblocks = ceil_div(p.C, NHWC_CB);
  nhwc_filter_kernel<T, K, S><<<p.cblocks * p.SL, G::THREADS, 0, st>>>(x, dy, partial, p);
}

}  // namespace

// Slices of the (image, tile) list per block of 32 channels: about four CTAs per SM in all,
// never more slices than tiles.
int nhwc_filter_slices(const Shape &s) {
  if (!nhwc_filter_ok(s)) return 1;
  const int cblocks = ceil_div(s.C, NHWC_CB);
  const int R = nhwc_rows(s.kh, s.sh, true), TW = s.sh == 1 ? 16 : 8;
  const long long total = (long long)s.N * ceil_div(s.Ho, R) * ceil_div(s.Wo, TW);
  long long SL = ceil_div(4 * 148, cblocks);
  if (SL > total) SL = total;
  return SL < 1 ? 1 : (int)SL;
}

template <typename T>
int nhwc_forward(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep, cudaStream_t st) {
  if constexpr (!NhwcDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!nhwc_filter_ok(s)) return ROWS_DECLINED;
    NhwcParams p{};
    p.N = s.N; p.C = s.C; p.Hin = s.H; p.Win = s.W; p.Hout = s.Ho; p.Wout = s.Wo;
    p.pt = s.ph; p.pl = s.pw; p.flip = 0; p.ep = ep;
    if (nhwc_tma_conv<T>(x, w, y, p, s.kh, s.sh, st) == ROWS_SERVED) return ROWS_SERVED;
    switch (s.kh * 10 + s.sh) {
      case 31: launch_conv<T, 3, 1, 1>(x, w, y, p, st); break;
      case 51: launch_conv<T, 5, 1, 1>(x, w, y, p, st); break;
      case 71: launch_conv<T, 7, 1, 1>(x, w, y, p, st); break;
      case 32: launch_conv<T, 3, 2, 1>(x, w, y, p, st); break;
      case 52: launch_conv<T, 5, 2, 1>(x, w, y, p, st); break;
      case 72: launch_conv<T, 7, 2, 1>(x, w, y, p, st); break;
      default: return ROWS_DECLINED;
    }
    return ROWS_SERVED;
  }
}

// The stride-1 correlation of dy, up-sampled by the forward stride and padded by k-1-p, with the
// flipped filter (torch_dwconv/dwconv.py:39-44,57-64).
template <typename T>
int nhwc_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st) {
  if constexpr (!NhwcDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!nhwc_filter_ok(s) || s.ph > s.kh - 1 || s.pw > s.kw - 1) return ROWS_DECLINED;
    NhwcParams p{};
    p.N = s.N; p.C = s.C; p.Hin = s.Ho; p.Win = s.Wo; p.Hout = s.H; p.Wout = s.W;
    p.pt = s.kh - 1 - s.ph; p.pl = s.kw - 1 - s.pw; p.flip = 1;
    p.ep = EpilogueArgs{nullptr, nullptr, 0, 0};
    if (s.sh == 1 && nhwc_tma_conv<T>(dy, w, dx, p, s.kh, 1, st) == ROWS_SERVED) return ROWS_SERVED;
    if (s.sh == 2 && nhwc_tma_bwd2<T>(dy, w, dx, p, s.kh, st) == ROWS_SERVED) return ROWS_SERVED;
    switch (s.kh * 10 + s.sh) {
      case 31: launch_conv<T, 3, 1, 1>(dy, w, dx, p, st); break;
      case 51: launch_conv<T, 5, 1, 1>(dy, w, dx, p, st); break;
      case 71: launch_conv<T, 7, 1, 1>(dy, w, dx, p, st); break;
      case 32: launch_conv<T, 3, 1, 2>(dy, w, dx, p, st); break;
      case 52: launch_conv<T, 5, 1, 2>(dy, w, dx, p, st); break;
      case 72: launch_conv<T, 7, 1, 2>(dy, w, dx, p, st); break;
      default: return ROWS_DECLINED;
    }
    return ROWS_SERVED;
  }
}

// First pass of the filter gradient: partial[C][nhwc_filter_slices(s)][K*K].
template <typename T>
int nhwc_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                         cudaStream_t st, int *slices_out) {
  if constexpr (!NhwcDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!nhwc_filter_ok(s)) return ROWS_DECLINED;
    NhwcFilterParams p{};
    p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
    p.pt = s.ph; p.pl = s.pw; p.SL = nhwc_filter_slices(s);
    *slices_out = p.SL;
    if (nhwc_tma_filter<T>(x, dy, partial, p, s.kh, s.sh, st) == ROWS_SERVED) return ROWS_SERVED;
    switch (s.kh * 10 + s.sh) {
      case 31: launch_filter<T, 3, 1>(x, dy, partial, p, st); break;
      case 51: launch_filter<T, 5, 1>(x, dy, partial, p, st); break;
      case 71: launch_filter<T, 7, 1>(x, dy, partial, p, st); break;
      case 32: launch_filter<T, 3, 2>(x, dy, partial, p, st); break;
      case 52: launch_filter<T, 5, 2>(x, dy, partial, p, st); break;
      case 72: launch_filter<T, 7, 2>(x, dy, partial, p, st); break;
      default: return ROWS_DECLINED;
    }
    return ROWS_SERVED;
  }
}

// dx and the first pass of the filter gradient from one pass over dy (stride 1, 3x3 / 5x5, tensors
// the copy engine can address); ROWS_DECLINED otherwise: the caller runs the two operators.
template <typename T>
int nhwc_backward(const T *x, const T *dy, const T *w, T *dx, typename Elem<T>::acc_t *partial,
                  const Shape &s, cudaStream_t st, int *slices_out) {
  if constexpr (!NhwcDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!nhwc_filter_ok(s) || s.sh != 1 || s.ph > s.kh - 1 || s.pw > s.kw - 1) return ROWS_DECLINED;
    NhwcFilterParams p{};
    p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
    p.pt = s.kh - 1 - s.ph; p.pl = s.kw - 1 - s.pw; p.SL = nhwc_filter_slices(s);
    *slices_out = p.SL;
    return nhwc_tma_backward<T>(x, dy, w, dx, partial, p, s.kh, st);
  }
}

#define DWB_NHWC_INSTANTIATE(T)                                                                   \
  template int nhwc_forward<T>(const T *, const T *, T *, const Shape &, const EpilogueArgs &,    \
                               cudaStream_t);                                                      \
  template int nhwc_backward_input<T>(const T *, const T *, T *, const Shape &, cudaStream_t);     \
  template int nhwc_backward_filter<T>(const T *, const T *, typename Elem<T>::acc_t *,            \
                                       const Shape &, cudaStream_t, int *);                        \
  template int nhwc_backward<T>(const T *, const T *, const T *, T *, typename Elem<T>::acc_t *,   \
                                const Shape &, cudaStream_t, int *);
DWB_NHWC_INSTANTIATE(float)
DWB_NHWC_INSTANTIATE(__half)
DWB_NHWC_INSTANTIATE(__nv_bfloat16)
DWB_NHWC_INSTANTIATE(double)
#undef DWB_NHWC_INSTANTIATE

}  // namespace dwb
