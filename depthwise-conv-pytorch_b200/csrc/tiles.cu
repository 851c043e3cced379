// Tiles family: variant selection and launches (kernels: tile_kernels.cuh).
#include "tile_kernels.cuh"
#include "rows_api.cuh"

#include <atomic>
#include <cstdlib>

namespace dwb {

// tiles_tma.cu: the stride-1 kernels whose input tile arrives by one tensor copy.
template <typename T>
int tiles_tma_conv(const T *in, const T *w, T *out, const TileParams &p, int K, int tw, cudaStream_t st);
template <typename T>
int tiles_tma_filter(const T *x, const T *dy, float *partial, const TileFilterParams &p, int K, int tw,
                     int bound, cudaStream_t st, int *slices_used);

namespace {

template <typename T> struct TilesDtype { static constexpr bool ok = false; };
template <> struct TilesDtype<float> { static constexpr bool ok = true; };
template <> struct TilesDtype<__half> { static constexpr bool ok = true; };
template <> struct TilesDtype<__nv_bfloat16> { static constexpr bool ok = true; };

inline bool tiles_filter_ok(const Shape &s) {
  return s.kh == s.kw && (s.kh == 3 || s.kh == 5 || s.kh == 7) && s.sh == s.sw &&
         (s.sh == 1 || s.sh == 2);
}
// Tiny maps would leave most of a tile empty: they stay on the one-thread-per-output kernels.
inline bool tiles_worth_it(int Hout, int Wout) { return Wout >= 16 && Hout >= 8; }

// 64-column tiles unless 32-column tiles waste fewer columns (narrow or just-over-64 maps).
inline int pick_tw(int Wout) {
  const int w64 = ceil_div(Wout, 64) * 64, w32 = ceil_div(Wout, 32) * 32;
  return w32 < w64 ? 32 : 64;
}

// Tuning builds can switch the tensor-copy kernels off to time the other staging forms.
inline bool tiles_tma_off() {
#ifdef DWCONV_B200_TUNING
  const char *v = getenv("DWCONV_B200_TILES_TMA");
  return v != nullptr && v[0] == '0';
#else
  return false;
#endif
}

// 16-byte staging needs every row of the map to start on a 16-byte boundary.
template <typename T> inline bool rows_aligned16(const T *base, int width) {
  constexpr int V = 16 / (int)sizeof(T);
  return width % V == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}
// Columns between the 16-byte boundary at or left of the halo and the halo: a tile's first
// output column times the stride is a multiple of the chunk, so only the padding counts.
template <typename T> inline int stage_off(int pl) {
  constexpr int V = 16 / (int)sizeof(T);
  return ((-pl) % V + V) % V;
}

template <typename T, int K, int S, int TW>
void launch_conv(const T *in, const T *w, T *out, TileParams p, cudaStream_t st) {
  constexpr int TH = TileGeo<T, K, S, TW>::TH;
  constexpr int V = 16 / (int)sizeof(T);
  p.tiles_x = ceil_div(p.Wout, TW);
  p.tiles_y = ceil_div(p.Hout, TH);
  p.ntiles = (long long)p.NC * p.tiles_x * p.tiles_y;
  // x: tile position inside a plane; y: as many planes side by side as keep about 16 CTAs per
  // SM in the grid, the rest of the planes by striding inside the kernel
  const int per_plane = p.tiles_x * p.tiles_y;
  const int cap = 148 * 16;
  int gy = cap / per_plane;
  if (gy < 1) gy = 1;
  if (gy > p.NC) gy = p.NC;
  const dim3 grid(per_plane, gy);
  {
    if (rows_aligned16(in, p.Win)) {
      // stride 1: one tensor copy per tile; else (or if the driver offers no encoder) 16-byte
      // loads and stores through registers
      if constexpr (S == 1) {
        if (!tiles_tma_off() && tiles_tma_conv<T>(in, w, out, p, K, TW, st) == ROWS_SERVED) return;
      }
      p.off = stage_off<T>(p.pl);
      tile_conv_kernel<T, K, S, TW, V><<<grid, TILE_THREADS, 0, st>>>(in, w, out, p);
      return;
    }
  }
  tile_conv_kernel<T, K, S, TW><<<grid, TILE_THREADS, 0, st>>>(in, w, out, p);
}

template <typename T, int K, int S>
void launch_conv_tw(const T *in, const T *w, T *out, const TileParams &p, cudaStream_t st) {
  if (pick_tw(p.Wout) == 32)
    launch_conv<T, K, S, 32>(in, w, out, p, st);
  else
    launch_conv<T, K, S, 64>(in, w, out, p, st);
}

// Stride-2 backward-input (polyphase kernel): p describes dy -> dx with pt / pl = k-1-padding.
template <typename T, int K, int TW>
void launch_bwd2(const T *dy, const T *w, T *dx, TileParams p, cudaStream_t st) {
  constexpr int V = 16 / (int)sizeof(T);
  constexpr int TH = Bwd2Geo<K, TW, 0>::TH;
  p.tiles_x = ceil_div(p.Wout, TW);
  p.tiles_y = ceil_div(p.Hout, TH);
  p.ntiles = (long long)p.NC * p.tiles_x * p.tiles_y;
  const int per_plane = p.tiles_x * p.tiles_y;
  const int cap = 148 * 16;
  int gy = cap / per_plane;
  if (gy < 1) gy = 1;
  if (gy > p.NC) gy = p.NC;
  const dim3 grid(per_plane, gy);
  if (rows_aligned16(dy, p.Win)) {
    // the dense dy tile starts at column floor((x0 - pl) / 2); x0 / 2 is a multiple of the chunk
    const int first = -((p.pl + (p.pl & 1)) / 2);
    p.off = (first % V + V) % V;
    tile_bwd2_kernel<T, K, TW, V><<<grid, TILE_THREADS, 0, st>>>(dy, w, dx, p);
    return;
  }
  tile_bwd2_kernel<T, K, TW, 0><<<grid, TILE_THREADS, 0, st>>>(dy, w, dx, p);
}

template <typename T, int K>
void launch_bwd2_tw(const T *dy, const T *w, T *dx, const TileParams &p, cudaStream_t st) {
  if (pick_tw(p.Wout) == 32)
    launch_bwd2<T, K, 32>(dy, w, dx, p, st);
  else
    launch_bwd2<T, K, 64>(dy, w, dx, p, st);
}

template <typename T>
int conv_dispatch(const T *in, const T *w, T *out, const TileParams &p, int K, int S, cudaStream_t st) {
  switch (K * 10 + S) {
    case 31: launch_conv_tw<T, 3, 1>(in, w, out, p, st); return ROWS_SERVED;
    case 51: launch_conv_tw<T, 5, 1>(in, w, out, p, st); return ROWS_SERVED;
    case 71: launch_conv_tw<T, 7, 1>(in, w, out, p, st); return ROWS_SERVED;
    case 32: launch_conv_tw<T, 3, 2>(in, w, out, p, st); return ROWS_SERVED;
    case 52: launch_conv_tw<T, 5, 2>(in, w, out, p, st); return ROWS_SERVED;
    case 72: launch_conv_tw<T, 7, 2>(in, w, out, p, st); return ROWS_SERVED;
    default: return ROWS_DECLINED;
  }
}

template <typename T, int K, int S, int TW>
int launch_filter(const T *x, const T *dy, float *partial, TileFilterParams p, int bound, cudaStream_t st) {
  constexpr int TH = TileGeo<T, K, S, TW>::TH;
  p.tiles_x = ceil_div(p.Wo, TW);
  p.tiles_y = ceil_div(p.Ho, TH);
  constexpr int V = 16 / (int)sizeof(T);
  using GV = TileGeo<T, K, S, TW, V>;
  // the wider staged rows of the 16-byte form must still fit the static shared memory of a CTA
  constexpr bool fits =
      (GV::IH * GV::PITCH + GV::TH * TW + TILE_THREADS / 32 * K * K) * sizeof(float) <= 48 * 1024;
  if constexpr (S == 1) {
    if (rows_aligned16(x, p.W) && rows_aligned16(dy, p.Wo) && !tiles_tma_off()) {
      int used = 0;
      if (tiles_tma_filter<T>(x, dy, partial, p, K, TW, bound, st, &used) == ROWS_SERVED) return used;
    }
  }
  if constexpr (fits) {
    if (rows_aligned16(x, p.W) && rows_aligned16(dy, p.Wo)) {
      p.off = stage_off<T>(p.pl);
      p.SL = filter_slices_for<tile_filter_kernel<T, K, S, TW, V>>(p, bound);
      tile_filter_kernel<T, K, S, TW, V><<<p.C * p.SL, TILE_THREADS, 0, st>>>(x, dy, partial, p);
      return p.SL;
    }
  }
  p.SL = filter_slices_for<tile_filter_kernel<T, K, S, TW, 0>>(p, bound);
  tile_filter_kernel<T, K, S, TW><<<p.C * p.SL, TILE_THREADS, 0, st>>>(x, dy, partial, p);
  return p.SL;
}

template <typename T, int K, int S>
int launch_filter_tw(const T *x, const T *dy, float *partial, const TileFilterParams &p, int bound,
                     cudaStream_t st) {
  if (pick_tw(p.Wo) == 32) return launch_filter<T, K, S, 32>(x, dy, partial, p, bound, st);
  return launch_filter<T, K, S, 64>(x, dy, partial, p, bound, st);
}

}  // namespace

template <typename T>
int tiles_forward(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep, cudaStream_t st) {
  if constexpr (!TilesDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!tiles_filter_ok(s) || !tiles_worth_it(s.Ho, s.Wo)) return ROWS_DECLINED;
    TileParams p{};
    p.NC = s.N * s.C; p.C = s.C;
    p.Hin = s.H; p.Win = s.W; p.Hout = s.Ho; p.Wout = s.Wo;
    p.pt = s.ph; p.pl = s.pw; p.flip = 0;
    p.ep = ep;
    return conv_dispatch<T>(x, w, y, p, s.kh, s.sh, st);
  }
}

// The transposed operation is the stride-1 correlation of dy, up-sampled by the forward stride
// and padded by k-1-p, with the flipped filter (torch_dwconv/dwconv.py:39-44,57-64).
template <typename T>
int tiles_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st) {
  if constexpr (!TilesDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!tiles_filter_ok(s) || s.ph > s.kh - 1 || s.pw > s.kw - 1 || !tiles_worth_it(s.H, s.W))
      return ROWS_DECLINED;
    TileParams p{};
    p.NC = s.N * s.C; p.C = s.C;
    p.Hin = s.Ho; p.Win = s.Wo; p.Hout = s.H; p.Wout = s.W;
    p.pt = s.kh - 1 - s.ph; p.pl = s.kw - 1 - s.pw; p.flip = 1;
    if (s.sh == 1) return conv_dispatch<T>(dy, w, dx, p, s.kh, 1, st);
    switch (s.kh) {
      case 3: launch_bwd2_tw<T, 3>(dy, w, dx, p, st); return ROWS_SERVED;
      case 5: launch_bwd2_tw<T, 5>(dy, w, dx, p, st); return ROWS_SERVED;
      case 7: launch_bwd2_tw<T, 7>(dy, w, dx, p, st); return ROWS_SERVED;
      default: return ROWS_DECLINED;
    }
  }
}

int tiles_filter_slices(const Shape &s) {
  if (!tiles_filter_ok(s) || !tiles_worth_it(s.Ho, s.Wo)) return 0;
  const int TW = pick_tw(s.Wo), TH = TILE_THREADS / TW * TILE_R;
  const long long total = (long long)s.N * ceil_div(s.Wo, TW) * ceil_div(s.Ho, TH);
  long long S = 8 * 148 / s.C;  // no kernel of the family keeps more than 8 CTAs on an SM
  if (S > total) S = total;
  return S < 1 ? 1 : (int)S;
}

// First pass of the filter gradient: partial[C][*slices_used][K*K], *slices_used <= slices (the
// bound the caller sized the workspace for, tiles_filter_slices).
template <typename T>
int tiles_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                          int slices, cudaStream_t st, int *slices_used) {
  if constexpr (!TilesDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (!tiles_filter_ok(s) || !tiles_worth_it(s.Ho, s.Wo) || slices < 1) return ROWS_DECLINED;
    TileFilterParams p{};
    p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
    p.pt = s.ph; p.pl = s.pw;
    int used = 0;
    switch (s.kh * 10 + s.sh) {
      case 31: used = launch_filter_tw<T, 3, 1>(x, dy, partial, p, slices, st); break;
      case 51: used = launch_filter_tw<T, 5, 1>(x, dy, partial, p, slices, st); break;
      case 71: used = launch_filter_tw<T, 7, 1>(x, dy, partial, p, slices, st); break;
      case 32: used = launch_filter_tw<T, 3, 2>(x, dy, partial, p, slices, st); break;
      case 52: used = launch_filter_tw<T, 5, 2>(x, dy, partial, p, slices, st); break;
      case 72: used = launch_filter_tw<T, 7, 2>(x, dy, partial, p, slices, st); break;
      default: return ROWS_DECLINED;
    }
    *slices_used = used;
    return ROWS_SERVED;
  }
}

#define DWB_TILES_INSTANTIATE(T)                                                              \
  template int tiles_forward<T>(const T *, const T *, T *, const Shape &, const EpilogueArgs &, \
                                cudaStream_t);                                                  \
  template int tiles_backward_input<T>(const T *, const T *, T *, const Shape &, cudaStream_t); \
  template int tiles_backward_filter<T>(const T *, const T *, typename Elem<T>::acc_t *,        \
                                        const Shape &, int, cudaStream_t, int *);
DWB_TILES_INSTANTIATE(float)
DWB_TILES_INSTANTIATE(__half)
DWB_TILES_INSTANTIATE(__nv_bfloat16)
DWB_TILES_INSTANTIATE(double)
#undef DWB_TILES_INSTANTIATE

}  // namespace dwb
