// Tiles family, tensor-copy staged kernels: tensor-map encoding and launches
// (kernels: tile_tma_kernels.cuh).
#include "tile_tma_kernels.cuh"
#include "tensor_map.cuh"

#include <atomic>

namespace dwb {

namespace {

__device__ int g_tiles_tma_error_flag;

int *error_flag_ptr() {
  static std::atomic<int *> cached{nullptr};
  int *p = cached.load(std::memory_order_relaxed);
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void **)&p, g_tiles_tma_error_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached.store(p, std::memory_order_relaxed);
  }
  return p;
}

// The maps [planes][H][W] as a (W, H, planes) tensor read in boxes of (bw, bh, 1) elements.
template <typename T>
bool encode_planes(CUtensorMap *map, const T *base, int W, int H, int planes, int bw, int bh) {
  const cuuint64_t dims[3] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)planes};
  const cuuint64_t strides[2] = {(cuuint64_t)W * sizeof(T), (cuuint64_t)W * H * sizeof(T)};
  const cuuint32_t box[3] = {(cuuint32_t)bw, (cuuint32_t)bh, 1u};
  return encode_tensor_map<T>(map, base, 3, dims, strides, box);
}

template <typename T, int K, int TW>
int launch(const T *in, const T *w, T *out, TileParams p, cudaStream_t st) {
  using G = TileTmaGeo<T, K, TW>;
  static_assert(2 * G::STAGE_BYTES + 64 <= 48 * 1024, "two stages must fit static shared memory");
  static_assert(G::BW <= 256 && G::IH <= 256, "a box dimension is at most 256 elements");
  int *flag = error_flag_ptr();
  if (flag == nullptr) return ROWS_DECLINED;
  p.off = ((-p.pl) % G::V + G::V) % G::V;
  if ((p.pl + p.off) % G::V != 0) return ROWS_DECLINED;  // the box must start on a 16-byte boundary
  alignas(64) CUtensorMap map;
  if (!encode_planes<T>(&map, in, p.Win, p.Hin, p.NC, G::BW, G::IH)) return ROWS_DECLINED;
  p.tiles_x = ceil_div(p.Wout, TW);
  p.tiles_y = ceil_div(p.Hout, G::TH);
  p.ntiles = (long long)p.NC * p.tiles_x * p.tiles_y;
  const int per_plane = p.tiles_x * p.tiles_y;
  // as many CTAs as the device holds at once (the kernel's launch bounds); each walks its share
  // of the planes, its two stages overlapping copy and arithmetic
  const int gy = walk_groups(148 * (K == 3 ? 6 : (K == 5 ? 4 : 3)), per_plane, p.NC);
  tile_tma_conv_kernel<T, K, TW><<<dim3(per_plane, gy), TILE_THREADS, 0, st>>>(map, w, out, p, flag);
  return ROWS_SERVED;
}

template <typename T, int K>
int launch_tw(const T *in, const T *w, T *out, const TileParams &p, int tw, cudaStream_t st) {
  return tw == 32 ? launch<T, K, 32>(in, w, out, p, st) : launch<T, K, 64>(in, w, out, p, st);
}

template <typename T, int K, int TW>
int launch_filter(const T *x, const T *dy, float *partial, TileFilterParams p, int bound, cudaStream_t st,
                  int *used) {
  using G = TileTmaGeo<T, K, TW>;
  int *flag = error_flag_ptr();
  if (flag == nullptr) return ROWS_DECLINED;
  p.off = ((-p.pl) % G::V + G::V) % G::V;
  if ((p.pl + p.off) % G::V != 0) return ROWS_DECLINED;
  alignas(64) CUtensorMap x_map, dy_map;
  if (!encode_planes<T>(&x_map, x, p.W, p.H, p.N * p.C, G::BW, G::IH)) return ROWS_DECLINED;
  if (!encode_planes<T>(&dy_map, dy, p.Wo, p.Ho, p.N * p.C, TW, G::TH)) return ROWS_DECLINED;
  p.tiles_x = ceil_div(p.Wo, TW);
  p.tiles_y = ceil_div(p.Ho, G::TH);
  p.SL = filter_slices_for<tile_tma_filter_kernel<T, K, TW>>(p, bound);
  tile_tma_filter_kernel<T, K, TW><<<p.C * p.SL, TILE_THREADS, 0, st>>>(x_map, dy_map, partial, p, flag);
  *used = p.SL;
  return ROWS_SERVED;
}

}  // namespace

// First pass of the stride-1 filter gradient staged by tensor copies (x and dy rows on 16-byte
// boundaries); `bound` is the slice count the workspace was sized for, *slices_used what was
// launched.
template <typename T>
int tiles_tma_filter(const T *x, const T *dy, float *partial, const TileFilterParams &p, int K, int tw,
                     int bound, cudaStream_t st, int *slices_used) {
  constexpr int V = 16 / (int)sizeof(T);
  if (p.W % V != 0 || p.Wo % V != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(dy) & 15) != 0)
    return ROWS_DECLINED;
  if ((long long)p.N * p.C > (1 << 30) || (long long)p.W * p.H * (long long)sizeof(T) >= (1ll << 40))
    return ROWS_DECLINED;
  switch (K * 100 + tw) {
    case 332: return launch_filter<T, 3, 32>(x, dy, partial, p, bound, st, slices_used);
    case 364: return launch_filter<T, 3, 64>(x, dy, partial, p, bound, st, slices_used);
    case 532: return launch_filter<T, 5, 32>(x, dy, partial, p, bound, st, slices_used);
    case 564: return launch_filter<T, 5, 64>(x, dy, partial, p, bound, st, slices_used);
    case 732: return launch_filter<T, 7, 32>(x, dy, partial, p, bound, st, slices_used);
    case 764: return launch_filter<T, 7, 64>(x, dy, partial, p, bound, st, slices_used);
    default: return ROWS_DECLINED;
  }
}

template int tiles_tma_filter<float>(const float *, const float *, float *, const TileFilterParams &, int,
                                     int, int, cudaStream_t, int *);
template int tiles_tma_filter<__half>(const __half *, const __half *, float *, const TileFilterParams &,
                                      int, int, int, cudaStream_t, int *);
template int tiles_tma_filter<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, float *,
                                             const TileFilterParams &, int, int, int, cudaStream_t, int *);

// Stride-1 correlation of `in` (rows on 16-byte boundaries) staged by tensor copies; `tw` is
// the tile width the caller chose (32 or 64).  ROWS_DECLINED when this form cannot run (no
// encoder in the driver, a geometry outside what a box can describe).
template <typename T>
int tiles_tma_conv(const T *in, const T *w, T *out, const TileParams &p, int K, int tw, cudaStream_t st) {
  constexpr int V = 16 / (int)sizeof(T);
  if (p.Win % V != 0 || (reinterpret_cast<uintptr_t>(in) & 15) != 0) return ROWS_DECLINED;
  if (p.NC > (1 << 30) || (long long)p.Win * p.Hin * (long long)sizeof(T) >= (1ll << 40)) return ROWS_DECLINED;
  switch (K) {
    case 3: return launch_tw<T, 3>(in, w, out, p, tw, st);
    case 5: return launch_tw<T, 5>(in, w, out, p, tw, st);
    case 7: return launch_tw<T, 7>(in, w, out, p, tw, st);
    default: return ROWS_DECLINED;
  }
}

template int tiles_tma_conv<float>(const float *, const float *, float *, const TileParams &, int, int,
                                   cudaStream_t);
template int tiles_tma_conv<__half>(const __half *, const __half *, __half *, const TileParams &, int, int,
                                    cudaStream_t);
template int tiles_tma_conv<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *,
                                           const TileParams &, int, int, cudaStream_t);

// Reads and clears this translation unit's error flag (bit 0: a bounded wait expired).
int tiles_tma_take_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tiles_tma_error_flag, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (v != 0) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_tiles_tma_error_flag, &zero, sizeof(int));
  }
  return v;
}

}  // namespace dwb
