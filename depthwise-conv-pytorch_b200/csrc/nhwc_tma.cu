// Channels-last kernels staged by tensor copies: tensor-map encoding and launches
// (kernels: nhwc_tma_kernels.cuh).
#include "nhwc_tma_kernels.cuh"
#include "tensor_map.cuh"

#include <atomic>

namespace dwb {

namespace {

__device__ int g_nhwc_tma_error_flag;

int *error_flag_ptr() {
  static std::atomic<int *> cached{nullptr};
  int *p = cached.load(std::memory_order_relaxed);
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void **)&p, g_nhwc_tma_error_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached.store(p, std::memory_order_relaxed);
  }
  return p;
}

// [N][H][W][C] as a (C, W, H, N) tensor read in boxes of (32, bw, bh, 1) elements.
template <typename T>
bool encode_nhwc(CUtensorMap *map, const T *base, int C, int W, int H, int N, int bw, int bh) {
  const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  const cuuint64_t strides[3] = {(cuuint64_t)C * sizeof(T), (cuuint64_t)W * C * sizeof(T),
                                 (cuuint64_t)H * W * C * sizeof(T)};
  const cuuint32_t box[4] = {(cuuint32_t)NHWC_CB, (cuuint32_t)bw, (cuuint32_t)bh, 1u};
  return encode_tensor_map<T>(map, base, 4, dims, strides, box);
}

template <typename T> bool tensor_ok(const T *base, int C, int W, int H) {
  constexpr int V = 16 / (int)sizeof(T);
  return C % V == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0 &&
         (long long)C * W * H * (long long)sizeof(T) < (1ll << 40);
}

// Once per kernel (the kernel is a template ARGUMENT: kernels of one signature share a function
// type, and a cache per type would be shared among them): allow its dynamic shared memory, and
// ask how many CTAs the device holds.
template <auto kernel> int prepare(int threads, int smem_bytes) {
  static std::atomic<int> cached{0};
  int v = cached.load(std::memory_order_acquire);
  if (v == 0) {
    int per_sm = 0, dev = 0, sms = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem_bytes) != cudaSuccess ||
        cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm < 1) {
      (void)cudaGetLastError();
      return -1;
    }
    v = per_sm * sms;
    cached.store(v, std::memory_order_release);
  }
  return v;
}

template <typename T, int K, int S>
int launch_conv(const T *in, const T *w, T *out, NhwcParams p, cudaStream_t st) {
  using G = NhwcGeo<K, S>;
  using TG = NhwcTmaGeo<T, K, S>;
  static_assert(G::IW <= 256 && G::IH <= 256, "a box dimension is at most 256 elements");
  int *flag = error_flag_ptr();
  if (flag == nullptr) return ROWS_DECLINED;
  const int resident = prepare<nhwc_tma_conv_kernel<T, K, S>>(G::THREADS, TG::SMEM_BYTES);
  if (resident < 1) return ROWS_DECLINED;
  alignas(64) CUtensorMap map;
  if (!encode_nhwc<T>(&map, in, p.C, p.Win, p.Hin, p.N, G::IW, G::IH)) return ROWS_DECLINED;
  p.tiles_x = ceil_div(p.Wout, G::TW);
  p.tiles_y = ceil_div(p.Hout, G::R);
  p.cblocks = ceil_div(p.C, NHWC_CB);
  const long long per_img = (long long)p.tiles_x * p.tiles_y * p.cblocks;
  if (per_img > (1ll << 30)) return ROWS_DECLINED;
  p.ntiles = per_img * p.N;
  const int gy = walk_groups(resident, per_img, p.N);  // each CTA walks its share of the images
  nhwc_tma_conv_kernel<T, K, S><<<dim3((unsigned)per_img, (unsigned)gy), G::THREADS, TG::SMEM_BYTES, st>>>(
      map, w, out, p, flag);
  return ROWS_SERVED;
}

template <typename T, int K>
int launch_bwd2(const T *dy, const T *w, T *dx, NhwcParams p, cudaStream_t st) {
  using G = NhwcBwd2Geo<K>;
  int *flag = error_flag_ptr();
  if (flag == nullptr) return ROWS_DECLINED;
  const int resident = prepare<nhwc_tma_bwd2_kernel<T, K>>(G::THREADS, 0);
  if (resident < 1) return ROWS_DECLINED;
  alignas(64) CUtensorMap map;
  if (!encode_nhwc<T>(&map, dy, p.C, p.Win, p.Hin, p.N, G::IW, G::ND)) return ROWS_DECLINED;
  p.tiles_x = ceil_div(p.Wout, G::TW);
  p.tiles_y = ceil_div(p.Hout, G::R);
  p.cblocks = ceil_div(p.C, NHWC_CB);
  const long long per_img = (long long)p.tiles_x * p.tiles_y * p.cblocks;
  if (per_img > (1ll << 30)) return ROWS_DECLINED;
  p.ntiles = per_img * p.N;
  const int gy = walk_groups(resident, per_img, p.N);
  nhwc_tma_bwd2_kernel<T, K><<<dim3((unsigned)per_img, (unsigned)gy), G::THREADS, 0, st>>>(map, w, dx, p, flag);
  return ROWS_SERVED;
}

template <typename T, int K, int S>
int launch_filter(const T *x, const T *dy, float *partial, NhwcFilterParams p, cudaStream_t st) {
  using G = NhwcGeo<K, S, true>;
  using TG = NhwcTmaGeo<T, K, S, true>;
  int *flag = error_flag_ptr();
  if (flag == nullptr) return ROWS_DECLINED;
  if (prepare<nhwc_tma_filter_kernel<T, K, S>>(G::THREADS, TG::SMEM_BYTES) < 1) return ROWS_DECLINED;
  alignas(64) CUtensorMap x_map, dy_map;
  if (!encode_nhwc<T>(&x_map, x, p.C, p.W, p.H, p.N, G::IW, G::IH)) return ROWS_DECLINED;
  if (!encode_nhwc<T>(&dy_map, dy, p.C, p.Wo, p.Ho, p.N, G::TW, G::R)) return ROWS_DECLINED;
  p.tiles_x = ceil_div(p.Wo, G::TW);
  p.tiles_y = ceil_div(p.Ho, G::R);
  p.cblocks = ceil_div(p.C, NHWC_CB);
  nhwc_tma_filter_kernel<T, K, S><<<p.cblocks * p.SL, G::THREADS, TG::SMEM_BYTES, st>>>(x_map, dy_map, partial,
                                                                                       p, flag);
  return ROWS_SERVED;
}

template <typename T, int K>
int launch_backward(const T *x, const T *dy, const T *w, T *dx, float *partial, NhwcFilterParams p,
                    cudaStream_t st) {
  using G = NhwcGeo<K, 1, true>;
  using TG = NhwcTmaGeo<T, K, 1, true>;
  int *flag = error_flag_ptr();
  if (flag == nullptr) return ROWS_DECLINED;
  if (prepare<nhwc_tma_backward_kernel<T, K>>(G::THREADS, TG::SMEM_BYTES) < 1) return ROWS_DECLINED;
  alignas(64) CUtensorMap dy_map, x_map;
  if (!encode_nhwc<T>(&dy_map, dy, p.C, p.Wo, p.Ho, p.N, G::IW, G::IH)) return ROWS_DECLINED;
  if (!encode_nhwc<T>(&x_map, x, p.C, p.W, p.H, p.N, G::TW, G::R)) return ROWS_DECLINED;
  p.tiles_x = ceil_div(p.W, G::TW);  // tiles of the x / dx map
  p.tiles_y = ceil_div(p.H, G::R);
  p.cblocks = ceil_div(p.C, NHWC_CB);
  nhwc_tma_backward_kernel<T, K><<<p.cblocks * p.SL, G::THREADS, TG::SMEM_BYTES, st>>>(dy_map, x_map, w, dx,
                                                                                       partial, p, flag);
  return ROWS_SERVED;
}

}  // namespace

// dx and the first pass of the filter gradient at stride 1 from one pass over dy; p: H x W = x,
// Ho x Wo = dy, pt / pl = k-1-padding, SL slices per channel block.
template <typename T>
int nhwc_tma_backward(const T *x, const T *dy, const T *w, T *dx, float *partial, const NhwcFilterParams &p,
                      int K, cudaStream_t st) {
  if (!tensor_ok(x, p.C, p.W, p.H) || !tensor_ok(dy, p.C, p.Wo, p.Ho) ||
      (reinterpret_cast<uintptr_t>(dx) & 15) != 0)
    return ROWS_DECLINED;
  switch (K) {
    case 3: return launch_backward<T, 3>(x, dy, w, dx, partial, p, st);
    case 5: return launch_backward<T, 5>(x, dy, w, dx, partial, p, st);
    default: return ROWS_DECLINED;
  }
}

// Forward (stride 1 or 2) or stride-1 backward-input on channels-last maps; ROWS_DECLINED when
// the tensors do not meet the copy engine's rules or the driver offers no encoder.
template <typename T>
int nhwc_tma_conv(const T *in, const T *w, T *out, const NhwcParams &p, int K, int S, cudaStream_t st) {
  if (!tensor_ok(in, p.C, p.Win, p.Hin)) return ROWS_DECLINED;
  switch (K * 10 + S) {
    case 31: return launch_conv<T, 3, 1>(in, w, out, p, st);
    case 51: return launch_conv<T, 5, 1>(in, w, out, p, st);
    case 71: return launch_conv<T, 7, 1>(in, w, out, p, st);
    case 32: return launch_conv<T, 3, 2>(in, w, out, p, st);
    case 52: return launch_conv<T, 5, 2>(in, w, out, p, st);
    case 72: return launch_conv<T, 7, 2>(in, w, out, p, st);
    default: return ROWS_DECLINED;
  }
}

// Stride-2 backward-input (polyphase): p describes dy -> dx with pt / pl = k-1-padding.
template <typename T>
int nhwc_tma_bwd2(const T *dy, const T *w, T *dx, const NhwcParams &p, int K, cudaStream_t st) {
  if (!tensor_ok(dy, p.C, p.Win, p.Hin)) return ROWS_DECLINED;
  switch (K) {
    case 3: return launch_bwd2<T, 3>(dy, w, dx, p, st);
    case 5: return launch_bwd2<T, 5>(dy, w, dx, p, st);
    case 7: return launch_bwd2<T, 7>(dy, w, dx, p, st);
    default: return ROWS_DECLINED;
  }
}

// First pass of the filter gradient with p.SL slices per channel block.
template <typename T>
int nhwc_tma_filter(const T *x, const T *dy, float *partial, const NhwcFilterParams &p, int K, int S,
                    cudaStream_t st) {
  if (!tensor_ok(x, p.C, p.W, p.H) || !tensor_ok(dy, p.C, p.Wo, p.Ho)) return ROWS_DECLINED;
  switch (K * 10 + S) {
    case 31: return launch_filter<T, 3, 1>(x, dy, partial, p, st);
    case 51: return launch_filter<T, 5, 1>(x, dy, partial, p, st);
    case 71: return launch_filter<T, 7, 1>(x, dy, partial, p, st);
    case 32: return launch_filter<T, 3, 2>(x, dy, partial, p, st);
    case 52: return launch_filter<T, 5, 2>(x, dy, partial, p, st);
    case 72: return launch_filter<T, 7, 2>(x, dy, partial, p, st);
    default: return ROWS_DECLINED;
  }
}

#define DWB_NHWC_TMA_INSTANTIATE(T)                                                               \
  template int nhwc_tma_conv<T>(const T *, const T *, T *, const NhwcParams &, int, int, cudaStream_t); \
  template int nhwc_tma_backward<T>(const T *, const T *, const T *, T *, float *, const NhwcFilterParams &, \
                                    int, cudaStream_t);                                                  \
  template int nhwc_tma_bwd2<T>(const T *, const T *, T *, const NhwcParams &, int, cudaStream_t);      \
  template int nhwc_tma_filter<T>(const T *, const T *, float *, const NhwcFilterParams &, int, int,    \
                                  cudaStream_t);
DWB_NHWC_TMA_INSTANTIATE(float)
DWB_NHWC_TMA_INSTANTIATE(__half)
DWB_NHWC_TMA_INSTANTIATE(__nv_bfloat16)
#undef DWB_NHWC_TMA_INSTANTIATE

// Reads and clears this translation unit's error flag (bit 0 conv kernels, bit 1 filter kernel).
int nhwc_tma_take_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_nhwc_tma_error_flag, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (v != 0) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_nhwc_tma_error_flag, &zero, sizeof(int));
  }
  return v;
}

}  // namespace dwb
