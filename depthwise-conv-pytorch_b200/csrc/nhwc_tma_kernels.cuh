// Channels-last kernels whose input tiles arrive by tensor copies (TMA).
//
// In NHWC the tile a CTA works on, R rows x TW columns of outputs for 32 channels, needs the box
// (32 channels, IW columns, IH rows) of one image: a box of the 4-d tensor (channel, column, row,
// image).  One cp.async.bulk.tensor.4d brings it into shared memory as [row][column][channel],
// exactly the layout the arithmetic of nhwc_kernels.cuh reads (lane = channel), and fills
// whatever lies outside the tensor with zeros: the padding on all four sides and the channels
// beyond C.  The innermost coordinate is the channel block (a multiple of 32 elements), so the
// 16-byte rule of the copy engine never meets the halo.  Needs C a multiple of 4 fp32 / 8 fp16
// elements (strides in multiples of 16 bytes) and a 16-byte aligned base; other tensors use
// nhwc_kernels.cuh.
//
// A CTA keeps its tile position and channel block (its taps are loaded once) and walks the
// images; two stages, thread 0 asks for image i+2's box as soon as all threads have read image
// i's.  Same thread-to-output mapping and order of multiply-adds as nhwc_conv_kernel: same bits.
// Waits are bounded; on expiry the thread raises the error flag and runs to the end.
#pragma once

#include <cuda.h>

#include "nhwc_kernels.cuh"
#include "rows_engine.cuh"  // mbarrier wrappers, bounded wait

namespace dwb {

template <typename T, int K, int S, bool FILTER = false>
struct NhwcTmaGeo {
  using G = NhwcGeo<K, S, FILTER>;
  static constexpr int X_BYTES = G::IH * G::IW * NHWC_CB * (int)sizeof(T);
  static constexpr int DY_BYTES = FILTER ? G::R * G::TW * NHWC_CB * (int)sizeof(T) : 0;
  static constexpr int X_SLOT = (X_BYTES + 127) / 128 * 128;
  static constexpr int STAGE_BYTES = X_SLOT + (DY_BYTES + 127) / 128 * 128;
  static constexpr int SMEM_BYTES = 2 * STAGE_BYTES + 128;  // + the two barriers
};

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            int c3, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// Forward (any stride the family has) and stride-1 backward-input (flip).  Grid: x = (tile row,
// tile column, channel block), channel blocks innermost; y = first image.
// (Two CTAs per SM as the register target at stride 1, 512 threads: left to itself the compiler
// aims at four and spills.)
template <typename T, int K, int S>
__global__ void __launch_bounds__(NhwcGeo<K, S>::THREADS, (S == 1 && K < 7) ? 2 : 1)
nhwc_tma_conv_kernel(const __grid_constant__ CUtensorMap in_map, const T *__restrict__ w,
                     T *__restrict__ out, const NhwcParams p, int *error_flag) {
  using G = NhwcGeo<K, S>;
  using TG = NhwcTmaGeo<T, K, S>;
  constexpr int KK = K * K;
  extern __shared__ __align__(128) unsigned char nhwc_smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(nhwc_smem + 2 * TG::STAGE_BYTES);
  const int lane = threadIdx.x & 31;
  const int col = threadIdx.x >> 5;  // output column inside the tile
  int rest = blockIdx.x;
  const int cb = rest % p.cblocks;
  rest /= p.cblocks;
  const int ty = rest / p.tiles_x, tx = rest - ty * p.tiles_x;
  const int y0 = ty * G::R, x0 = tx * G::TW, c0 = cb * NHWC_CB;
  const int c = c0 + lane;
  const int bx = x0 * S - p.pl, by = y0 * S - p.pt;  // first pixel of the box
  const int step = gridDim.y;
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  int asked0 = 0, asked1 = 0, landed0 = 0, landed1 = 0;  // thread 0: copies asked for / seen complete
  if (threadIdx.x == 0) {
    if ((int)blockIdx.y < p.N) {
      mbar_arrive_expect_tx(&full[0], TG::X_BYTES);
      tma_load_4d(nhwc_smem, &in_map, c0, bx, by, blockIdx.y, &full[0]);
      asked0 = 1;
    }
    if ((int)blockIdx.y + step < p.N) {
      mbar_arrive_expect_tx(&full[1], TG::X_BYTES);
      tma_load_4d(nhwc_smem + TG::STAGE_BYTES, &in_map, c0, bx, by, blockIdx.y + step, &full[1]);
      asked1 = 1;
    }
  }
  // the CTA's channels do not change: taps and epilogue coefficients are loaded once
  // (taps and staged values stay in the storage type: fma_mix multiplies them as they are)
  T tap[K][K];
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx)
      tap[ky][kx] = c < p.C ? __ldg(w + (size_t)c * KK + (p.flip ? KK - 1 - (ky * K + kx) : ky * K + kx))
                            : Elem<T>::from_acc(0.f);
  float sc = 1.f, bi = 0.f;
  if (p.ep.on && c < p.C) epilogue_coeffs<T>(p.ep, c, sc, bi);
  bool gave_up = false;
  int it = 0;
  for (int n = blockIdx.y; n < p.N; n += step, ++it) {
    const int s = it & 1;
    if (!gave_up) {
      if (mbar_wait_bounded(&full[s], (it >> 1) & 1)) {
        landed0 += 1 - s;
        landed1 += s;
      } else {
        gave_up = true;
        atomicOr(error_flag, 1);
      }
    }
    const unsigned char *stage = nhwc_smem + s * TG::STAGE_BYTES;
    float acc[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) acc[o] = 0.f;
#pragma unroll
    for (int ir = 0; ir < G::IH; ++ir) {
      T v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx)
        v[kx] = reinterpret_cast<const T *>(stage)[(ir * G::IW + col * S + kx) * NHWC_CB + lane];
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        const int ky = ir - o * S;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc[o] = fma_mix(v[kx], tap[ky][kx], acc[o]);
        }
      }
    }
    if (p.ep.on) {
#pragma unroll
      for (int o = 0; o < G::R; ++o) acc[o] = apply_epilogue<float>(acc[o], sc, bi, p.ep.act);
    }
    const int ox = x0 + col;
    if (ox < p.Wout && c < p.C) {
      T *op = out + (((size_t)n * p.Hout + y0) * p.Wout + ox) * p.C + c;
      const size_t row_stride = (size_t)p.Wout * p.C;
      const int rows = p.Hout - y0;
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        if (o < rows) *op = Elem<T>::from_acc(acc[o]);
        op += row_stride;
      }
    }
    __syncthreads();  // every thread has read stage s: it may be refilled
    if (threadIdx.x == 0 && !gave_up) {
      const int next = n + 2 * step;
      if (next < p.N) {
        mbar_arrive_expect_tx(&full[s], TG::X_BYTES);
        tma_load_4d(nhwc_smem + s * TG::STAGE_BYTES, &in_map, c0, bx, by, next, &full[s]);
        asked0 += 1 - s;
        asked1 += s;
      }
    }
  }
  // copies that may still be on their way after a thread gave up: another bounded wait each
  if (threadIdx.x == 0 && gave_up) {
    while (landed0 < asked0 && mbar_wait_bounded(&full[0], landed0 & 1)) ++landed0;
    while (landed1 < asked1 && mbar_wait_bounded(&full[1], landed1 & 1)) ++landed1;
  }
}

// Backward-input at stride 2, polyphase (the arithmetic of tile_bwd2_kernel in tile_kernels.cuh,
// with lane = channel): dy is fetched as it is (a dense box of (32 channels, TW/2 + ceil(K/2)
// columns, ND rows)), and only the products that meet data are issued, in ky-major / kx-minor
// order.  The output column, and with it the parity of the kx that meet data, is the same for all
// lanes of a warp.  A tile is 8 rows x 16 columns of dx; staged row d is dy row
// floor((y0 - pt) / 2) + d, and ky = 2d - P - o for output row y0 + o (P = pt & 1).
template <int K> struct NhwcBwd2Geo {
  static constexpr int R = 8, TW = 16;
  static constexpr int THREADS = NHWC_CB * TW;
  static constexpr int KH = (K + 1) / 2;
  static constexpr int ND = (K + R - 1) / 2 + 1;  // dy rows under a tile
  static constexpr int IW = TW / 2 + KH;          // dy columns under a tile
};

template <typename T, int K, bool PODD>
__device__ __forceinline__ void nhwc_bwd2_rows(const unsigned char *stage, int col0, int lane,
                                               const T (&tsel)[K][(K + 1) / 2], float (&acc)[8]) {
  using G = NhwcBwd2Geo<K>;
  constexpr int P = PODD ? 1 : 0;
#pragma unroll
  for (int d = 0; d < G::ND; ++d) {
    T v[G::KH];
#pragma unroll
    for (int j = 0; j < G::KH; ++j)
      v[j] = reinterpret_cast<const T *>(stage)[(d * G::IW + col0 + j) * NHWC_CB + lane];
#pragma unroll
    for (int o = 0; o < G::R; ++o) {
      const int ky = 2 * d - P - o;
      if (ky >= 0 && ky < K) {
#pragma unroll
        for (int j = 0; j < G::KH; ++j) acc[o] = fma_mix(v[j], tsel[ky][j], acc[o]);
      }
    }
  }
}

// p: Hin x Win = dy, Hout x Wout = dx, pt / pl = k-1-padding.
template <typename T, int K>
__global__ void __launch_bounds__(NhwcBwd2Geo<K>::THREADS, 2)
nhwc_tma_bwd2_kernel(const __grid_constant__ CUtensorMap dy_map, const T *__restrict__ w,
                     T *__restrict__ out, const NhwcParams p, int *error_flag) {
  using G = NhwcBwd2Geo<K>;
  constexpr int KK = K * K;
  constexpr int BOX_BYTES = G::ND * G::IW * NHWC_CB * (int)sizeof(T);
  constexpr int STAGE_BYTES = (BOX_BYTES + 127) / 128 * 128;
  static_assert(2 * STAGE_BYTES + 64 <= 48 * 1024, "two stages must fit static shared memory");
  __shared__ __align__(128) unsigned char stages[2][STAGE_BYTES];
  __shared__ uint64_t full[2];
  const int lane = threadIdx.x & 31;
  const int col = threadIdx.x >> 5;  // output column inside the tile
  int rest = blockIdx.x;
  const int cb = rest % p.cblocks;
  rest /= p.cblocks;
  const int ty = rest / p.tiles_x, tx = rest - ty * p.tiles_x;
  const int y0 = ty * G::R, x0 = tx * G::TW, c0 = cb * NHWC_CB;  // y0, x0 even
  const int c = c0 + lane;
  const int px = p.pl & 1;
  const int qx = (px + col) & 1;  // parity of the kx that meet data under this column
  const int col0 = (col + qx + px) >> 1;
  const int gy0 = (y0 - p.pt - (p.pt & 1)) / 2, gx0 = (x0 - p.pl - px) / 2;  // floor((y0-pt)/2), ...
  const int step = gridDim.y;
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  int asked0 = 0, asked1 = 0, landed0 = 0, landed1 = 0;
  if (threadIdx.x == 0) {
    if ((int)blockIdx.y < p.N) {
      mbar_arrive_expect_tx(&full[0], BOX_BYTES);
      tma_load_4d(stages[0], &dy_map, c0, gx0, gy0, blockIdx.y, &full[0]);
      asked0 = 1;
    }
    if ((int)blockIdx.y + step < p.N) {
      mbar_arrive_expect_tx(&full[1], BOX_BYTES);
      tma_load_4d(stages[1], &dy_map, c0, gx0, gy0, blockIdx.y + step, &full[1]);
      asked1 = 1;
    }
  }
  T tsel[K][G::KH];
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int j = 0; j < G::KH; ++j) {
      const int kx = qx + 2 * j;  // flipped filter: wf[ky][kx] = w[K-1-ky][K-1-kx]
      tsel[ky][j] = (kx < K && c < p.C) ? __ldg(w + (size_t)c * KK + (K - 1 - ky) * K + (K - 1 - kx))
                                        : Elem<T>::from_acc(0.f);
    }
  bool gave_up = false;
  int it = 0;
  for (int n = blockIdx.y; n < p.N; n += step, ++it) {
    const int s = it & 1;
    if (!gave_up) {
      if (mbar_wait_bounded(&full[s], (it >> 1) & 1)) {
        landed0 += 1 - s;
        landed1 += s;
      } else {
        gave_up = true;
        atomicOr(error_flag, 1);
      }
    }
    float acc[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) acc[o] = 0.f;
    if (p.pt & 1)
      nhwc_bwd2_rows<T, K, true>(stages[s], col0, lane, tsel, acc);
    else
      nhwc_bwd2_rows<T, K, false>(stages[s], col0, lane, tsel, acc);
    const int ox = x0 + col;
    if (ox < p.Wout && c < p.C) {
      T *op = out + (((size_t)n * p.Hout + y0) * p.Wout + ox) * p.C + c;
      const size_t row_stride = (size_t)p.Wout * p.C;
      const int rows = p.Hout - y0;
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        if (o < rows) *op = Elem<T>::from_acc(acc[o]);
        op += row_stride;
      }
    }
    __syncthreads();  // every thread has read stage s: it may be refilled
    if (threadIdx.x == 0 && !gave_up) {
      const int next = n + 2 * step;
      if (next < p.N) {
        mbar_arrive_expect_tx(&full[s], BOX_BYTES);
        tma_load_4d(stages[s], &dy_map, c0, gx0, gy0, next, &full[s]);
        asked0 += 1 - s;
        asked1 += s;
      }
    }
  }
  if (threadIdx.x == 0 && gave_up) {
    while (landed0 < asked0 && mbar_wait_bounded(&full[0], landed0 & 1)) ++landed0;
    while (landed1 < asked1 && mbar_wait_bounded(&full[1], landed1 & 1)) ++landed1;
  }
}

// Filter gradient, first pass: as nhwc_filter_kernel (block (channel block, slice) walks its
// share of the (image, tile) list, thread (channel, dy column) keeps K*K sums, the columns are
// added in order at the end), with the x tile and the dy tile of every step brought in by one
// tensor copy each, two steps in flight.  dy pixels beyond the map's edge read as zero and add
// nothing.
template <typename T, int K, int S>
__global__ void __launch_bounds__(NhwcGeo<K, S, true>::THREADS, (S == 1 && K < 7) ? 2 : 1)
nhwc_tma_filter_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap dy_map,
                       float *__restrict__ partial, const NhwcFilterParams p, int *error_flag) {
  using G = NhwcGeo<K, S, true>;
  using TG = NhwcTmaGeo<T, K, S, true>;
  constexpr int KK = K * K;
  static_assert(TG::STAGE_BYTES >= G::TW * K * NHWC_CB * (int)sizeof(float),
                "a stage doubles as the reduction buffer");
  extern __shared__ __align__(128) unsigned char nhwc_smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(nhwc_smem + 2 * TG::STAGE_BYTES);
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  const int lane = threadIdx.x & 31, col = threadIdx.x >> 5;
  const int cb = blockIdx.x / p.SL;
  const int slice = blockIdx.x - cb * p.SL;
  const int c0 = cb * NHWC_CB;
  const int per_img = p.tiles_y * p.tiles_x;
  const long long total = (long long)p.N * per_img;
  const long long t_begin = slice * total / p.SL, t_end = (slice + 1) * total / p.SL;
  const int steps = (int)(t_end - t_begin);
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  // thread 0: the next tile to ask for
  int n = (int)(t_begin / per_img);
  int ty = (int)(t_begin - (long long)n * per_img) / p.tiles_x;
  int tx = (int)(t_begin - (long long)n * per_img) - ty * p.tiles_x;
  int asked = 0, landed0 = 0, landed1 = 0;
  auto ask = [&](int s) {
    const int y0 = ty * G::R, x0 = tx * G::TW;
    unsigned char *stage = nhwc_smem + s * TG::STAGE_BYTES;
    mbar_arrive_expect_tx(&full[s], TG::X_BYTES + TG::DY_BYTES);
    tma_load_4d(stage, &x_map, c0, x0 * S - p.pl, y0 * S - p.pt, n, &full[s]);
    tma_load_4d(stage + TG::X_SLOT, &dy_map, c0, x0, y0, n, &full[s]);
    ++asked;
    if (++tx == p.tiles_x) {
      tx = 0;
      if (++ty == p.tiles_y) { ty = 0; ++n; }
    }
  };
  if (threadIdx.x == 0) {
    if (steps > 0) ask(0);
    if (steps > 1) ask(1);
  }
  float acc[K][K];
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx) acc[ky][kx] = 0.f;
  bool gave_up = false;
  for (int it = 0; it < steps; ++it) {
    const int s = it & 1;
    if (!gave_up) {
      if (mbar_wait_bounded(&full[s], (it >> 1) & 1)) {
        landed0 += 1 - s;
        landed1 += s;
      } else {
        gave_up = true;
        atomicOr(error_flag, 2);
      }
    }
    const unsigned char *sx = nhwc_smem + s * TG::STAGE_BYTES;
    const unsigned char *sdy = sx + TG::X_SLOT;
    T g[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) g[o] = reinterpret_cast<const T *>(sdy)[(o * G::TW + col) * NHWC_CB + lane];
#pragma unroll
    for (int ir = 0; ir < G::IH; ++ir) {
      T v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx)
        v[kx] = reinterpret_cast<const T *>(sx)[(ir * G::IW + col * S + kx) * NHWC_CB + lane];
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        const int ky = ir - o * S;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc[ky][kx] = fma_mix(g[o], v[kx], acc[ky][kx]);
        }
      }
    }
    __syncthreads();  // every thread has read stage s: it may be refilled
    if (threadIdx.x == 0 && !gave_up && asked < steps) ask(s);
  }
  if (threadIdx.x == 0 && gave_up) {
    const int asked0 = (asked + 1) / 2, asked1 = asked / 2;
    while (landed0 < asked0 && mbar_wait_bounded(&full[0], landed0 & 1)) ++landed0;
    while (landed1 < asked1 && mbar_wait_bounded(&full[1], landed1 & 1)) ++landed1;
  }
  // no copy is in flight (every one asked for was waited for, or given a last bounded wait):
  // stage 0 now holds, per tap row, [column][kx][channel], and the columns are added in order
  float *red = reinterpret_cast<float *>(nhwc_smem);
#pragma unroll
  for (int ky = 0; ky < K; ++ky) {
    __syncthreads();
#pragma unroll
    for (int kx = 0; kx < K; ++kx) red[(col * K + kx) * NHWC_CB + lane] = acc[ky][kx];
    __syncthreads();
    for (int idx = threadIdx.x; idx < K * NHWC_CB; idx += G::THREADS) {
      const int kx = idx / NHWC_CB, ln = idx - kx * NHWC_CB;
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < G::TW; ++q) sum += red[(q * K + kx) * NHWC_CB + ln];
      if (c0 + ln < p.C) partial[((size_t)(c0 + ln) * p.SL + slice) * KK + ky * K + kx] = sum;
    }
  }
}

// Both gradients at stride 1 from ONE pass over dy (the channels-last counterpart of the fused
// backward of rows_backward.cuh).  A step is a tile of R x TW positions of x / dx for 32 channels;
// it needs the dy box around it (halo k-1: the box backward-input reads) and the plain x box.
// Thread (channel, column) walks the dy box rows once; a value v = dy[r][col + kx] serves
//   dx[o]       += v * w[K-1-ky][K-1-kx]      (ky = r - o: backward-input, same order, same bits)
//   dW'[ky][kx] += x[o] * v                   (the gradient of tap (K-1-ky, K-1-kx))
// Block (channel block, slice) walks its share of the (image, tile) list as the filter kernel does
// and reduces dW' over its columns at the end.  p: H x W = x / dx, Ho x Wo = dy, pt / pl =
// k-1-padding.
template <typename T, int K>
__global__ void __launch_bounds__(NhwcGeo<K, 1, true>::THREADS, K == 3 ? 2 : 1)
nhwc_tma_backward_kernel(const __grid_constant__ CUtensorMap dy_map, const __grid_constant__ CUtensorMap x_map,
                         const T *__restrict__ w, T *__restrict__ dx, float *__restrict__ partial,
                         const NhwcFilterParams p, int *error_flag) {
  using G = NhwcGeo<K, 1, true>;
  using TG = NhwcTmaGeo<T, K, 1, true>;  // "X" slot: the box with halo (dy here); "DY" slot: the plain box (x here)
  constexpr int KK = K * K;
  static_assert(TG::STAGE_BYTES >= G::TW * K * NHWC_CB * (int)sizeof(float),
                "a stage doubles as the reduction buffer");
  extern __shared__ __align__(128) unsigned char nhwc_smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(nhwc_smem + 2 * TG::STAGE_BYTES);
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  const int lane = threadIdx.x & 31, col = threadIdx.x >> 5;
  const int cb = blockIdx.x / p.SL;
  const int slice = blockIdx.x - cb * p.SL;
  const int c0 = cb * NHWC_CB, c = c0 + lane;
  const int per_img = p.tiles_y * p.tiles_x;
  const long long total = (long long)p.N * per_img;
  const long long t_begin = slice * total / p.SL, t_end = (slice + 1) * total / p.SL;
  const int steps = (int)(t_end - t_begin);
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  // thread 0: the next tile to ask for; all threads: the tile being worked on (for the dx stores)
  int an = (int)(t_begin / per_img);
  int aty = (int)(t_begin - (long long)an * per_img) / p.tiles_x;
  int atx = (int)(t_begin - (long long)an * per_img) - aty * p.tiles_x;
  int n = an, ty = aty, tx = atx;
  int asked = 0, landed0 = 0, landed1 = 0;
  auto ask = [&](int s) {
    const int y0 = aty * G::R, x0 = atx * G::TW;
    unsigned char *stage = nhwc_smem + s * TG::STAGE_BYTES;
    mbar_arrive_expect_tx(&full[s], TG::X_BYTES + TG::DY_BYTES);
    tma_load_4d(stage, &dy_map, c0, x0 - p.pl, y0 - p.pt, an, &full[s]);
    tma_load_4d(stage + TG::X_SLOT, &x_map, c0, x0, y0, an, &full[s]);
    ++asked;
    if (++atx == p.tiles_x) {
      atx = 0;
      if (++aty == p.tiles_y) { aty = 0; ++an; }
    }
  };
  if (threadIdx.x == 0) {
    if (steps > 0) ask(0);
    if (steps > 1) ask(1);
  }
  T tapf[K][K];  // the flipped filter
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx)
      tapf[ky][kx] = c < p.C ? __ldg(w + (size_t)c * KK + (KK - 1 - (ky * K + kx))) : Elem<T>::from_acc(0.f);
  float acc[K][K];
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx) acc[ky][kx] = 0.f;
  bool gave_up = false;
  for (int it = 0; it < steps; ++it) {
    const int s = it & 1;
    if (!gave_up) {
      if (mbar_wait_bounded(&full[s], (it >> 1) & 1)) {
        landed0 += 1 - s;
        landed1 += s;
      } else {
        gave_up = true;
        atomicOr(error_flag, 3);
      }
    }
    const T *sdy = reinterpret_cast<const T *>(nhwc_smem + s * TG::STAGE_BYTES);
    const T *sx = reinterpret_cast<const T *>(nhwc_smem + s * TG::STAGE_BYTES + TG::X_SLOT);
    T xs[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) xs[o] = sx[(o * G::TW + col) * NHWC_CB + lane];
    float dxa[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) dxa[o] = 0.f;
#pragma unroll
    for (int r = 0; r < G::IH; ++r) {
      T v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx) v[kx] = sdy[(r * G::IW + col + kx) * NHWC_CB + lane];
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        const int ky = r - o;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) {
            dxa[o] = fma_mix(v[kx], tapf[ky][kx], dxa[o]);
            acc[ky][kx] = fma_mix(xs[o], v[kx], acc[ky][kx]);
          }
        }
      }
    }
    const int y0 = ty * G::R, ox = tx * G::TW + col;
    if (ox < p.W && c < p.C) {
      T *op = dx + (((size_t)n * p.H + y0) * p.W + ox) * p.C + c;
      const size_t row_stride = (size_t)p.W * p.C;
      const int rows = p.H - y0;
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        if (o < rows) *op = Elem<T>::from_acc(dxa[o]);
        op += row_stride;
      }
    }
    if (++tx == p.tiles_x) {
      tx = 0;
      if (++ty == p.tiles_y) { ty = 0; ++n; }
    }
    __syncthreads();  // every thread has read stage s: it may be refilled
    if (threadIdx.x == 0 && !gave_up && asked < steps) ask(s);
  }
  if (threadIdx.x == 0 && gave_up) {
    const int asked0 = (asked + 1) / 2, asked1 = asked / 2;
    while (landed0 < asked0 && mbar_wait_bounded(&full[0], landed0 & 1)) ++landed0;
    while (landed1 < asked1 && mbar_wait_bounded(&full[1], landed1 & 1)) ++landed1;
  }
  // stage 0 now holds, per tap row, [column][kx][channel]; the columns are added in order, and
  // dW'[ky][kx] is the gradient of tap (K-1-ky, K-1-kx)
  float *red = reinterpret_cast<float *>(nhwc_smem);
#pragma unroll
  for (int ky = 0; ky < K; ++ky) {
    __syncthreads();
#pragma unroll
    for (int kx = 0; kx < K; ++kx) red[(col * K + kx) * NHWC_CB + lane] = acc[ky][kx];
    __syncthreads();
    for (int idx = threadIdx.x; idx < K * NHWC_CB; idx += G::THREADS) {
      const int kx = idx / NHWC_CB, ln = idx - kx * NHWC_CB;
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < G::TW; ++q) sum += red[(q * K + kx) * NHWC_CB + ln];
      if (c0 + ln < p.C)
        partial[((size_t)(c0 + ln) * p.SL + slice) * KK + (K - 1 - ky) * K + (K - 1 - kx)] = sum;
    }
  }
}

}  // namespace dwb
