// Tiles family, stride 1, rows on 16-byte boundaries: the input tile comes in by ONE tensor
// copy (TMA, cp.async.bulk.tensor.3d) per tile instead of a loop of loads and stores.
//
// The map is described to the copy engine as a 3-d tensor (column, row, plane); a tile with
// its halo is a box of it.  The engine fills whatever part of the box lies outside the tensor
// with zeros: that IS the padding on all four sides, and no thread tests a bound while
// staging.  The box starts at the 16-byte boundary at or left of the halo (the engine wants
// the innermost coordinate on such a boundary; it may be negative), so the kernels below
// index from `off`, as the 16-byte register staging of tile_kernels.cuh does.  Elements stay
// in the tensors' type in shared memory and are converted when read.
//
// Two stages: thread 0 asks for the CTA's tile of plane i+2 as soon as all threads have read
// plane i's, so a copy is always in flight while the CTA computes.  A CTA keeps its tile
// position and walks the planes blockIdx.y, + gridDim.y, ...; the thread-to-output mapping and
// the order of the multiply-adds are those of tile_conv_kernel: same bits.
//
// Waits on the copies are bounded; on expiry the thread raises the error flag, stops waiting
// and runs to the end (its outputs are then wrong, the flag says so).
#pragma once

#include <cuda.h>  // CUtensorMap (type only; the encoder is looked up at run time)

#include "rows_engine.cuh"  // mbarrier wrappers, bounded wait
#include "tile_kernels.cuh"

namespace dwb {

template <typename T, int K, int TW>
struct TileTmaGeo {
  static constexpr int V = 16 / (int)sizeof(T);
  static constexpr int TH = TILE_THREADS / TW * TILE_R;  // output rows per tile
  static constexpr int IH = TH + K - 1;                  // input rows per tile
  static constexpr int IW = TW + K - 1;                  // input columns under the tile
  static constexpr int BW = (IW + 2 * V - 2) / V * V;    // box columns: IW + up to V-1, in chunks
  static constexpr int BOX_BYTES = IH * BW * (int)sizeof(T);
  static constexpr int STAGE_BYTES = (BOX_BYTES + 127) / 128 * 128;
  static constexpr int IR = TILE_R + K - 1;              // input rows under one thread's strip
};

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

// Forward and (flip, other paddings) backward-input at stride 1.  p.off as in TileParams.
template <typename T, int K, int TW>
__global__ void __launch_bounds__(TILE_THREADS, K == 3 ? 6 : (K == 5 ? 4 : 3))
tile_tma_conv_kernel(const __grid_constant__ CUtensorMap in_map, const T *__restrict__ w,
                     T *__restrict__ out, const TileParams p, int *error_flag) {
  using G = TileTmaGeo<T, K, TW>;
  constexpr int KK = K * K;
  __shared__ __align__(128) unsigned char stages[2][G::STAGE_BYTES];
  __shared__ uint64_t full[2];
  const int tc = threadIdx.x % TW;  // output column inside the tile
  const int tr = threadIdx.x / TW;  // strip of TILE_R output rows
  const int ty = (int)blockIdx.x / p.tiles_x, tx = (int)blockIdx.x - ty * p.tiles_x;
  const int y0 = ty * G::TH, x0 = tx * TW;       // first output of the tile
  const int bx = x0 - p.pl - p.off, by = y0 - p.pt;  // first element of the box (bx: 16-byte aligned)
  const int step = gridDim.y;
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  // thread 0: copies asked for / seen complete, per stage
  int asked0 = 0, asked1 = 0, landed0 = 0, landed1 = 0;
  if (threadIdx.x == 0) {
    if ((int)blockIdx.y < p.NC) {
      mbar_arrive_expect_tx(&full[0], G::BOX_BYTES);
      tma_load_3d(stages[0], &in_map, bx, by, blockIdx.y, &full[0]);
      asked0 = 1;
    }
    if ((int)blockIdx.y + step < p.NC) {
      mbar_arrive_expect_tx(&full[1], G::BOX_BYTES);
      tma_load_3d(stages[1], &in_map, bx, by, blockIdx.y + step, &full[1]);
      asked1 = 1;
    }
  }
  const size_t plane_out = (size_t)p.Hout * p.Wout;
  int chan = (int)blockIdx.y % p.C;
  const int chan_step = step % p.C;
  bool gave_up = false;
  int it = 0;
  for (int plane = blockIdx.y; plane < p.NC; plane += step, ++it) {
    const int s = it & 1;
    T tap[K][K];  // taps and staged values stay in the storage type: fma_mix multiplies them as they are
    {
      const T *tp = w + (size_t)chan * KK;
      if (p.flip) {  // (two copies of the loop: constant offsets in each, no select per tap)
#pragma unroll
        for (int ky = 0; ky < K; ++ky)
#pragma unroll
          for (int kx = 0; kx < K; ++kx) tap[ky][kx] = __ldg(tp + (KK - 1 - (ky * K + kx)));
      } else {
#pragma unroll
        for (int ky = 0; ky < K; ++ky)
#pragma unroll
          for (int kx = 0; kx < K; ++kx) tap[ky][kx] = __ldg(tp + (ky * K + kx));
      }
    }
    if (!gave_up) {
      if (mbar_wait_bounded(&full[s], (it >> 1) & 1)) {
        landed0 += 1 - s;
        landed1 += s;
      } else {
        gave_up = true;
        atomicOr(error_flag, 1);
      }
    }
    float acc[TILE_R];
#pragma unroll
    for (int o = 0; o < TILE_R; ++o) acc[o] = 0.f;
    const unsigned char *stage = stages[s];
    const int first = (tr * TILE_R) * G::BW + p.off + tc;
#pragma unroll
    for (int ir = 0; ir < G::IR; ++ir) {
      T v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx) v[kx] = reinterpret_cast<const T *>(stage)[first + ir * G::BW + kx];
#pragma unroll
      for (int o = 0; o < TILE_R; ++o) {
        const int ky = ir - o;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc[o] = fma_mix(v[kx], tap[ky][kx], acc[o]);
        }
      }
    }
    if (p.ep.on) {
      float sc, bi;
      epilogue_coeffs<T>(p.ep, chan, sc, bi);
#pragma unroll
      for (int o = 0; o < TILE_R; ++o) acc[o] = apply_epilogue<float>(acc[o], sc, bi, p.ep.act);
    }
    const int ox = x0 + tc;
    if (ox < p.Wout) {
      T *op = out + (size_t)plane * plane_out + (size_t)(y0 + tr * TILE_R) * p.Wout + ox;
      const int rows = p.Hout - (y0 + tr * TILE_R);  // rows of this strip inside the map
#pragma unroll
      for (int o = 0; o < TILE_R; ++o) {
        if (o < rows) *op = Elem<T>::from_acc(acc[o]);
        op += p.Wout;
      }
    }
    __syncthreads();  // every thread has read stage s: it may be refilled
    if (threadIdx.x == 0 && !gave_up) {
      const int next = plane + 2 * step;
      if (next < p.NC) {
        mbar_arrive_expect_tx(&full[s], G::BOX_BYTES);
        tma_load_3d(stages[s], &in_map, bx, by, next, &full[s]);
        asked0 += 1 - s;
        asked1 += s;
      }
    }
    chan += chan_step;
    if (chan >= p.C) chan -= p.C;
  }
  // a thread that gave up may still have copies on their way into this CTA's shared memory:
  // thread 0 (the only one that asks for copies, and only while it has not given up) gives
  // each outstanding one another bounded wait before the CTA ends
  if (threadIdx.x == 0 && gave_up) {
    while (landed0 < asked0 && mbar_wait_bounded(&full[0], landed0 & 1)) ++landed0;
    while (landed1 < asked1 && mbar_wait_bounded(&full[1], landed1 & 1)) ++landed1;
  }
}

// Filter gradient, first pass, stride 1: as tile_filter_kernel (block (c, slice) walks one of SL
// equal ranges of channel c's tiles, a thread owns a dy column and a strip of dy rows and keeps
// K*K sums), with the x tile (halo included) and the dy tile of every step brought in by one
// tensor copy each, two steps in flight.  Only thread 0 knows where a tile lies; the arithmetic
// is relative to the boxes.  What a box holds outside its tensor reads as zero: the padding of
// x, and dy elements beyond the map's edge (they add nothing).
template <typename T, int K, int TW>
__global__ void __launch_bounds__(TILE_THREADS, K == 3 ? 4 : (K == 5 ? 3 : 2))
tile_tma_filter_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap dy_map,
                       float *__restrict__ partial, const TileFilterParams p, int *error_flag) {
  using G = TileTmaGeo<T, K, TW>;
  constexpr int KK = K * K;
  constexpr int DY_BYTES = G::TH * TW * (int)sizeof(T);
  constexpr int X_BYTES = G::STAGE_BYTES;  // the x box, rounded up to 128 bytes
  constexpr int STEP_BYTES = X_BYTES + (DY_BYTES + 127) / 128 * 128;
  __shared__ __align__(128) unsigned char stages[2][STEP_BYTES];
  __shared__ uint64_t full[2];
  __shared__ float red[TILE_THREADS / 32][KK];
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  const int c = blockIdx.x / p.SL;
  const int slice = blockIdx.x - c * p.SL;
  const int per_img = p.tiles_x * p.tiles_y;
  const long long total = (long long)p.N * per_img;
  const long long t0 = slice * total / p.SL, t1 = (slice + 1) * total / p.SL;
  const int steps = (int)(t1 - t0);
  const int tc = threadIdx.x % TW, tr = threadIdx.x / TW;
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  // thread 0: the next tile to ask for, and the copies asked for / seen complete per stage
  int n = (int)(t0 / per_img);
  int ty = (int)(t0 - (long long)n * per_img) / p.tiles_x;
  int tx = (int)(t0 - (long long)n * per_img) - ty * p.tiles_x;
  int asked = 0, landed0 = 0, landed1 = 0;
  auto ask = [&](int s) {
    const int plane = n * p.C + c;
    const int y0 = ty * G::TH, x0 = tx * TW;
    mbar_arrive_expect_tx(&full[s], G::BOX_BYTES + DY_BYTES);
    tma_load_3d(stages[s], &x_map, x0 - p.pl - p.off, y0 - p.pt, plane, &full[s]);
    tma_load_3d(stages[s] + X_BYTES, &dy_map, x0, y0, plane, &full[s]);
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
    const unsigned char *xs = stages[s];
    const unsigned char *gs = stages[s] + X_BYTES;
    T g[TILE_R];
#pragma unroll
    for (int o = 0; o < TILE_R; ++o) g[o] = reinterpret_cast<const T *>(gs)[(tr * TILE_R + o) * TW + tc];
    const int first = (tr * TILE_R) * G::BW + p.off + tc;
#pragma unroll
    for (int ir = 0; ir < G::IR; ++ir) {
      T v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx) v[kx] = reinterpret_cast<const T *>(xs)[first + ir * G::BW + kx];
#pragma unroll
      for (int o = 0; o < TILE_R; ++o) {
        const int ky = ir - o;
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
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx) {
      const float v = warp_sum(acc[ky][kx]);
      if (lane == 0) red[wid][ky * K + kx] = v;
    }
  __syncthreads();
  if (threadIdx.x < KK) {
    float sum = 0.f;
#pragma unroll
    for (int q = 0; q < TILE_THREADS / 32; ++q) sum += red[q][threadIdx.x];
    partial[((size_t)c * p.SL + slice) * KK + threadIdx.x] = sum;
  }
}

}  // namespace dwb
