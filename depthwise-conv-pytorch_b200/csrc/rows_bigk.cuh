// Rows family, large filters: odd k from 9 to 31, stride 1, padding k/2, maps up to 32 columns
// wide (the reference has no kernel at all for these: k > 7 at stride 1 falls off the end of its
// dispatch, dwconv_kernel.cu:808-845, and small maps go to PyTorch, dwconv.py:125-128).
//
// Same pipeline as rows_conv_kernel (persistent CTAs, producer warp, bulk-copied tiles of whole
// planes, 16 zero bytes standing in for rows outside the map).  Differences, because k*k taps
// and a k-row window do not fit in registers:
//   * lane j of a segment owns ONE column; for every input row it builds the k-wide window
//     in[row][j-P .. j+P] with k-1 shuffles, once, and uses it for all the output rows of the
//     block that row contributes to (U = 16 rows per block, one accumulator each);
//   * the producer gathers the taps of the tile's channels into shared memory as fp32 rows of
//     KMAX entries (zero beyond k, flipped for backward-input); consumers read them with
//     128-bit broadcast loads: one load per four FMAs.
// Summation order per output: input rows ascending = tap rows ascending, taps left to right, one
// accumulator, one FMA per tap: the order of the reference kernels, bit-identical fp32.
#pragma once

#include "rows_engine.cuh"

namespace dwb {

constexpr int BIGK_U = 16;  // output rows per block

template <typename T, int KMAX, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_bigk_conv_kernel(const RowsParams p, const int K, const uint32_t inv_KK, int *__restrict__ error_flag) {
  extern __shared__ __align__(128) unsigned char rows_smem[];
  RowsRing ring = rows_ring_init(rows_smem, p.TAPB, p.NST);

  const T *__restrict__ gin = static_cast<const T *>(p.in);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  T *__restrict__ gout = static_cast<T *>(p.out);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int P = K / 2;
  const size_t plane_in = (size_t)p.Hin * p.Win;
  const size_t plane_out = (size_t)p.Hout * p.Wout;
  const int KROW = K * KMAX;  // fp32 entries of one channel's taps in a stage

  if (warp == ROWS_CWARPS) {
    // ------------------------------- producer warp -------------------------------
    int stage = -1, use = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
      if (++stage == p.NST) {
        stage = 0;
        ++use;
      }
      if (use > 0 && !mbar_wait_bounded(&ring.empty[stage], (use - 1) & 1)) {
        *ring.abort_flag = 1;
        atomicExch(error_flag, 1);
      }
      if (*ring.abort_flag) break;
      const int gcount = min(p.G, p.NC - tile * p.G);  // whole planes: tile == plane group
      unsigned char *sb = ring.stage(stage);
      uint32_t tx = 0;
      if (lane == 0) {
        fence_proxy_async_smem();
        tx = stage_range(reinterpret_cast<T *>(sb + p.TAPB + 16), gin + (size_t)tile * p.G * plane_in,
                         gcount * (int)plane_in, &ring.full[stage]);
      }
      // taps: fp32, KMAX per row, zero beyond k, flipped for backward-input; 16 loads in flight
      float *staps = reinterpret_cast<float *>(sb);
      const int ntap = gcount * KROW;
      const int c_base = (int)(((long long)tile * p.G) % p.C);
      constexpr int TB = 16;
      for (int base = 0; base < ntap; base += 32 * TB) {
        float v[TB];
#pragma unroll
        for (int k = 0; k < TB; ++k) {
          const int idx = base + k * 32 + lane;
          v[k] = 0.f;
          if (idx < ntap) {
            const int g = magic_div(idx, inv_KK);
            const int rem = idx - g * KROW;
            const int ty = rem / KMAX;
            const int txx = rem - ty * KMAX;
            if (txx < K) {
              const int t = ty * K + txx;
              v[k] = Elem<T>::ld(gw + (size_t)((c_base + g) % p.C) * (K * K) + (p.flip ? (K * K - 1 - t) : t));
            }
          }
        }
#pragma unroll
        for (int k = 0; k < TB; ++k) {
          const int idx = base + k * 32 + lane;
          if (idx < ntap) staps[idx] = v[k];
        }
      }
      tx = warp_sum(tx);
      __syncwarp();
      if (lane == 0) {
        if (tx)
          mbar_arrive_expect_tx(&ring.full[stage], tx);
        else
          mbar_arrive(&ring.full[stage]);
      }
    }
    return;
  }

  // ------------------------------- consumer warps -------------------------------
  const int LW = p.LW;
  const int segs_per_warp = 32 / LW;
  const int j = lane & (LW - 1);
  const int seg = warp * segs_per_warp + lane / LW;
  const int NSEG = ROWS_CWARPS * segs_per_warp;
  const bool col_alive = j < p.Win;  // Win == Wout

  // window column tx is input column j - P + tx; real data iff inside the map and tx < k
  uint32_t win_mask[KMAX];
#pragma unroll
  for (int tx = 0; tx < KMAX; ++tx) {
    const int col = j - P + tx;
    win_mask[tx] = (tx < K && col >= 0 && col < p.Win) ? 0xffffffffu : 0u;
  }
  const int lane_base = lane - P;

  const int ntasks = p.G * p.NRB;
  const uint32_t row_bytes = (uint32_t)p.Win * (uint32_t)sizeof(T);
  int stage = -1, use = 0;
  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
    if (++stage == p.NST) {
      stage = 0;
      ++use;
    }
    if (!mbar_wait_bounded(&ring.full[stage], use & 1)) {
      *ring.abort_flag = 1;
      atomicExch(error_flag, 1);
    }
    if (*ring.abort_flag) break;
    const int gcount = min(p.G, p.NC - tile * p.G);
    unsigned char *sb = ring.stage(stage);
    const uint32_t staps = smem_u32(sb);
    const uint32_t zaddr = smem_u32(sb + p.TAPB);
    const int phase = slot_phase(gin + (size_t)tile * p.G * plane_in);
    const uint32_t sdata = zaddr + 16u + (uint32_t)(phase * (int)sizeof(T));

    for (int t0 = 0; t0 < ntasks; t0 += NSEG) {
      const int task = t0 + seg;
      const int g = magic_div(task, p.inv_NRB);
      const int rb = task - g * p.NRB;
      const bool active = (task < ntasks) && (g < gcount);
      const int plane = tile * p.G + (active ? g : 0);
      int r_begin, r_end;
      task_rows_fast<1>(rb, p.NRB, p.inv_NRB, 0, p.Hout, r_begin, r_end);
      const uint32_t tp = staps + (uint32_t)((active ? g : 0) * KROW * 4);
      const int lim = (active && col_alive) ? p.Hin : 0;
      const uint32_t plane_addr = sdata + (uint32_t)((g * p.Hin * p.Win + j) * (int)sizeof(T));
      T *orow = gout + (size_t)plane * plane_out + (size_t)r_begin * p.Wout + j;
      int rows_left = (active && col_alive) ? (r_end - r_begin) : 0;

      for (int rr = 0; rr < p.RBH; rr += BIGK_U) {
        const int r0 = r_begin + rr;
        float acc[BIGK_U];
#pragma unroll
        for (int u = 0; u < BIGK_U; ++u) acc[u] = 0.f;
        // input rows r0 - P .. r0 + U - 1 + P, in order
        int q = r0 - P;
        uint32_t a = plane_addr + (uint32_t)q * row_bytes;  // wraps for q < 0; never used then
        for (int n = 0; n < BIGK_U + K - 1; ++n) {
          float own[1];
          SmemLd<T, 1>::ld(((unsigned)q < (unsigned)lim) ? a : zaddr, own);
          float win[KMAX];
#pragma unroll
          for (int tx = 0; tx < KMAX; ++tx)
            win[tx] = __uint_as_float(
                __shfl_sync(0xffffffffu, __float_as_uint(own[0]), (lane_base + tx) & 31) & win_mask[tx]);
          // this input row is tap row ty = n - u of output row r0 + u
#pragma unroll
          for (int u = 0; u < BIGK_U; ++u) {
            const int ty = n - u;
            if ((unsigned)ty < (unsigned)K) {
              const uint32_t trow = tp + (uint32_t)(ty * KMAX * 4);
#pragma unroll
              for (int t4 = 0; t4 < KMAX / 4; ++t4) {
                float w4[4];
                SmemLd<float, 4>::ld(trow + t4 * 16, w4);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[u] = fmaf(win[t4 * 4 + e], w4[e], acc[u]);
              }
            }
          }
          a += row_bytes;
          q += 1;
        }
#pragma unroll
        for (int u = 0; u < BIGK_U; ++u) {
          if (u < rows_left) *orow = Elem<T>::from_acc(acc[u]);
          orow += p.Wout;
        }
        rows_left -= BIGK_U;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[stage]);
  }
}

// Backward-filter for large filters.  Work items and tiles as in rows_filter_kernel (group of
// G consecutive channels x slice of the image list; a tile = the x planes and dy planes of the
// group in one image, two bulk copies).  A task (channel g, block of dy rows rb) belongs to one
// whole warp, and here lane = tap COLUMN tx: the lane builds, for every x row, the window
// x[row][tx-P .. tx-P+W-1] with shuffles (the same window as the forward kernel, lane and column
// swapping roles) and adds dy[r][0..W-1] . window into acc[ty] for the k tap rows ty that pair
// this x row with a dy row r of the block; dy rows are 128-bit broadcast loads.  No reduction
// across lanes is needed: lane tx ends up holding dW[c][0..k-1][tx], written to the slot
// (channel, slice, row block) of the partials; the finalize kernel adds the slots in order.
template <typename T, int KMAX, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_bigk_filter_kernel(const RowsFilterParams p, const int K, int *__restrict__ error_flag) {
  extern __shared__ __align__(128) unsigned char rows_smem[];
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  RowsRing ring = rows_ring_init(rows_smem, 0, p.NST);

  const T *__restrict__ gx = static_cast<const T *>(p.x);
  const T *__restrict__ gdy = static_cast<const T *>(p.dy);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int P = K / 2;
  const size_t plane = (size_t)p.H * p.W;  // x and dy planes have the same extent
  const int nitems = p.NCG * p.SL;

  if (warp == ROWS_CWARPS) {
    // ------------------------------- producer warp -------------------------------
    bool stop = false;
    int stage = -1, use = 0;
    for (int item = blockIdx.x; item < nitems && !stop; item += gridDim.x) {
      const int cg = item / p.SL;
      const int slice = item - cg * p.SL;
      const int c0 = cg * p.G;
      const int gcount = min(p.G, p.C - c0);
      const int t_begin = (int)(((long long)slice * p.TPC) / p.SL);
      const int t_end = (int)(((long long)(slice + 1) * p.TPC) / p.SL);
      for (int n = t_begin; n < t_end; ++n) {
        if (++stage == p.NST) {
          stage = 0;
          ++use;
        }
        if (use > 0 && !mbar_wait_bounded(&ring.empty[stage], (use - 1) & 1)) {
          *ring.abort_flag = 1;
          atomicExch(error_flag, 2);
        }
        if (*ring.abort_flag) {
          stop = true;
          break;
        }
        unsigned char *sb = ring.stage(stage);
        const size_t pl0 = (size_t)n * p.C + c0;
        uint32_t tx = 0;
        if (lane == 0) {
          fence_proxy_async_smem();
          tx = stage_range(reinterpret_cast<T *>(sb + 16), gx + pl0 * plane, gcount * (int)plane,
                           &ring.full[stage]);
        } else if (lane == 1) {
          fence_proxy_async_smem();
          tx = stage_range(reinterpret_cast<T *>(sb + p.DYOFF), gdy + pl0 * plane,
                           gcount * (int)plane, &ring.full[stage]);
        }
        tx = warp_sum(tx);
        __syncwarp();
        if (lane == 0) {
          if (tx)
            mbar_arrive_expect_tx(&ring.full[stage], tx);
          else
            mbar_arrive(&ring.full[stage]);
        }
      }
    }
    return;
  }

  // ------------------------------- consumer warps -------------------------------
  const int ntasks = p.G * p.NRB;  // <= consumer warps
  const int g = magic_div(warp, p.inv_NRB);
  const int rb = warp - g * p.NRB;
  const bool col_alive = lane < p.W;
  // window entry jj is x column lane - P + jj; real data iff inside the map, for a real tap column
  uint32_t win_mask[32];
#pragma unroll
  for (int jj = 0; jj < 32; ++jj) {
    const int col = lane - P + jj;
    win_mask[jj] = (lane < K && jj < p.W && col >= 0 && col < p.W) ? 0xffffffffu : 0u;
  }
  const int lane_base = lane - P;
  const uint32_t row_bytes = (uint32_t)p.W * (uint32_t)sizeof(T);
  int r_begin, r_end;
  task_rows_fast<1>(rb, p.NRB, p.inv_NRB, 0, p.Ho, r_begin, r_end);

  int stage = -1, use = 0;
  bool aborted = false;
  for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
    const int cg = item / p.SL;
    const int slice = item - cg * p.SL;
    const int c0 = cg * p.G;
    const int gcount = min(p.G, p.C - c0);
    const int t_begin = (int)(((long long)slice * p.TPC) / p.SL);
    const int t_end = (int)(((long long)(slice + 1) * p.TPC) / p.SL);
    const bool active = (warp < ntasks) && (g < gcount);

    float acc[KMAX];
#pragma unroll
    for (int ty = 0; ty < KMAX; ++ty) acc[ty] = 0.f;

    for (int n = t_begin; n < t_end; ++n) {
      if (++stage == p.NST) {
        stage = 0;
        ++use;
      }
      if (!aborted && (*ring.abort_flag || !mbar_wait_bounded(&ring.full[stage], use & 1))) {
        aborted = true;
        *ring.abort_flag = 1;
        atomicExch(error_flag, 2);
      }
      if (aborted) continue;
      unsigned char *sb = ring.stage(stage);
      const size_t pl0 = (size_t)n * p.C + c0;
      const uint32_t zaddr = smem_u32(sb);
      const int xphase = slot_phase(gx + pl0 * plane);
      const int dphase = slot_phase(gdy + pl0 * plane);
      if (active) {  // warp-uniform
        const uint32_t xplane =
            zaddr + 16u + (uint32_t)((xphase + g * (int)plane + lane) * (int)sizeof(T));
        const uint32_t dplane =
            smem_u32(sb + p.DYOFF) + (uint32_t)((dphase + g * (int)plane) * (int)sizeof(T));
        const int lim = col_alive ? p.H : 0;
        // x rows r_begin - P .. r_end - 1 + P pair with the dy rows of the block
        int q = r_begin - P;
        uint32_t a = xplane + (uint32_t)q * row_bytes;
        for (; q < r_end + P; ++q, a += row_bytes) {
          float own[1];
          SmemLd<T, 1>::ld(((unsigned)q < (unsigned)lim) ? a : zaddr, own);
          float win[32];
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            win[jj] = __uint_as_float(
                __shfl_sync(0xffffffffu, __float_as_uint(own[0]), (lane_base + jj) & 31) & win_mask[jj]);
#pragma unroll
          for (int ty = 0; ty < KMAX; ++ty) {
            const int r = q - ty + P;  // dy row this x row meets through tap row ty
            if (ty < K && r >= r_begin && r < r_end) {
              const uint32_t drow = dplane + (uint32_t)r * row_bytes;
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) {
                if (j4 * 4 < p.W) {
                  float d4[4];
                  SmemLd<T, 4>::ld(drow + j4 * 4 * (int)sizeof(T), d4);
#pragma unroll
                  for (int e = 0; e < 4; ++e) acc[ty] = fmaf(d4[e], win[j4 * 4 + e], acc[ty]);
                }
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty[stage]);
    }
    // lane tx holds dW[c0+g][ty][tx] of this (slice, row block)
    if (active && lane < K) {
      float *dst = p.partial + (((size_t)(c0 + g) * p.SL + slice) * p.NRB + rb) * (size_t)(K * K) + lane;
#pragma unroll
      for (int ty = 0; ty < KMAX; ++ty)
        if (ty < K) dst[ty * K] = acc[ty];
    }
  }
}

}  // namespace dwb

