// Rows family, fused backward: ONE pass over dy produces both gradients.
//
// The reference issues the two gradients as separate operators, each reading dy from memory
// (torch_dwconv/dwconv.py:56-68).  Here a tile brings the dy rows and the x rows of a group of
// planes into shared memory once; a segment of a warp streams the dy rows through the register
// window of the backward-input kernel (own columns by one vector load, halo columns by shuffle)
// and uses every window value twice:
//
//     dx[r][c]      += win[ty][c + tx] * flipped_tap[ty][tx]      (the backward-input sum, same
//                                                                   order: bit-identical)
//     dW'[ty][tx]   += win[ty][c + tx] * x[r][c]                   (x: own columns only, no halo)
//
// dW'[ty][tx] is the gradient of tap (K-1-ty, K-1-tx): the pairs (x element, dy element) that
// meet in dx's sum are exactly the pairs of the filter gradient.  With stride 2 the window is
// the polyphase window of the backward-input kernel and a (row, tap) pair contributes only when
// its parity matches, for both sums alike.
//
// Work decomposition is the backward-filter kernel's: a work item is (group of consecutive
// channels, slice of the (image, row tile) list), one item per resident CTA; a segment keeps its
// (channel, row block), its taps and its K*K gradient accumulators for the whole item; partial
// sums per (channel, slice, tap) have one writer and are added in order by the second pass.
#pragma once

#include <cooperative_groups.h>

#include "rows_engine.cuh"

namespace dwb {

// Second pass inside the first, for problems whose work items all run at once (one per CTA) with
// at most 8 image slices per channel group: the SL CTAs of a channel group are launched as one
// thread-block CLUSTER; each leaves its per-channel sums in its own shared memory, the cluster
// meets, and CTA 0 of the cluster adds the SL values of every (channel, tap) in slice order
// straight out of the other CTAs' shared memory (distributed shared memory) and writes dW.  No
// partial sums in global memory, no second kernel: one launch fewer per backward, which is what
// small problems are made of.  Deterministic (fixed order), no atomics.
// `fin`: gcount * KK floats in this CTA's shared memory, complete on entry for this CTA's consumer
// threads (they have met); called by ALL threads of every CTA of the cluster (`worker` false for
// the producer warp, which only takes part in the two cluster barriers).
template <typename T>
__device__ __forceinline__ void cluster_finalize(float *fin, int count, T *__restrict__ dw_group,
                                                 int slices, bool worker) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();  // every CTA's sums are in its shared memory
  if (worker && cluster.block_rank() == 0) {
    for (int idx = threadIdx.x; idx < count; idx += ROWS_CWARPS * 32) {
      float total = 0.f;
      for (int r = 0; r < slices; ++r) total += *cluster.map_shared_rank(fin + idx, r);
      dw_group[idx] = Elem<T>::from_acc(total);
    }
  }
  cluster.sync();  // nobody's shared memory goes away before CTA 0 has read it
}

struct RowsBackwardParams {
  const void *x;
  const void *dy;
  const void *w;
  void *dx;
  float *partial;  // [C][SL][K*K]
  int N, C, H, W, Ho, Wo;
  int G;      // consecutive channels (planes of one image) per tile; whole planes when NRT == 1
  int NRT;    // row tiles per plane (G == 1 when > 1)
  int TH;     // dx (= x) rows per row tile
  int NRB, RBH, LW;  // G * NRB <= segments per CTA: a segment keeps its (channel, row block)
  uint32_t inv_NRB;
  int NST;    // stages in the ring
  int NCG;    // channel groups = ceil(C / G)
  int TPC;    // tiles per channel group = N * NRT
  int SL;     // work items (slices of that tile list) per channel group
  int XOFF;   // byte offset of the x rows inside a stage (16-byte aligned); the stage starts
              // with 16 zero bytes, the dy rows follow
  void *dw_direct;  // not null: one item per CTA, SL CTAs per cluster, dW written here (see
                    // cluster_finalize); `partial` is then unused
};

struct BackwardTile {
  int n, R0, th, in_lo, in_hi;
};
template <int K, int S, int MODE>
__device__ __forceinline__ BackwardTile backward_tile(const RowsBackwardParams &p, int tt) {
  BackwardTile t;
  t.n = tt / p.NRT;
  const int rt = tt - t.n * p.NRT;
  t.R0 = rt * p.TH;
  t.th = min(p.TH, p.H - t.R0);
  if (p.NRT == 1) {
    t.in_lo = 0;
    t.in_hi = p.Ho;
  } else {
    tile_in_rows(K, S, MODE, t.R0, t.th, p.Ho, t.in_lo, t.in_hi);
  }
  return t;
}

// MODE: geometry of the dy window.  Stride 1: MODE_FWD (the transposed operation is the same
// correlation with the flipped filter); stride 2: MODE_BWD (polyphase).
// VI: dy columns per lane, VO: dx / x columns per lane.
template <typename T, int K, int S, int MODE, int VI, int VO, int U, bool MASK, bool EXACT, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_backward_kernel(const RowsBackwardParams p, int *__restrict__ error_flag) {
  using Geo = RowsGeo<K, S, MODE, VI, VO, U>;
  constexpr int KK = K * K;
  constexpr int RS = (MODE == MODE_BWD) ? S : 1;
  extern __shared__ __align__(128) unsigned char rows_smem[];
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  RowsRing ring = rows_ring_init(rows_smem, 0, p.NST);
  pdl_wait();  // everything earlier in the stream has completed; global memory may be touched

  const T *__restrict__ gx = static_cast<const T *>(p.x);
  const T *__restrict__ gdy = static_cast<const T *>(p.dy);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  T *__restrict__ gdx = static_cast<T *>(p.dx);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const size_t plane_x = (size_t)p.H * p.W;
  const size_t plane_dy = (size_t)p.Ho * p.Wo;
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
      for (int tt = t_begin; tt < t_end; ++tt) {
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
        const BackwardTile t = backward_tile<K, S, MODE>(p, tt);
        unsigned char *sb = ring.stage(stage);
        const size_t pl0 = (size_t)t.n * p.C + c0;
        uint32_t tx = 0;
        if (lane == 0) {
          fence_proxy_async_smem();
          const int de = (p.NRT == 1) ? gcount * (int)plane_dy : (t.in_hi - t.in_lo) * p.Wo;
          tx = stage_range(reinterpret_cast<T *>(sb + 16),
                           gdy + pl0 * plane_dy + (size_t)t.in_lo * p.Wo, de, &ring.full[stage]);
        } else if (lane == 1) {
          fence_proxy_async_smem();
          const int xe = (p.NRT == 1) ? gcount * (int)plane_x : t.th * p.W;
          tx = stage_range(reinterpret_cast<T *>(sb + p.XOFF),
                           gx + pl0 * plane_x + (size_t)t.R0 * p.W, xe, &ring.full[stage]);
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
    if (p.dw_direct != nullptr) cluster_finalize<T>(nullptr, 0, static_cast<T *>(nullptr), 0, false);
    return;
  }

  // ------------------------------- consumer warps -------------------------------
  const int LW = p.LW;
  const int segs_per_warp = 32 / LW;
  const int j = lane & (LW - 1);
  const int seg = warp * segs_per_warp + lane / LW;
  const bool in_alive = j * VI < p.Wo;   // Wo % VI == 0
  const bool out_alive = j * VO < p.W;   // W % VO == 0

  int src_lane[Geo::NIN];
  uint32_t halo_mask[Geo::NIN];
  make_lane_tables<Geo, VI>(src_lane, halo_mask, lane, j, p.Wo);

  const int ntasks = p.G * p.NRB;  // <= segments per CTA
  const int g = magic_div(seg, p.inv_NRB);  // this segment's channel within the group, row block
  const int rb = seg - g * p.NRB;
  const uint32_t row_bytes = (uint32_t)p.Wo * (uint32_t)sizeof(T);   // dy
  const uint32_t xrow_bytes = (uint32_t)p.W * (uint32_t)sizeof(T);   // x
  float *red = ring.scratch;  // [ntasks][KK]
  // A warp whose wait expired keeps walking the loops without waiting or computing, so that
  // it still meets the other consumer warps at every consumer_sync().
  bool aborted = false;
  int stage = -1, use = 0;
  for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
    const int cg = item / p.SL;
    const int slice = item - cg * p.SL;
    const int c0 = cg * p.G;
    const int gcount = min(p.G, p.C - c0);
    const int t_begin = (int)(((long long)slice * p.TPC) / p.SL);
    const int t_end = (int)(((long long)(slice + 1) * p.TPC) / p.SL);
    const bool active = (seg < ntasks) && (g < gcount);

    // the channel's taps, flipped in both axes, for the whole item
    float taps[K][K];
    {
      const T *tp = gw + (size_t)(c0 + (active ? g : 0)) * KK;
#pragma unroll
      for (int ty = 0; ty < K; ++ty)
#pragma unroll
        for (int tx = 0; tx < K; ++tx)
          taps[ty][tx] = active ? Elem<T>::ld(tp + (KK - 1 - (ty * K + tx))) : 0.f;
    }
    float dwacc[K][K];
#pragma unroll
    for (int ty = 0; ty < K; ++ty)
#pragma unroll
      for (int tx = 0; tx < K; ++tx) dwacc[ty][tx] = 0.f;

    for (int tt = t_begin; tt < t_end; ++tt) {
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
      const BackwardTile t = backward_tile<K, S, MODE>(p, tt);
      unsigned char *sb = ring.stage(stage);
      const size_t pl0 = (size_t)t.n * p.C + c0;
      const uint32_t zaddr = smem_u32(sb);  // 16 bytes that are always zero
      const int nrows = t.in_hi - t.in_lo;  // staged dy rows per plane
      const int dphase = slot_phase(gdy + pl0 * plane_dy + (size_t)t.in_lo * p.Wo);
      const int xphase = slot_phase(gx + pl0 * plane_x + (size_t)t.R0 * p.W);
      const int xrows = (p.NRT == 1) ? p.H : t.th;  // staged x rows per plane

      int r_begin, r_end;
      task_rows_fast<RS>(rb, p.NRB, p.inv_NRB, t.R0, t.th, r_begin, r_end);
      int q = (MODE == MODE_FWD ? r_begin * S : r_begin / S) + Geo::RMIN - t.in_lo;
      int lim = 0;
      uint32_t a = zaddr;
      if (active && in_alive) {
        lim = nrows;
        a = zaddr + 16u + (uint32_t)((dphase + (g * nrows + q) * p.Wo + j * VI) * (int)sizeof(T));
      }
      const bool st_ok = active && out_alive;
      uint32_t xa = zaddr;
      uint32_t xpitch = 0;
      if (st_ok) {
        xa = smem_u32(sb + p.XOFF) +
             (uint32_t)((xphase + (g * xrows + (r_begin - t.R0)) * p.W + j * VO) * (int)sizeof(T));
        xpitch = xrow_bytes;
      }
      T *orow = gdx + (pl0 + (active ? g : 0)) * plane_x + (size_t)r_begin * p.W + j * VO;
      int rows_left = st_ok ? (r_end - r_begin) : 0;

      float rows[Geo::KR][Geo::NIN];
      {
        float own[Geo::KR - Geo::ADV][VI];
#pragma unroll
        for (int i = 0; i < Geo::KR - Geo::ADV; ++i)
          load_own_row<T, VI>(own[i], a, row_bytes, q, lim, zaddr);
#pragma unroll
        for (int i = 0; i < Geo::KR - Geo::ADV; ++i)
          build_window_row<Geo, VI, MASK>(rows[i], own[i], src_lane, halo_mask);
      }
      for (int rr = 0; rr < p.RBH; rr += U) {
        float xs[U][VO];
        {
          float own[Geo::ADV][VI];
#pragma unroll
          for (int i = 0; i < Geo::ADV; ++i) load_own_row<T, VI>(own[i], a, row_bytes, q, lim, zaddr);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            // rows past the task's end read zeros: they add nothing to the filter gradient
            SmemLd<T, VO>::ld((EXACT || u < rows_left) ? xa : zaddr, xs[u]);
            xa += xpitch;
          }
#pragma unroll
          for (int i = 0; i < Geo::ADV; ++i)
            build_window_row<Geo, VI, MASK>(rows[Geo::KR - Geo::ADV + i], own[i], src_lane, halo_mask);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float acc[VO];
#pragma unroll
          for (int e = 0; e < VO; ++e) acc[e] = 0.f;
#pragma unroll
          for (int ty = 0; ty < K; ++ty) {
            if (!Geo::used(u, ty)) continue;
            const int ri = Geo::rel(u, ty) - Geo::RMIN;
#pragma unroll
            for (int tx = 0; tx < K; ++tx) {
#pragma unroll
              for (int e = 0; e < VO; ++e) {
                if (!Geo::used(e, tx)) continue;
                const float v = rows[ri][Geo::rel(e, tx) - Geo::CMIN];
                acc[e] = fmaf(v, taps[ty][tx], acc[e]);
                dwacc[ty][tx] = fmaf(v, xs[u][e], dwacc[ty][tx]);
              }
            }
          }
          if (EXACT ? st_ok : (u < rows_left)) GmemSt<T, VO>::st(orow, acc);
          orow += p.W;
        }
#pragma unroll
        for (int i = 0; i < Geo::KR - Geo::ADV; ++i)
#pragma unroll
          for (int ci = 0; ci < Geo::NIN; ++ci) rows[i][ci] = rows[i + Geo::ADV][ci];
        if (!EXACT) rows_left -= U;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty[stage]);
    }

    // item done: sum over the segment's lanes, then over the channel's row blocks; window
    // position (ty, tx) is the gradient of tap (K-1-ty, K-1-tx)
#pragma unroll
    for (int ty = 0; ty < K; ++ty)
#pragma unroll
      for (int tx = 0; tx < K; ++tx) {
        float v = dwacc[ty][tx];
        for (int off = LW >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (j == 0 && seg < ntasks) red[seg * KK + (KK - 1 - (ty * K + tx))] = v;
      }
    consumer_sync();
    // direct mode: the ring is idle (this CTA's only item is done), its first stage holds the sums
    float *fin = reinterpret_cast<float *>(ring.stage(0) + 16);
    for (int idx = threadIdx.x; idx < gcount * KK; idx += ROWS_CWARPS * 32) {
      const int gg = idx / KK;
      const int tap = idx - gg * KK;
      float s = 0.f;
      for (int b = 0; b < p.NRB; ++b) s += red[(gg * p.NRB + b) * KK + tap];
      if (p.dw_direct != nullptr)
        fin[idx] = s;
      else
        p.partial[((size_t)(c0 + gg) * p.SL + slice) * KK + tap] = s;
    }
    consumer_sync();  // red is rewritten by the next item; fin is complete
    if (p.dw_direct != nullptr)
      cluster_finalize<T>(fin, gcount * KK, static_cast<T *>(p.dw_direct) + (size_t)c0 * KK, p.SL, true);
  }
}

}  // namespace dwb
