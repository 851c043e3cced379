// Forward / stride-1 backward-input for SMALL maps (7, 14 or 28 columns wide), padding k/2:
// "a lane owns a row", the layout of lanerow_backward.cuh applied to the single-output operators.
//
// A tile is a group of whole planes adjacent in memory (one bulk copy in); consumer lane L of
// the CTA owns row L of the tile (plane-major), reads the K input rows around it from shared
// memory itself (rows outside the plane: a block of zero bytes), keeps one input row and the W
// accumulators of its output row in registers, and writes the finished row to a staging area laid
// out like the tensor; the tile leaves with one bulk store.  No shuffles, no per-column lane
// tables; every column index, and every tap that falls off the map edge, is resolved at compile
// time.  Taps are applied ty-major / tx-minor with one FMA each (products with padding zeros are
// not issued: they leave the sum unchanged), so results are bit-identical to rows_conv_kernel's.
#pragma once

#include "lanerow_backward.cuh"

namespace dwb {

struct LaneRowConvParams {
  const void *in;
  const void *w;
  void *out;
  int NC, C, H;
  int G;        // planes per tile: G * H <= consumer lanes
  int NST;
  int ntiles;
  int flip;     // apply the filter flipped in both axes (backward-input)
  int INOFF, OUTOFF;  // byte offsets inside a stage; the stage starts with LANEROW_ZERO_BYTES zeros
  EpilogueArgs ep;
};

template <typename T, int K, int W, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
lanerow_conv_kernel(const LaneRowConvParams p, int *__restrict__ error_flag) {
  constexpr int KK = K * K;
  constexpr int P = K / 2;
  constexpr int ES = (int)sizeof(T);
  constexpr uint32_t ROWB = W * ES;
  static_assert(ROWB <= LANEROW_ZERO_BYTES, "a row of zeros must fit the zero block");
  extern __shared__ __align__(128) unsigned char rows_smem[];
  pdl_launch_dependents();  // the next kernel in the stream may take freed SMs early
  RowsRing ring = rows_ring_init(rows_smem, 0, p.NST);
  if (threadIdx.x < p.NST * (LANEROW_ZERO_BYTES / 16))
    *reinterpret_cast<uint4 *>(rows_smem + (threadIdx.x / (LANEROW_ZERO_BYTES / 16)) * ring.stage_bytes +
                               (threadIdx.x % (LANEROW_ZERO_BYTES / 16)) * 16) = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  pdl_wait();  // everything earlier in the stream has completed; global memory may be touched

  const T *__restrict__ gin = static_cast<const T *>(p.in);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  T *__restrict__ gout = static_cast<T *>(p.out);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int plane_elems = p.H * W;

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
      if (lane == 0) {
        unsigned char *sb = ring.stage(stage);
        const int gcount = min(p.G, p.NC - tile * p.G);
        fence_proxy_async_smem();
        const uint32_t tx = stage_range(reinterpret_cast<T *>(sb + p.INOFF),
                                        gin + (size_t)tile * p.G * plane_elems, gcount * plane_elems,
                                        &ring.full[stage]);
        if (tx)
          mbar_arrive_expect_tx(&ring.full[stage], tx);
        else
          mbar_arrive(&ring.full[stage]);
      }
      __syncwarp();
    }
    return;
  }

  // ------------------------------- consumer warps -------------------------------
  const int L = warp * 32 + lane;  // this lane's row of the tile (plane-major)
  const int g = L / p.H;
  const int r = L - g * p.H;
  const bool elected = (L == 0);
  bool aborted = false;
  int stage = -1, use = 0;
  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
    if (++stage == p.NST) {
      stage = 0;
      ++use;
    }
    const int gcount = min(p.G, p.NC - tile * p.G);
    const bool active = g < gcount;
    const size_t pl0 = (size_t)tile * p.G;
    const int ch = (int)((pl0 + (active ? g : 0)) % p.C);
    // this plane's taps, from global memory (a few cache lines per tile), before the wait
    float taps[K][K];
    {
      const T *tp = gw + (size_t)ch * KK;
#pragma unroll
      for (int ty = 0; ty < K; ++ty)
#pragma unroll
        for (int tx = 0; tx < K; ++tx)
          taps[ty][tx] = active ? Elem<T>::ld(tp + (p.flip ? KK - 1 - (ty * K + tx) : ty * K + tx)) : 0.f;
    }
    if (!aborted && (*ring.abort_flag || !mbar_wait_bounded(&ring.full[stage], use & 1))) {
      aborted = true;
      *ring.abort_flag = 1;
      atomicExch(error_flag, 1);
    }
    unsigned char *sb = ring.stage(stage);
    if (!aborted) {
      const uint32_t zaddr = smem_u32(sb);
      const int iphase = slot_phase(gin + pl0 * plane_elems);
      const int ophase = slot_phase(gout + pl0 * plane_elems);
      const uint32_t inbase = smem_u32(sb + p.INOFF) + (uint32_t)((iphase + g * plane_elems) * ES);
      float acc[W];
#pragma unroll
      for (int c = 0; c < W; ++c) acc[c] = 0.f;
#pragma unroll
      for (int ty = 0; ty < K; ++ty) {
        const int rr = r - P + ty;  // input row under tap row ty
        float d[W];
        RowIO<T, W>::ld((active && (unsigned)rr < (unsigned)p.H) ? inbase + (uint32_t)rr * ROWB : zaddr, d);
#pragma unroll
        for (int tx = 0; tx < K; ++tx) {
#pragma unroll
          for (int c = 0; c < W; ++c) {
            const int cc = c - P + tx;  // input column under tap column tx
            if (cc < 0 || cc >= W) continue;  // off the map: a zero that adds nothing
            acc[c] = fmaf(d[cc], taps[ty][tx], acc[c]);
          }
        }
      }
      if (p.ep.on) {
        float sc, bi;
        epilogue_coeffs<T>(p.ep, ch, sc, bi);
#pragma unroll
        for (int c = 0; c < W; ++c) acc[c] = apply_epilogue<float>(acc[c], sc, bi, p.ep.act);
      }
      if (active)
        RowIO<T, W>::st(smem_u32(sb + p.OUTOFF) + (uint32_t)((ophase + g * plane_elems + r * W) * ES), acc);
      fence_proxy_async_smem();  // the rows just written are read by the bulk store below
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty[stage]);  // the input rows of this stage are consumed
    }
    // before everybody meets, the elected lane makes sure the staging area the NEXT tile will
    // write is free (its bulk store, NST tiles ago, has read it)
    if (elected) {
      if (p.NST == 2)
        bulk_wait_read<0>();
      else
        bulk_wait_read<1>();
    }
    consumer_sync();
    if (elected && !aborted)
      store_range(gout + pl0 * plane_elems, reinterpret_cast<const T *>(sb + p.OUTOFF),
                  gcount * plane_elems);
  }
  if (elected) bulk_wait_all();  // every tile has reached global memory
}

}  // namespace dwb
