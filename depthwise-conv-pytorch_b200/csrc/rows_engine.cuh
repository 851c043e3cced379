// "Rows" kernel family: the B200 path for filters 3x3 / 5x5 / 7x7, stride 1 or 2, "same"
// padding (p = k/2), fp32 and fp16, maps up to 128 columns wide.
//
// Structure shared by forward, backward-input and backward-filter:
//
//  * A persistent CTA walks a list of tiles.  A tile is a run of full-width rows of one plane,
//    or a group of whole small planes; either way it is ONE contiguous byte range of the NCHW
//    tensor, so it is brought into shared memory by a single bulk asynchronous copy
//    (cp.async.bulk, the TMA unit) that signals an mbarrier.  Stages form a ring; the copy of
//    tile i+2 is in flight while tile i is computed.  Ranges that do not meet the 16-byte rules
//    of the bulk copy (misaligned base, ragged last group) are staged by plain loads instead.
//  * A tile is split into tasks (plane, block of output rows).  A task is executed by a
//    SEGMENT of a warp: LW = 8, 16 or 32 adjacent lanes.  Lane j of the segment owns VI
//    adjacent input columns and VO adjacent output columns.  It reads its own columns of an
//    input row from shared memory with one vector load and gets the k-1 halo columns from
//    neighbouring lanes by warp shuffle; rows stream through a register window, so each
//    input element is read from shared memory once per task.
//  * The filter taps of the task's channel sit in registers.  Every output has one
//    accumulator, taps are applied row-major with one FMA each: the summation order of the
//    reference kernels (torch_dwconv/dwconv_kernel.cu:164-172), hence bit-identical fp32.
//  * Outputs leave as VO-wide vector stores, contiguous across the segment.
//
// All waits on mbarriers are bounded; on expiry the CTA raises a flag the host can read
// (rows_take_device_error) and leaves after a bounded wait for its copies in flight.
#pragma once

#include "common.cuh"
#include "rows_api.cuh"

namespace dwb {

enum { MODE_FWD = 0, MODE_BWD = 1 };

constexpr int ROWS_THREADS = 256;
constexpr int ROWS_WARPS = ROWS_THREADS / 32;
constexpr int ROWS_STAGES = 3;
constexpr int ROWS_STAGE_BYTES = 32 * 1024;
constexpr int ROWS_SMEM_BYTES = ROWS_STAGES * ROWS_STAGE_BYTES + 128;
constexpr unsigned ROWS_WAIT_LIMIT = 1u << 22;  // mbarrier polls before giving up

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Generic-proxy accesses to shared memory (earlier reads of a stage) ordered before the
// async-proxy write of the next bulk copy into it.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, uint32_t bytes,
                                              uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false if the phase did not complete within ROWS_WAIT_LIMIT polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
  for (unsigned i = 0; i < ROWS_WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// ---------------------------------------------------------------------------------------
// Compile-time geometry of one kernel variant.
//   FWD, stride S: out row r+u reads in rows (r+u)*S - P + ty; columns alike.
//   BWD, stride S: out (=dx) row r+u, r a multiple of S, reads in (=dy) row (r+u-P+ty)/S for the
//                  taps ty with (u-P+ty) divisible by S; taps are the flipped filter.
// "rel" values are relative to the chunk's base input row (r*S resp. r/S) and to the lane's
// first own input column (j*VI).
// ---------------------------------------------------------------------------------------
template <int K, int S, int MODE, int VI, int VO, int U>
struct RowsGeo {
  static constexpr int P = K / 2;
  static constexpr int fdiv(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }
  static constexpr bool used(int u, int t) {
    return MODE == MODE_FWD ? true : (((u - P + t) % S) + S) % S == 0;
  }
  static constexpr int rel(int u, int t) {
    return MODE == MODE_FWD ? u * S - P + t : fdiv(u - P + t, S);
  }
  static constexpr int min_rel(int n) {
    int m = 1 << 20;
    for (int u = 0; u < n; ++u)
      for (int t = 0; t < K; ++t)
        if (used(u, t) && rel(u, t) < m) m = rel(u, t);
    return m;
  }
  static constexpr int max_rel(int n) {
    int m = -(1 << 20);
    for (int u = 0; u < n; ++u)
      for (int t = 0; t < K; ++t)
        if (used(u, t) && rel(u, t) > m) m = rel(u, t);
    return m;
  }
  static constexpr int RMIN = min_rel(U), RMAX = max_rel(U);
  static constexpr int KR = RMAX - RMIN + 1;                    // window rows per chunk
  static constexpr int ADV = MODE == MODE_FWD ? U * S : U / S;  // input rows per chunk
  static constexpr int CMIN = min_rel(VO), CMAX = max_rel(VO);
  static constexpr int NIN = CMAX - CMIN + 1;  // window columns
  static_assert(MODE == MODE_FWD || (U % S == 0 && VO % S == 0), "BWD: U, VO multiples of S");
  static_assert(MODE == MODE_FWD ? VI == VO * S : VO == VI * S, "VI/VO inconsistent with stride");
  static_assert(KR > ADV, "window must overlap the next chunk");
};

// First / one-past-last input row a tile of output rows [R0, R0+th) reads, clipped to the map.
template <int K, int S, int MODE>
__host__ __device__ __forceinline__ void tile_in_rows(int R0, int th, int Hin, int &lo, int &hi) {
  constexpr int P = K / 2;
  int a, b;
  if (MODE == MODE_FWD) {
    a = R0 * S - P;
    b = (R0 + th - 1) * S - P + K;
  } else {
    const int n0 = R0 - P, n1 = R0 + th - 1 - P + K - 1;
    a = n0 >= 0 ? n0 / S : -((-n0 + S - 1) / S);
    b = (n1 >= 0 ? n1 / S : -((-n1 + S - 1) / S)) + 1;
  }
  lo = a < 0 ? 0 : a;
  hi = b > Hin ? Hin : b;
  if (hi < lo) hi = lo;
}

struct RowsParams {
  const void *in;
  const void *w;
  void *out;
  int NC, C;
  int Hin, Win, Hout, Wout;
  int G;    // planes per tile (whole planes when > 1)
  int NRT;  // row tiles per plane group (1 when G > 1)
  int TH;   // output rows per row tile
  int NRB;  // row blocks (tasks) per plane inside a tile
  int RBH;  // row-loop trip count of a task, a multiple of U
  int LW;   // lanes per segment: 8, 16 or 32
  int ntiles;
  int flip;  // apply the filter flipped in both axes (backward-input)
};

template <typename T, int V> struct VecIO;
// VI/VO elements between shared or global memory and fp32 registers.
template <> struct VecIO<float, 1> {
  static __device__ __forceinline__ void ld(const float *p, float (&v)[1]) { v[0] = *p; }
  static __device__ __forceinline__ void st(float *p, const float (&v)[1]) { *p = v[0]; }
};
template <> struct VecIO<float, 2> {
  static __device__ __forceinline__ void ld(const float *p, float (&v)[2]) {
    const float2 t = *reinterpret_cast<const float2 *>(p);
    v[0] = t.x; v[1] = t.y;
  }
  static __device__ __forceinline__ void st(float *p, const float (&v)[2]) {
    *reinterpret_cast<float2 *>(p) = make_float2(v[0], v[1]);
  }
};
template <> struct VecIO<float, 4> {
  static __device__ __forceinline__ void ld(const float *p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void st(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct VecIO<__half, 1> {
  static __device__ __forceinline__ void ld(const __half *p, float (&v)[1]) { v[0] = __half2float(*p); }
  static __device__ __forceinline__ void st(__half *p, const float (&v)[1]) { *p = __float2half_rn(v[0]); }
};
template <> struct VecIO<__half, 2> {
  static __device__ __forceinline__ void ld(const __half *p, float (&v)[2]) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(p));
    v[0] = t.x; v[1] = t.y;
  }
  static __device__ __forceinline__ void st(__half *p, const float (&v)[2]) {
    *reinterpret_cast<__half2 *>(p) = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
  }
};
template <> struct VecIO<__half, 4> {
  static __device__ __forceinline__ void ld(const __half *p, float (&v)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void st(__half *p, const float (&v)[4]) {
    __half2 a = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
    __half2 b = __halves2half2(__float2half_rn(v[2]), __float2half_rn(v[3]));
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t *>(&a);
    raw.y = *reinterpret_cast<uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(p) = raw;
  }
};

// Shared-memory bookkeeping of the stage ring.
struct RowsRing {
  unsigned char *base;
  uint64_t *bar;   // ROWS_STAGES barriers
  int *abort_flag;
  uint32_t phase;  // bit s = parity the next wait on stage s expects
  __device__ __forceinline__ unsigned char *stage(int s) const { return base + s * ROWS_STAGE_BYTES; }
};

__device__ __forceinline__ RowsRing rows_ring_init(unsigned char *smem) {
  RowsRing r;
  r.base = smem;
  r.bar = reinterpret_cast<uint64_t *>(smem + ROWS_STAGES * ROWS_STAGE_BYTES);
  r.abort_flag = reinterpret_cast<int *>(r.bar + ROWS_STAGES);
  r.phase = 0;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < ROWS_STAGES; ++s) mbar_init(&r.bar[s], 1);
    *r.abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  return r;
}

// A contiguous byte range can go through the bulk-copy unit iff both ends obey its rules.
__device__ __forceinline__ bool bulk_ok(const void *src, size_t bytes) {
  return bytes > 0 && ((reinterpret_cast<uintptr_t>(src) | bytes) & 15) == 0;
}

// Plain-load staging of a range the bulk copy cannot take.  All threads; caller syncs.
template <typename T>
__device__ __forceinline__ void stage_by_loads(T *dst, const T *src, int n) {
  for (int i = threadIdx.x; i < n; i += ROWS_THREADS) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------
// One chunk-row of the register window: own columns from shared memory, halo by shuffle.
// ---------------------------------------------------------------------------------------
template <typename T, typename Geo, int VI>
__device__ __forceinline__ void load_window_row(float (&win)[Geo::NIN], const T *row_ptr,
                                                const bool row_ok, const int lane,
                                                const uint32_t (&halo_mask)[Geo::NIN]) {
  float own[VI];
#pragma unroll
  for (int i = 0; i < VI; ++i) own[i] = 0.f;
  if (row_ok) VecIO<T, VI>::ld(row_ptr, own);
#pragma unroll
  for (int ci = 0; ci < Geo::NIN; ++ci) {
    const int c = ci + Geo::CMIN;
    const int dl = Geo::fdiv(c, VI);
    const int el = c - dl * VI;
    if (dl == 0) {
      win[ci] = own[el];
    } else {
      const uint32_t bits =
          __shfl_sync(0xffffffffu, __float_as_uint(own[el]), (lane + dl) & 31) & halo_mask[ci];
      win[ci] = __uint_as_float(bits);
    }
  }
}

// Per-lane masks: window column c is real data iff 0 <= j*VI + c < Win.
template <typename Geo, int VI>
__device__ __forceinline__ void make_halo_masks(uint32_t (&halo_mask)[Geo::NIN], int j, int Win) {
#pragma unroll
  for (int ci = 0; ci < Geo::NIN; ++ci) {
    const int col = j * VI + ci + Geo::CMIN;
    halo_mask[ci] = (col >= 0 && col < Win) ? 0xffffffffu : 0u;
  }
}

// ---------------------------------------------------------------------------------------
// forward / backward-input
// ---------------------------------------------------------------------------------------
template <typename T, int K, int S, int MODE, int VI, int VO, int U, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_conv_kernel(const RowsParams p, int *__restrict__ error_flag) {
  using Geo = RowsGeo<K, S, MODE, VI, VO, U>;
  extern __shared__ __align__(128) unsigned char rows_smem[];
  RowsRing ring = rows_ring_init(rows_smem);

  const T *__restrict__ gin = static_cast<const T *>(p.in);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  T *__restrict__ gout = static_cast<T *>(p.out);

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int LW = p.LW;
  const int segs_per_warp = 32 / LW;
  const int j = lane & (LW - 1);
  const int seg = warp * segs_per_warp + lane / LW;
  const int NSEG = ROWS_WARPS * segs_per_warp;
  const bool in_alive = j * VI < p.Win;    // Win % VI == 0: a lane's block is all in or all out
  const bool out_alive = j * VO < p.Wout;  // Wout % VO == 0

  uint32_t halo_mask[Geo::NIN];
  make_halo_masks<Geo, VI>(halo_mask, j, p.Win);

  const size_t plane_in = (size_t)p.Hin * p.Win;
  const size_t plane_out = (size_t)p.Hout * p.Wout;
  const int ntasks = p.G * p.NRB;

  // tile -> source range; identical on every thread
  auto tile_geom = [&](int tile, int &pg, int &R0, int &th, int &gcount, int &in_lo, int &in_hi) {
    pg = tile / p.NRT;
    const int rt = tile - pg * p.NRT;
    R0 = rt * p.TH;
    th = min(p.TH, p.Hout - R0);
    gcount = min(p.G, p.NC - pg * p.G);
    if (p.G > 1) {
      in_lo = 0;
      in_hi = p.Hin;
    } else {
      tile_in_rows<K, S, MODE>(R0, th, p.Hin, in_lo, in_hi);
    }
  };
  auto tile_src = [&](int pg, int gcount, int in_lo, int in_hi, const T *&src, size_t &elems) {
    src = gin + (size_t)pg * p.G * plane_in + (size_t)in_lo * p.Win;
    elems = (p.G > 1) ? (size_t)gcount * plane_in : (size_t)(in_hi - in_lo) * p.Win;
  };
  auto issue = [&](int tile, int stage) {  // thread 0 only
    int pg, R0, th, gcount, in_lo, in_hi;
    tile_geom(tile, pg, R0, th, gcount, in_lo, in_hi);
    const T *src;
    size_t elems;
    tile_src(pg, gcount, in_lo, in_hi, src, elems);
    const size_t bytes = elems * sizeof(T);
    if (bulk_ok(src, bytes)) {
      mbar_expect_tx(&ring.bar[stage], (uint32_t)bytes);
      bulk_copy_g2s(ring.stage(stage), src, (uint32_t)bytes, &ring.bar[stage]);
    }
  };

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < ROWS_STAGES - 1; ++s) {
      const int t = blockIdx.x + s * gridDim.x;
      if (t < p.ntiles) issue(t, s);
    }
  }

  int it = 0;
  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++it) {
    const int stage = it % ROWS_STAGES;
    if (threadIdx.x == 0) {
      const int nt = tile + (ROWS_STAGES - 1) * gridDim.x;
      if (nt < p.ntiles) {
        fence_proxy_async_smem();
        issue(nt, (it + ROWS_STAGES - 1) % ROWS_STAGES);
      }
    }
    int pg, R0, th, gcount, in_lo, in_hi;
    tile_geom(tile, pg, R0, th, gcount, in_lo, in_hi);
    const T *src;
    size_t elems;
    tile_src(pg, gcount, in_lo, in_hi, src, elems);
    T *sdata = reinterpret_cast<T *>(ring.stage(stage));
    if (bulk_ok(src, elems * sizeof(T))) {
      const uint32_t parity = (ring.phase >> stage) & 1u;
      ring.phase ^= 1u << stage;
      if (!mbar_wait_bounded(&ring.bar[stage], parity)) {
        *ring.abort_flag = 1;
        atomicExch(error_flag, 1);
      }
    } else {
      stage_by_loads(sdata, src, (int)elems);
      __syncthreads();
    }
    const int tile_rows = in_hi - in_lo;

    for (int t0 = 0; t0 < ntasks; t0 += NSEG) {
      const int task = t0 + seg;
      const int g = task / p.NRB;
      const int rb = task - g * p.NRB;
      const bool active = (task < ntasks) && (g < gcount);
      const int plane = pg * p.G + (active ? g : 0);
      // balanced split of the tile's rows over the NRB row blocks, starts on multiples of S
      constexpr int RS = (MODE == MODE_BWD) ? S : 1;
      const int r_begin = R0 + ((rb * th) / p.NRB) / RS * RS;
      const int r_end = (rb == p.NRB - 1) ? (R0 + th) : R0 + (((rb + 1) * th) / p.NRB) / RS * RS;

      float taps[K][K];
      {
        const T *wp = gw + (size_t)(plane % p.C) * (K * K);
#pragma unroll
        for (int ty = 0; ty < K; ++ty)
#pragma unroll
          for (int tx = 0; tx < K; ++tx) {
            const int idx = ty * K + tx;
            taps[ty][tx] = active ? Elem<T>::ld(wp + (p.flip ? (K * K - 1 - idx) : idx)) : 0.f;
          }
      }
      const T *splane = sdata + (size_t)(active ? g : 0) * tile_rows * p.Win + j * VI;
      T *oplane = gout + (size_t)plane * plane_out + j * VO;

      float rows[Geo::KR][Geo::NIN];
      // chunk base input row: r*S (FWD) or r/S (BWD), plus RMIN
      int ibase = (MODE == MODE_FWD ? r_begin * S : r_begin / S) + Geo::RMIN;
#pragma unroll
      for (int i = 0; i < Geo::KR - Geo::ADV; ++i) {
        const int ir = ibase + i;
        const bool ok = active && in_alive && ir >= in_lo && ir < in_hi;
        load_window_row<T, Geo, VI>(rows[i], splane + (size_t)(ir - in_lo) * p.Win, ok, lane,
                                    halo_mask);
      }
      for (int rr = 0; rr < p.RBH; rr += U) {
        const int r = r_begin + rr;
#pragma unroll
        for (int i = Geo::KR - Geo::ADV; i < Geo::KR; ++i) {
          const int ir = ibase + i;
          const bool ok = active && in_alive && ir >= in_lo && ir < in_hi;
          load_window_row<T, Geo, VI>(rows[i], splane + (size_t)(ir - in_lo) * p.Win, ok, lane,
                                      halo_mask);
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
                acc[e] = fmaf(rows[ri][Geo::rel(e, tx) - Geo::CMIN], taps[ty][tx], acc[e]);
              }
            }
          }
          if (active && out_alive && (r + u) < r_end)
            VecIO<T, VO>::st(oplane + (size_t)(r + u) * p.Wout, acc);
        }
#pragma unroll
        for (int i = 0; i < Geo::KR - Geo::ADV; ++i)
#pragma unroll
          for (int ci = 0; ci < Geo::NIN; ++ci) rows[i][ci] = rows[i + Geo::ADV][ci];
        ibase += Geo::ADV;
      }
    }
    __syncthreads();  // every warp is done with this stage before it is refilled
    if (*ring.abort_flag) break;
  }
  // Leaving early with copies in flight would let them land in shared memory that no longer
  // belongs to this CTA: give each pending stage a bounded wait.
  if (*ring.abort_flag && threadIdx.x == 0) {
    for (int s = 0; s < ROWS_STAGES; ++s) (void)mbar_wait_bounded(&ring.bar[s], (ring.phase >> s) & 1u);
  }
}


// ---------------------------------------------------------------------------------------
// backward-filter, first pass
// ---------------------------------------------------------------------------------------
struct RowsFilterParams {
  const void *x;
  const void *dy;
  float *partial;  // [C][SL][K*K]
  int N, C, H, W, Ho, Wo;
  int G;    // images (planes of one channel) per tile; whole planes when > 1
  int NRT;  // row tiles per plane
  int TH;   // dy rows per row tile
  int NRB, RBH, LW;
  int TPC;  // tiles per channel = ceil(N / G) * NRT
  int SL;   // CTAs (slices of the tile list) per channel
  int XPL;  // elements reserved per x plane in a stage
  int DPL;  // elements reserved per dy plane in a stage
  int DYOFF;  // byte offset of the dy region inside a stage (multiple of 128)
  int x_bulk, dy_bulk;  // plane byte sizes are multiples of 16 (all planes equally aligned)
};

// CTA (channel c, slice): accumulates dW[c] over its share of the (image, row tile) list.
// Lane layout as in the forward kernel: the x window is the forward window, dy is the lane's VO
// own output columns.  Each lane keeps K*K accumulators across all its tasks; one warp-shuffle
// sum and one cross-warp sum in shared memory at the end give the slice's partial, written
// to its own slot (no atomics); a second kernel adds the slices in order.
template <typename T, int K, int S, int VI, int VO, int U, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_filter_kernel(const RowsFilterParams p, int *__restrict__ error_flag) {
  using Geo = RowsGeo<K, S, MODE_FWD, VI, VO, U>;
  extern __shared__ __align__(128) unsigned char rows_smem[];
  RowsRing ring = rows_ring_init(rows_smem);

  const T *__restrict__ gx = static_cast<const T *>(p.x);
  const T *__restrict__ gdy = static_cast<const T *>(p.dy);

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int LW = p.LW;
  const int segs_per_warp = 32 / LW;
  const int j = lane & (LW - 1);
  const int seg = warp * segs_per_warp + lane / LW;
  const int NSEG = ROWS_WARPS * segs_per_warp;
  const bool in_alive = j * VI < p.W;
  const bool out_alive = j * VO < p.Wo;

  uint32_t halo_mask[Geo::NIN];
  make_halo_masks<Geo, VI>(halo_mask, j, p.W);

  const int c = blockIdx.x / p.SL;
  const int slice = blockIdx.x - c * p.SL;
  const int t_begin = (int)(((long long)slice * p.TPC) / p.SL);
  const int t_end = (int)(((long long)(slice + 1) * p.TPC) / p.SL);
  const size_t plane_x = (size_t)p.H * p.W;
  const size_t plane_dy = (size_t)p.Ho * p.Wo;
  const int ntasks = p.G * p.NRB;

  struct TileGeom {
    int n0, gcount, R0, th, in_lo, in_hi;
    bool bx, bd;
    uint32_t xbytes, dbytes;
  };
  auto tile_geom = [&](int tt) {
    TileGeom g;
    const int ng = tt / p.NRT;
    const int rt = tt - ng * p.NRT;
    g.n0 = ng * p.G;
    g.gcount = min(p.G, p.N - g.n0);
    g.R0 = rt * p.TH;
    g.th = min(p.TH, p.Ho - g.R0);
    if (p.G > 1) {
      g.in_lo = 0;
      g.in_hi = p.H;
    } else {
      tile_in_rows<K, S, MODE_FWD>(g.R0, g.th, p.H, g.in_lo, g.in_hi);
    }
    g.xbytes = (uint32_t)((g.in_hi - g.in_lo) * p.W * (int)sizeof(T));
    g.dbytes = (uint32_t)(g.th * p.Wo * (int)sizeof(T));
    const T *xs = gx + ((size_t)g.n0 * p.C + c) * plane_x + (size_t)g.in_lo * p.W;
    const T *ds = gdy + ((size_t)g.n0 * p.C + c) * plane_dy + (size_t)g.R0 * p.Wo;
    g.bx = p.x_bulk && bulk_ok(xs, g.xbytes);
    g.bd = p.dy_bulk && bulk_ok(ds, g.dbytes);
    return g;
  };
  auto issue = [&](int tt, int stage) {  // all lanes of warp 0
    const TileGeom g = tile_geom(tt);
    const uint32_t total = (uint32_t)g.gcount * ((g.bx ? g.xbytes : 0u) + (g.bd ? g.dbytes : 0u));
    if (total == 0) return;
    if (lane == 0) mbar_expect_tx(&ring.bar[stage], total);
    __syncwarp();
    T *xs_s = reinterpret_cast<T *>(ring.stage(stage));
    T *ds_s = reinterpret_cast<T *>(ring.stage(stage) + p.DYOFF);
    for (int gi = lane; gi < g.gcount; gi += 32) {
      const size_t pl = (size_t)(g.n0 + gi) * p.C + c;
      if (g.bx)
        bulk_copy_g2s(xs_s + (size_t)gi * p.XPL, gx + pl * plane_x + (size_t)g.in_lo * p.W, g.xbytes,
                      &ring.bar[stage]);
      if (g.bd)
        bulk_copy_g2s(ds_s + (size_t)gi * p.DPL, gdy + pl * plane_dy + (size_t)g.R0 * p.Wo, g.dbytes,
                      &ring.bar[stage]);
    }
  };

  if (warp == 0) {
#pragma unroll
    for (int s = 0; s < ROWS_STAGES - 1; ++s)
      if (t_begin + s < t_end) issue(t_begin + s, s);
  }

  float acc[K][K];
#pragma unroll
  for (int ty = 0; ty < K; ++ty)
#pragma unroll
    for (int tx = 0; tx < K; ++tx) acc[ty][tx] = 0.f;

  int it = 0;
  for (int tt = t_begin; tt < t_end; ++tt, ++it) {
    const int stage = it % ROWS_STAGES;
    if (warp == 0) {
      const int nt = tt + ROWS_STAGES - 1;
      if (nt < t_end) {
        fence_proxy_async_smem();
        issue(nt, (it + ROWS_STAGES - 1) % ROWS_STAGES);
      }
    }
    const TileGeom g = tile_geom(tt);
    T *xs_s = reinterpret_cast<T *>(ring.stage(stage));
    T *ds_s = reinterpret_cast<T *>(ring.stage(stage) + p.DYOFF);
    if (g.bx || g.bd) {
      const uint32_t parity = (ring.phase >> stage) & 1u;
      ring.phase ^= 1u << stage;
      if (!mbar_wait_bounded(&ring.bar[stage], parity)) {
        *ring.abort_flag = 1;
        atomicExch(error_flag, 2);
      }
    }
    if (!g.bx || !g.bd) {
      const int xe = (g.in_hi - g.in_lo) * p.W, de = g.th * p.Wo;
      for (int gi = 0; gi < g.gcount; ++gi) {
        const size_t pl = (size_t)(g.n0 + gi) * p.C + c;
        if (!g.bx)
          stage_by_loads(xs_s + (size_t)gi * p.XPL, gx + pl * plane_x + (size_t)g.in_lo * p.W, xe);
        if (!g.bd)
          stage_by_loads(ds_s + (size_t)gi * p.DPL, gdy + pl * plane_dy + (size_t)g.R0 * p.Wo, de);
      }
      __syncthreads();
    }

    for (int t0 = 0; t0 < ntasks; t0 += NSEG) {
      const int task = t0 + seg;
      const int gi = task / p.NRB;
      const int rb = task - gi * p.NRB;
      const bool active = (task < ntasks) && (gi < g.gcount);
      const int r_begin = g.R0 + (rb * g.th) / p.NRB;
      const int r_end = (rb == p.NRB - 1) ? (g.R0 + g.th) : g.R0 + ((rb + 1) * g.th) / p.NRB;
      const T *splane = xs_s + (size_t)(active ? gi : 0) * p.XPL + j * VI;
      const T *dplane = ds_s + (size_t)(active ? gi : 0) * p.DPL + j * VO;

      float rows[Geo::KR][Geo::NIN];
      int ibase = r_begin * S + Geo::RMIN;
#pragma unroll
      for (int i = 0; i < Geo::KR - Geo::ADV; ++i) {
        const int ir = ibase + i;
        const bool ok = active && in_alive && ir >= g.in_lo && ir < g.in_hi;
        load_window_row<T, Geo, VI>(rows[i], splane + (size_t)(ir - g.in_lo) * p.W, ok, lane,
                                    halo_mask);
      }
      for (int rr = 0; rr < p.RBH; rr += U) {
        const int r = r_begin + rr;
#pragma unroll
        for (int i = Geo::KR - Geo::ADV; i < Geo::KR; ++i) {
          const int ir = ibase + i;
          const bool ok = active && in_alive && ir >= g.in_lo && ir < g.in_hi;
          load_window_row<T, Geo, VI>(rows[i], splane + (size_t)(ir - g.in_lo) * p.W, ok, lane,
                                      halo_mask);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float dyv[VO];
#pragma unroll
          for (int e = 0; e < VO; ++e) dyv[e] = 0.f;
          if (active && out_alive && (r + u) < r_end)
            VecIO<T, VO>::ld(dplane + (size_t)(r + u - g.R0) * p.Wo, dyv);
#pragma unroll
          for (int ty = 0; ty < K; ++ty) {
            const int ri = Geo::rel(u, ty) - Geo::RMIN;
#pragma unroll
            for (int tx = 0; tx < K; ++tx)
#pragma unroll
              for (int e = 0; e < VO; ++e)
                acc[ty][tx] = fmaf(dyv[e], rows[ri][Geo::rel(e, tx) - Geo::CMIN], acc[ty][tx]);
          }
        }
#pragma unroll
        for (int i = 0; i < Geo::KR - Geo::ADV; ++i)
#pragma unroll
          for (int ci = 0; ci < Geo::NIN; ++ci) rows[i][ci] = rows[i + Geo::ADV][ci];
        ibase += Geo::ADV;
      }
    }
    __syncthreads();
    if (*ring.abort_flag) break;
  }

  if (*ring.abort_flag) {
    if (threadIdx.x == 0)
      for (int s = 0; s < ROWS_STAGES; ++s)
        (void)mbar_wait_bounded(&ring.bar[s], (ring.phase >> s) & 1u);
    __syncthreads();
  }
  // every copy this CTA issued has landed: stage 0 is free to hold the cross-warp sums
  float *red = reinterpret_cast<float *>(ring.stage(0));
#pragma unroll
  for (int ty = 0; ty < K; ++ty)
#pragma unroll
    for (int tx = 0; tx < K; ++tx) {
      const float v = warp_sum(acc[ty][tx]);
      if (lane == 0) red[warp * (K * K) + ty * K + tx] = v;
    }
  __syncthreads();
  if (threadIdx.x < K * K) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < ROWS_WARPS; ++w) s += red[w * (K * K) + threadIdx.x];
    p.partial[((size_t)c * p.SL + slice) * (K * K) + threadIdx.x] = s;
  }
}

}  // namespace dwb
