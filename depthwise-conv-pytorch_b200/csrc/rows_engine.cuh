// "Rows" kernel family: the B200 path for filters 3x3 / 5x5 / 7x7, stride 1 or 2, "same"
// padding (p = k/2), fp32 and fp16, maps up to 128 columns wide.
//
// Structure shared by forward, backward-input and backward-filter:
//
//  * Persistent, warp-specialised CTAs: 7 consumer warps compute, 1 producer warp moves data.
//    A tile is a run of full-width rows of one plane, or a group of whole small planes that are
//    adjacent in memory; either way it is ONE contiguous byte range of the NCHW tensor, so the
//    producer brings it into shared memory with one bulk asynchronous copy (cp.async.bulk, the
//    TMA unit) that signals a "full" mbarrier; consumers hand a stage back through an "empty"
//    mbarrier.  The 96 KB ring has 3 stages of 32 KB or 2 of 48 KB (chosen per problem), so
//    tiles are in flight while one is computed.  The staged range keeps its source's phase
//    within 16 bytes, so the aligned interior of ANY range is a legal bulk copy; only ragged
//    heads and tails (< 16 bytes) are moved by a producer lane with plain loads.
//  * A tile is split into tasks (plane, block of output rows).  A task is executed by a
//    SEGMENT of a warp: LW = 8, 16 or 32 adjacent lanes.  Lane j owns VI adjacent input
//    columns and VO adjacent output columns.  It reads its own columns of an input row from
//    shared memory with one vector load and gets the k-1 halo columns from neighbouring lanes
//    by warp shuffle.  Rows above / below the map are read from 16 zero bytes kept in every
//    stage (an address select, no data-dependent branch); lanes beyond the map width read
//    those zeros too, which supplies the left / right padding when a segment has spare lanes
//    (otherwise halo values are masked).  Rows stream through a register window: each input
//    element is read from shared memory once per task.
//  * The filter taps of the tile's channels are consecutive in the filter tensor, so they are
//    staged with bulk copies too and held in registers during a task.  Every output has one
//    accumulator, taps are applied row-major with one FMA each: the summation order of the
//    reference kernels (torch_dwconv/dwconv_kernel.cu:164-172), hence bit-identical fp32.
//  * Outputs leave as VO-wide vector stores, contiguous across the segment.
//  * Backward-filter: a work item is (group of consecutive channels, slice of the image list);
//    a segment keeps its (channel, row block) and its K*K accumulators for the whole item; the
//    partial of every (channel, slice) has exactly one writer and a second kernel adds the
//    slices in order: deterministic, no atomics.
//
// All waits on mbarriers are bounded; on expiry the warp raises a flag the host can read
// (dwconv_b200_device_status), stops waiting and runs to the end of the kernel.
#pragma once

#include "common.cuh"
#include "rows_api.cuh"

namespace dwb {

enum { MODE_FWD = 0, MODE_BWD = 1 };

constexpr int ROWS_CWARPS = 7;                        // consumer warps
constexpr int ROWS_THREADS = (ROWS_CWARPS + 1) * 32;  // + 1 producer warp
// The 96 KB ring is cut into 3 stages of 32 KB or 2 stages of 48 KB, chosen per problem.
constexpr int ROWS_STAGES = 3;  // at most
constexpr int ROWS_RING_BYTES = 96 * 1024;
constexpr int ROWS_TAIL_BYTES = 8192;  // barriers, flags, cross-segment reduction scratch
constexpr int ROWS_SMEM_BYTES = ROWS_RING_BYTES + ROWS_TAIL_BYTES;
constexpr unsigned ROWS_WAIT_LIMIT = 1u << 15;   // mbarrier polls before giving up
constexpr unsigned ROWS_WAIT_HINT_NS = 100000;  // a poll may suspend the warp this long

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
// Orders this thread's earlier generic-proxy shared-memory accesses before later
// async-proxy (bulk copy) accesses to the same locations.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ROWS_WAIT_HINT_NS)
      : "memory");
  return ok != 0;
}
// Bounded wait; false if the phase did not complete within ROWS_WAIT_LIMIT polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
  for (unsigned i = 0; i < ROWS_WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Barrier among the consumer warps only (the producer warp never joins it).
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(ROWS_CWARPS * 32) : "memory");
}

// ---------------------------------------------------------------------------------------
// Compile-time geometry of one kernel variant.
//   FWD, stride S: out row r+u reads in rows (r+u)*S - P + ty; columns alike.
//   BWD, stride S: out (=dx) row r+u, r a multiple of S, reads in (=dy) row (r+u-P+ty)/S for the
//                  taps ty with (u-P+ty) divisible by S; taps are the flipped filter.
// "rel" values are relative to the chunk's base input row (r*S resp. r/S) and to the lane's
// first own input column (j*VI).
// ---------------------------------------------------------------------------------------
__host__ __device__ constexpr int geo_fdiv(int a, int b) {
  return a >= 0 ? a / b : -((-a + b - 1) / b);
}
__host__ __device__ constexpr bool geo_used(int K, int S, int mode, int u, int t) {
  return mode == MODE_FWD ? true : (((u - K / 2 + t) % S) + S) % S == 0;
}
__host__ __device__ constexpr int geo_rel(int K, int S, int mode, int u, int t) {
  return mode == MODE_FWD ? u * S - K / 2 + t : geo_fdiv(u - K / 2 + t, S);
}
__host__ __device__ constexpr int geo_min_rel(int K, int S, int mode, int n) {
  int m = 1 << 20;
  for (int u = 0; u < n; ++u)
    for (int t = 0; t < K; ++t)
      if (geo_used(K, S, mode, u, t) && geo_rel(K, S, mode, u, t) < m) m = geo_rel(K, S, mode, u, t);
  return m;
}
__host__ __device__ constexpr int geo_max_rel(int K, int S, int mode, int n) {
  int m = -(1 << 20);
  for (int u = 0; u < n; ++u)
    for (int t = 0; t < K; ++t)
      if (geo_used(K, S, mode, u, t) && geo_rel(K, S, mode, u, t) > m) m = geo_rel(K, S, mode, u, t);
  return m;
}

template <int K, int S, int MODE, int VI, int VO, int U>
struct RowsGeo {
  static constexpr int P = K / 2;
  static constexpr int fdiv(int a, int b) { return geo_fdiv(a, b); }
  static constexpr bool used(int u, int t) { return geo_used(K, S, MODE, u, t); }
  static constexpr int rel(int u, int t) { return geo_rel(K, S, MODE, u, t); }
  static constexpr int RMIN = geo_min_rel(K, S, MODE, U), RMAX = geo_max_rel(K, S, MODE, U);
  static constexpr int KR = RMAX - RMIN + 1;                    // window rows per chunk
  static constexpr int ADV = MODE == MODE_FWD ? U * S : U / S;  // input rows per chunk
  static constexpr int CMIN = geo_min_rel(K, S, MODE, VO), CMAX = geo_max_rel(K, S, MODE, VO);
  static constexpr int NIN = CMAX - CMIN + 1;  // window columns
  static_assert(MODE == MODE_FWD || (U % S == 0 && VO % S == 0), "BWD: U, VO multiples of S");
  static_assert(MODE == MODE_FWD ? VI == VO * S : VO == VI * S, "VI/VO inconsistent with stride");
  static_assert(KR > ADV, "window must overlap the next chunk");
};

// First / one-past-last input row a tile of output rows [R0, R0+th) reads, clipped to the map.
__host__ __device__ __forceinline__ void tile_in_rows(int K, int S, int mode, int R0, int th,
                                                      int Hin, int &lo, int &hi) {
  const int P = K / 2;
  int a, b;
  if (mode == MODE_FWD) {
    a = R0 * S - P;
    b = (R0 + th - 1) * S - P + K;
  } else {
    a = geo_fdiv(R0 - P, S);
    b = geo_fdiv(R0 + th - 1 - P + K - 1, S) + 1;
  }
  lo = a < 0 ? 0 : a;
  hi = b > Hin ? Hin : b;
  if (hi < lo) hi = lo;
}

// n / d for small operands (n * d < 2^32) by multiplication with inv = ceil(2^32 / d).
__host__ __device__ __forceinline__ uint32_t magic_of(int d) {
  return (uint32_t)((0x100000000ull + (unsigned)d - 1) / (unsigned)d);
}
// (d == 1 has no 32-bit magic: magic_of(1) wraps to 0, which stands for "divide by one".)
__device__ __forceinline__ int magic_div(int n, uint32_t inv) {
  return inv ? (int)__umulhi((uint32_t)n, inv) : n;
}

// Split of a tile's th output rows over NRB row blocks; starts on multiples of RS.
__host__ __device__ __forceinline__ void task_rows(int rb, int NRB, int R0, int th, int RS,
                                                   int &r_begin, int &r_end) {
  r_begin = R0 + ((rb * th) / NRB) / RS * RS;
  r_end = (rb == NRB - 1) ? (R0 + th) : R0 + (((rb + 1) * th) / NRB) / RS * RS;
}
// The same on the device, with the division by NRB done by multiplication.
template <int RS>
__device__ __forceinline__ void task_rows_fast(int rb, int NRB, uint32_t inv_nrb, int R0, int th,
                                               int &r_begin, int &r_end) {
  r_begin = R0 + magic_div(rb * th, inv_nrb) / RS * RS;
  r_end = (rb == NRB - 1) ? (R0 + th) : R0 + magic_div((rb + 1) * th, inv_nrb) / RS * RS;
}

struct RowsParams {
  const void *in;
  const void *w;
  void *out;
  int NC, C;
  int Hin, Win, Hout, Wout;
  int G;     // planes per tile (whole planes when NRT == 1)
  int NRT;   // row tiles per plane (G == 1 when > 1)
  int TH;    // output rows per row tile
  int NRB;   // row blocks (tasks) per plane inside a tile
  int RBH;   // row-loop trip count of a task, a multiple of U
  int LW;    // lanes per segment: 8, 16 or 32
  uint32_t inv_NRB;  // magic_of(NRB)
  int NST;   // stages in the ring: 3 (32 KB each) or 2 (48 KB each)
  int TAPB;  // bytes at the head of a stage that hold the taps of the tile's channels; 16 zero
             // bytes follow, then the tile's rows
  int ntiles;
  int flip;  // apply the filter flipped in both axes (backward-input)
  EpilogueArgs ep;  // forward with a fused epilogue (kernels compiled with EPI) only
};

// V elements from shared memory (32-bit shared address) into fp32 registers.
template <typename T, int V> struct SmemLd;
template <> struct SmemLd<float, 1> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[1]) {
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[0]) : "r"(a));
  }
};
template <> struct SmemLd<float, 2> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[2]) {
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(a));
  }
};
template <> struct SmemLd<float, 4> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[4]) {
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3])
                 : "r"(a));
  }
};
// 16-bit types (fp16, bf16): the same loads, converted through Pack16<T>.
template <typename T, int V> struct SmemLd16;
template <typename T> struct SmemLd16<T, 1> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[1]) {
    unsigned short h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(a));
    v[0] = Pack16<T>::from_bits(h);
  }
};
template <typename T> struct SmemLd16<T, 2> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[2]) {
    uint32_t r;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(r) : "r"(a));
    const float2 t = Pack16<T>::unpack(r);
    v[0] = t.x; v[1] = t.y;
  }
};
template <typename T> struct SmemLd16<T, 4> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[4]) {
    uint32_t r0, r1;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
    const float2 x = Pack16<T>::unpack(r0);
    const float2 y = Pack16<T>::unpack(r1);
    v[0] = x.x; v[1] = x.y; v[2] = y.x; v[3] = y.y;
  }
};
template <int V> struct SmemLd<__half, V> : SmemLd16<__half, V> {};
template <int V> struct SmemLd<__nv_bfloat16, V> : SmemLd16<__nv_bfloat16, V> {};

// V fp32 registers to global memory as one vector store of T.  The stores are streaming
// (evict-first): an output map is not read again by the kernel that writes it, and keeping it from
// displacing the input maps lets the next operator of a training step find x / dy still in L2.
template <typename T, int V> struct GmemSt;
template <> struct GmemSt<float, 1> {
  static __device__ __forceinline__ void st(float *p, const float (&v)[1]) { __stcs(p, v[0]); }
};
template <> struct GmemSt<float, 2> {
  static __device__ __forceinline__ void st(float *p, const float (&v)[2]) {
    __stcs(reinterpret_cast<float2 *>(p), make_float2(v[0], v[1]));
  }
};
template <> struct GmemSt<float, 4> {
  static __device__ __forceinline__ void st(float *p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <typename T, int V> struct GmemSt16;
template <typename T> struct GmemSt16<T, 1> {
  static __device__ __forceinline__ void st(T *p, const float (&v)[1]) {
    __stcs(reinterpret_cast<unsigned short *>(p), Pack16<T>::to_bits(v[0]));
  }
};
template <typename T> struct GmemSt16<T, 2> {
  static __device__ __forceinline__ void st(T *p, const float (&v)[2]) {
    __stcs(reinterpret_cast<unsigned int *>(p), Pack16<T>::pack(v[0], v[1]));
  }
};
template <typename T> struct GmemSt16<T, 4> {
  static __device__ __forceinline__ void st(T *p, const float (&v)[4]) {
    uint2 raw;
    raw.x = Pack16<T>::pack(v[0], v[1]);
    raw.y = Pack16<T>::pack(v[2], v[3]);
    __stcs(reinterpret_cast<uint2 *>(p), raw);
  }
};
template <int V> struct GmemSt<__half, V> : GmemSt16<__half, V> {};
template <int V> struct GmemSt<__nv_bfloat16, V> : GmemSt16<__nv_bfloat16, V> {};

// Shared-memory bookkeeping: stages, then full[], empty[] barriers, the abort flag and a
// scratch area for cross-warp sums.
struct RowsRing {
  unsigned char *base;
  uint64_t *full;
  uint64_t *empty;
  volatile int *abort_flag;
  float *scratch;  // (ROWS_TAIL_BYTES - 128) bytes
  int stage_bytes;
  __device__ __forceinline__ unsigned char *stage(int s) const { return base + s * stage_bytes; }
};

// Sets up the barriers and clears, in every stage, the 16 bytes at `zero_off` that stand in
// for rows outside the map (nothing else ever writes them).
__device__ __forceinline__ RowsRing rows_ring_init(unsigned char *smem, int zero_off, int nst) {
  RowsRing r;
  r.base = smem;
  r.stage_bytes = ROWS_RING_BYTES / nst;
  unsigned char *tail = smem + ROWS_RING_BYTES;
  r.full = reinterpret_cast<uint64_t *>(tail);
  r.empty = r.full + ROWS_STAGES;
  r.abort_flag = reinterpret_cast<volatile int *>(r.empty + ROWS_STAGES);
  r.scratch = reinterpret_cast<float *>(tail + 128);
  if (threadIdx.x < nst)
    *reinterpret_cast<uint4 *>(smem + threadIdx.x * r.stage_bytes + zero_off) =
        make_uint4(0u, 0u, 0u, 0u);
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < ROWS_STAGES; ++s) {
      mbar_init(&r.full[s], 1);             // the producer's arrive (+ the copies' bytes)
      mbar_init(&r.empty[s], ROWS_CWARPS);  // one arrive per consumer warp
    }
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

// Element offset at which a range starting at global address `src` is placed behind the
// 16-byte aligned start of its slot: the slot keeps the source's phase within 16 bytes, so that
// the interior of the range is a legal bulk copy whatever the source alignment.
template <typename T> __device__ __forceinline__ int slot_phase(const T *src) {
  return (int)((reinterpret_cast<uintptr_t>(src) & 15) / sizeof(T));
}

// One lane stages `n` elements from global `src` into a data area that starts at the 16-byte
// aligned shared address `dst16`; they land at dst16 + slot_phase(src).  The 16-byte aligned
// interior goes through the bulk-copy unit (completion on `bar`); the ragged head and tail
// (< 16 bytes each) are moved with plain loads.  Returns the bulk-copied bytes.
template <typename T>
__device__ __forceinline__ uint32_t stage_range(T *dst16, const T *src, int n, uint64_t *bar) {
  constexpr int EPB = 16 / (int)sizeof(T);  // elements per 16 bytes
  const int phase = slot_phase(src);
  T *dst = dst16 + phase;
  int head = (EPB - phase) & (EPB - 1);
  if (head > n) head = n;
  const int interior = (n - head) & ~(EPB - 1);
  const int tail = n - head - interior;
  if (interior > 0)
    bulk_copy_g2s(dst + head, src + head, (uint32_t)interior * (uint32_t)sizeof(T), bar);
  T hv[EPB], tv[EPB];
#pragma unroll
  for (int i = 0; i < EPB - 1; ++i) {
    hv[i] = (i < head) ? src[i] : Elem<T>::from_acc(0);
    tv[i] = (i < tail) ? src[head + interior + i] : Elem<T>::from_acc(0);
  }
#pragma unroll
  for (int i = 0; i < EPB - 1; ++i) {
    if (i < head) dst[i] = hv[i];
    if (i < tail) dst[head + interior + i] = tv[i];
  }
  return (uint32_t)interior * (uint32_t)sizeof(T);
}

// ---------------------------------------------------------------------------------------
// One chunk-row of the register window: own columns from shared memory, halo by shuffle.
// MASK: the segment has no spare zero lanes on its sides, halo values crossing the map edge
// must be masked explicitly.
// ---------------------------------------------------------------------------------------
// A window row is fetched in two steps so that a chunk can issue all its shared-memory loads
// back to back before the first dependent shuffle.
// Step 1: the lane's own VI columns.  `q` is the row's index inside the staged rows of the
// lane's plane; rows outside [0, lim) are the zero padding above / below the map and are read
// from the stage's zero bytes instead.
template <typename T, int VI>
__device__ __forceinline__ void load_own_row(float (&own)[VI], uint32_t &addr, const uint32_t pitch,
                                             int &q, const int lim, const uint32_t zaddr) {
  SmemLd<T, VI>::ld(((unsigned)q < (unsigned)lim) ? addr : zaddr, own);
  addr += pitch;
  q += 1;
}
// Step 2: the halo columns from the neighbouring lanes.
template <typename Geo, int VI, bool MASK>
__device__ __forceinline__ void build_window_row(float (&win)[Geo::NIN], const float (&own)[VI],
                                                 const int (&src_lane)[Geo::NIN],
                                                 const uint32_t (&halo_mask)[Geo::NIN]) {
#pragma unroll
  for (int ci = 0; ci < Geo::NIN; ++ci) {
    const int c = ci + Geo::CMIN;
    const int dl = Geo::fdiv(c, VI);
    const int el = c - dl * VI;
    if (dl == 0) {
      win[ci] = own[el];
    } else {
      uint32_t bits = __shfl_sync(0xffffffffu, __float_as_uint(own[el]), src_lane[ci]);
      if (MASK) bits &= halo_mask[ci];
      win[ci] = __uint_as_float(bits);
    }
  }
}

template <typename Geo, int VI>
__device__ __forceinline__ void make_lane_tables(int (&src_lane)[Geo::NIN],
                                                 uint32_t (&halo_mask)[Geo::NIN], int lane, int j,
                                                 int Win) {
#pragma unroll
  for (int ci = 0; ci < Geo::NIN; ++ci) {
    const int c = ci + Geo::CMIN;
    src_lane[ci] = (lane + Geo::fdiv(c, VI)) & 31;
    const int col = j * VI + c;
    halo_mask[ci] = (col >= 0 && col < Win) ? 0xffffffffu : 0u;
  }
}

// Geometry of one conv tile, identical on every thread.
struct ConvTile {
  int pg, R0, th, gcount, in_lo, in_hi;
};
template <int K, int S, int MODE>
__device__ __forceinline__ ConvTile conv_tile(const RowsParams &p, int tile) {
  ConvTile t;
  if (p.NRT == 1) {
    t.pg = tile;
    t.R0 = 0;
    t.th = p.Hout;
    t.in_lo = 0;
    t.in_hi = p.Hin;
  } else {
    t.pg = tile / p.NRT;
    const int rt = tile - t.pg * p.NRT;
    t.R0 = rt * p.TH;
    t.th = min(p.TH, p.Hout - t.R0);
    tile_in_rows(K, S, MODE, t.R0, t.th, p.Hin, t.in_lo, t.in_hi);
  }
  t.gcount = min(p.G, p.NC - t.pg * p.G);
  return t;
}

// Where the taps of a tile's channels sit in the stage.  Channels c_base .. c_base+count-1
// (mod C): range A = [c_base, min(C, c_base+count)), range B = the wrapped remainder [0, nB).
// Each range keeps its source's 16-byte phase; B starts on the next 16-byte boundary behind A.
struct TapLayout {
  int c_base, nA, nB;
  int phaseA, phaseB;  // elements
  int offB16;          // element offset of B's aligned start
  bool direct;         // false: count > C, the producer gathers taps[g*KK + t] with plain loads
};
template <typename T, int KK>
__device__ __forceinline__ TapLayout tap_layout(const T *gw, int first_plane, int count, int C) {
  constexpr int EPB = 16 / (int)sizeof(T);
  TapLayout l;
  l.c_base = first_plane % C;
  l.direct = count <= C;
  l.nA = min(count, C - l.c_base);
  l.nB = l.direct ? count - l.nA : 0;
  l.phaseA = slot_phase(gw + (size_t)l.c_base * KK);
  l.phaseB = slot_phase(gw);
  l.offB16 = (l.phaseA + l.nA * KK + EPB - 1) / EPB * EPB;
  return l;
}

// The producer warp of the forward / backward-input kernels: walks this CTA's tiles and brings
// each tile's rows and taps into the next free stage of the ring.
template <typename T, int K, int S, int MODE>
__device__ __forceinline__ void conv_producer(const RowsParams &p, const RowsRing &ring,
                                              int *__restrict__ error_flag) {
  constexpr int KK = K * K;
  const T *__restrict__ gin = static_cast<const T *>(p.in);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  const int lane = threadIdx.x & 31;
  const size_t plane_in = (size_t)p.Hin * p.Win;
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
    const ConvTile t = conv_tile<K, S, MODE>(p, tile);
    unsigned char *sb = ring.stage(stage);
    // the tile's rows are one contiguous range of the tensor: one bulk copy, issued first
    // so that the tap loads below overlap with it
    uint32_t tx = 0;
    if (lane == 0) {
      fence_proxy_async_smem();
      const int nrows = t.in_hi - t.in_lo;
      const int elems = (p.NRT == 1) ? t.gcount * (int)plane_in : nrows * p.Win;
      const T *src0 = gin + (size_t)t.pg * p.G * plane_in + (size_t)t.in_lo * p.Win;
      tx = stage_range(reinterpret_cast<T *>(sb + p.TAPB + 16), src0, elems, &ring.full[stage]);
    }
    // taps of the tile's channels: consecutive channels are one contiguous range of the
    // filter tensor (two when the group wraps past the last channel), so they are bulk
    // copies too, issued by lanes 1 and 2
    const TapLayout tl = tap_layout<T, KK>(gw, t.pg * p.G, t.gcount, p.C);
    T *staps = reinterpret_cast<T *>(sb);
    if (tl.direct) {
      if (lane == 1) {
        fence_proxy_async_smem();
        tx = stage_range(staps, gw + (size_t)tl.c_base * KK, tl.nA * KK, &ring.full[stage]);
      } else if (lane == 2 && tl.nB > 0) {
        fence_proxy_async_smem();
        tx = stage_range(staps + tl.offB16, gw, tl.nB * KK, &ring.full[stage]);
      }
    } else {
      // more planes in the tile than channels in the tensor: gather with plain loads
      for (int idx = lane; idx < t.gcount * KK; idx += 32) {
        const int g = idx / KK;
        staps[idx] = gw[(size_t)((tl.c_base + g) % p.C) * KK + (idx - g * KK)];
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
}

// ---------------------------------------------------------------------------------------
// forward / backward-input
// ---------------------------------------------------------------------------------------
// EXACT: every task of every tile has exactly RBH rows, so no per-row test guards the stores.
// EPI: the forward with a fused epilogue (scale, bias, activation on the accumulator).
template <typename T, int K, int S, int MODE, int VI, int VO, int U, bool MASK, bool EXACT, int MINB,
          bool EPI = false>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_conv_kernel(const RowsParams p, int *__restrict__ error_flag) {
  using Geo = RowsGeo<K, S, MODE, VI, VO, U>;
  constexpr int KK = K * K;
  extern __shared__ __align__(128) unsigned char rows_smem[];
  pdl_launch_dependents();  // the next kernel in the stream may take freed SMs early
  RowsRing ring = rows_ring_init(rows_smem, p.TAPB, p.NST);
  pdl_wait();  // everything earlier in the stream has completed; global memory may be touched

  const T *__restrict__ gin = static_cast<const T *>(p.in);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  T *__restrict__ gout = static_cast<T *>(p.out);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const size_t plane_in = (size_t)p.Hin * p.Win;
  const size_t plane_out = (size_t)p.Hout * p.Wout;

  if (warp == ROWS_CWARPS) {
    conv_producer<T, K, S, MODE>(p, ring, error_flag);
    return;
  }

  // ------------------------------- consumer warps -------------------------------
  const int LW = p.LW;
  const int segs_per_warp = 32 / LW;
  const int j = lane & (LW - 1);
  const int seg = warp * segs_per_warp + lane / LW;
  const int NSEG = ROWS_CWARPS * segs_per_warp;
  const bool in_alive = j * VI < p.Win;    // Win % VI == 0: a lane's block is all in or all out
  const bool out_alive = j * VO < p.Wout;  // Wout % VO == 0
  constexpr int RS = (MODE == MODE_BWD) ? S : 1;

  int src_lane[Geo::NIN];
  uint32_t halo_mask[Geo::NIN];
  make_lane_tables<Geo, VI>(src_lane, halo_mask, lane, j, p.Win);

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
    const ConvTile t = conv_tile<K, S, MODE>(p, tile);
    unsigned char *sb = ring.stage(stage);
    const T *staps = reinterpret_cast<const T *>(sb);
    const TapLayout tl = tap_layout<T, KK>(gw, t.pg * p.G, t.gcount, p.C);
    const uint32_t zaddr = smem_u32(sb + p.TAPB);  // 16 bytes that are always zero
    const int nrows = t.in_hi - t.in_lo;           // staged rows per plane
    const int phase =
        slot_phase(gin + (size_t)t.pg * p.G * plane_in + (size_t)t.in_lo * p.Win);
    const uint32_t sdata = zaddr + 16u + (uint32_t)(phase * (int)sizeof(T));

    for (int t0 = 0; t0 < ntasks; t0 += NSEG) {
      const int task = t0 + seg;
      const int g = magic_div(task, p.inv_NRB);
      const int rb = task - g * p.NRB;
      const bool active = (task < ntasks) && (g < t.gcount);
      const int plane = t.pg * p.G + (active ? g : 0);
      int r_begin, r_end;
      task_rows_fast<RS>(rb, p.NRB, p.inv_NRB, t.R0, t.th, r_begin, r_end);

      // The K*K taps live in registers for the task (backward-input reads them back to front).
      float taps[K][K];
      {
        const int cw = tl.c_base + g;
        const T *tp = staps;
        if (active) {
          tp = !tl.direct ? staps + g * KK
               : (cw < p.C) ? staps + tl.phaseA + g * KK
                            : staps + tl.offB16 + tl.phaseB + (cw - p.C) * KK;
        }
        const int t_first = p.flip ? KK - 1 : 0, t_step = p.flip ? -1 : 1;
#pragma unroll
        for (int ty = 0; ty < K; ++ty)
#pragma unroll
          for (int tx = 0; tx < K; ++tx)
            taps[ty][tx] = active ? Elem<T>::to_acc(tp[t_first + t_step * (ty * K + tx)]) : 0.f;
      }
      // row index (inside the plane's staged rows) of window row 0, its shared address, and the
      // row pitch; lanes with nothing to read have lim = 0 and only ever read the zero bytes
      int q = (MODE == MODE_FWD ? r_begin * S : r_begin / S) + Geo::RMIN - t.in_lo;
      int lim = 0;
      uint32_t a = zaddr;
      if (active && in_alive) {
        lim = nrows;
        a = sdata + (uint32_t)(((g * nrows + q) * p.Win + j * VI) * (int)sizeof(T));
      }
      T *orow = gout + (size_t)plane * plane_out + (size_t)r_begin * p.Wout + j * VO;
      const bool st_ok = active && out_alive;
      int rows_left = st_ok ? (r_end - r_begin) : 0;
      float ep_scale = 1.f, ep_bias = 0.f;
      if constexpr (EPI) epilogue_coeffs<T>(p.ep, plane % p.C, ep_scale, ep_bias);

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
        {
          float own[Geo::ADV][VI];
#pragma unroll
          for (int i = 0; i < Geo::ADV; ++i) load_own_row<T, VI>(own[i], a, row_bytes, q, lim, zaddr);
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
              const float tap = taps[ty][tx];
#pragma unroll
              for (int e = 0; e < VO; ++e) {
                if (!Geo::used(e, tx)) continue;
                acc[e] = fmaf(rows[ri][Geo::rel(e, tx) - Geo::CMIN], tap, acc[e]);
              }
            }
          }
          if constexpr (EPI) {
#pragma unroll
            for (int e = 0; e < VO; ++e) acc[e] = apply_epilogue<float>(acc[e], ep_scale, ep_bias, p.ep.act);
          }
          if (EXACT ? st_ok : (u < rows_left)) GmemSt<T, VO>::st(orow, acc);
          orow += p.Wout;
        }
#pragma unroll
        for (int i = 0; i < Geo::KR - Geo::ADV; ++i)
#pragma unroll
          for (int ci = 0; ci < Geo::NIN; ++ci) rows[i][ci] = rows[i + Geo::ADV][ci];
        if (!EXACT) rows_left -= U;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[stage]);  // this warp is done with the stage
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
  int G;      // consecutive channels (planes of one image) per tile; whole planes when NRT == 1
  int NRT;    // row tiles per plane (G == 1 when > 1)
  int TH;     // dy rows per row tile
  int NRB, RBH, LW;  // G * NRB <= segments per CTA: a segment keeps its (channel, row block)
  uint32_t inv_NRB;  // magic_of(NRB)
  int NST;    // stages in the ring: 3 (32 KB each) or 2 (48 KB each)
  int NCG;    // channel groups = ceil(C / G)
  int TPC;    // tiles per channel group = N * NRT
  int SL;     // work items (slices of that tile list) per channel group
  int DYOFF;  // byte offset of the dy rows inside a stage (16-byte aligned); the stage starts
              // with 16 zero bytes, the x rows follow
};

struct FilterTile {
  int n, R0, th, in_lo, in_hi;
};
template <int K, int S>
__device__ __forceinline__ FilterTile filter_tile(const RowsFilterParams &p, int tt) {
  FilterTile t;
  t.n = tt / p.NRT;
  const int rt = tt - t.n * p.NRT;
  t.R0 = rt * p.TH;
  t.th = min(p.TH, p.Ho - t.R0);
  if (p.NRT == 1) {
    t.in_lo = 0;
    t.in_hi = p.H;
  } else {
    tile_in_rows(K, S, MODE_FWD, t.R0, t.th, p.H, t.in_lo, t.in_hi);
  }
  return t;
}

// Persistent CTAs walk work items (group of G consecutive channels, slice of the (image, row
// tile) list).  A tile holds the x rows and dy rows of the group's planes in one image: two
// contiguous ranges, two bulk copies.  Segment s of the CTA owns (channel g, row block rb) =
// (s / NRB, s % NRB) for the whole item; lane layout as in the forward kernel (the x window is
// the forward window, dy the lane's VO own output columns).  Each lane keeps K*K accumulators
// over the item; at its end they are summed over the segment's lanes by shuffle, then over the
// channel's row blocks through shared memory in a fixed order, and written to the (channel,
// slice) slot of the partials (no atomics).  A second kernel adds a channel's slices in order.
// EXACT: every task of every tile has exactly RBH rows, so every row of the loop contributes
// and the inner loop has no branch (lanes without work multiply zeros).
template <typename T, int K, int S, int VI, int VO, int U, bool MASK, bool EXACT, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
rows_filter_kernel(const RowsFilterParams p, int *__restrict__ error_flag) {
  using Geo = RowsGeo<K, S, MODE_FWD, VI, VO, U>;
  constexpr int KK = K * K;
  extern __shared__ __align__(128) unsigned char rows_smem[];
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  RowsRing ring = rows_ring_init(rows_smem, 0, p.NST);
  pdl_wait();  // everything earlier in the stream has completed; global memory may be touched

  const T *__restrict__ gx = static_cast<const T *>(p.x);
  const T *__restrict__ gdy = static_cast<const T *>(p.dy);
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
        const FilterTile t = filter_tile<K, S>(p, tt);
        unsigned char *sb = ring.stage(stage);
        const size_t pl0 = (size_t)t.n * p.C + c0;
        uint32_t tx = 0;
        if (lane == 0) {
          fence_proxy_async_smem();
          const int xe = (p.NRT == 1) ? gcount * (int)plane_x : (t.in_hi - t.in_lo) * p.W;
          tx = stage_range(reinterpret_cast<T *>(sb + 16), gx + pl0 * plane_x + (size_t)t.in_lo * p.W,
                           xe, &ring.full[stage]);
        } else if (lane == 1) {
          fence_proxy_async_smem();
          const int de = (p.NRT == 1) ? gcount * (int)plane_dy : t.th * p.Wo;
          tx = stage_range(reinterpret_cast<T *>(sb + p.DYOFF),
                           gdy + pl0 * plane_dy + (size_t)t.R0 * p.Wo, de, &ring.full[stage]);
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
  const int LW = p.LW;
  const int segs_per_warp = 32 / LW;
  const int j = lane & (LW - 1);
  const int seg = warp * segs_per_warp + lane / LW;
  const bool in_alive = j * VI < p.W;
  const bool out_alive = j * VO < p.Wo;

  int src_lane[Geo::NIN];
  uint32_t halo_mask[Geo::NIN];
  make_lane_tables<Geo, VI>(src_lane, halo_mask, lane, j, p.W);

  const int ntasks = p.G * p.NRB;  // <= segments per CTA
  const int g = magic_div(seg, p.inv_NRB);  // this segment's channel within the group, row block
  const int rb = seg - g * p.NRB;
  const uint32_t row_bytes = (uint32_t)p.W * (uint32_t)sizeof(T);
  const uint32_t drow_bytes = (uint32_t)p.Wo * (uint32_t)sizeof(T);
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

    float acc[K][K];
#pragma unroll
    for (int ty = 0; ty < K; ++ty)
#pragma unroll
      for (int tx = 0; tx < K; ++tx) acc[ty][tx] = 0.f;

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
      const FilterTile t = filter_tile<K, S>(p, tt);
      unsigned char *sb = ring.stage(stage);
      const size_t pl0 = (size_t)t.n * p.C + c0;
      const uint32_t zaddr = smem_u32(sb);  // 16 bytes that are always zero
      const int nrows = t.in_hi - t.in_lo;
      const int xphase = slot_phase(gx + pl0 * plane_x + (size_t)t.in_lo * p.W);
      const int dphase = slot_phase(gdy + pl0 * plane_dy + (size_t)t.R0 * p.Wo);
      const int drows = (p.NRT == 1) ? p.Ho : t.th;  // staged dy rows per plane

      int r_begin, r_end;
      task_rows_fast<1>(rb, p.NRB, p.inv_NRB, t.R0, t.th, r_begin, r_end);
      int q = r_begin * S + Geo::RMIN - t.in_lo;
      int lim = 0;
      uint32_t a = zaddr;
      if (active && in_alive) {
        lim = nrows;
        a = zaddr + 16u + (uint32_t)((xphase + (g * nrows + q) * p.W + j * VI) * (int)sizeof(T));
      }
      const bool dy_ok = active && out_alive;
      uint32_t da = zaddr;
      uint32_t dpitch = 0;
      if (dy_ok) {
        da = smem_u32(sb + p.DYOFF) +
             (uint32_t)((dphase + (g * drows + (r_begin - t.R0)) * p.Wo + j * VO) * (int)sizeof(T));
        dpitch = drow_bytes;
      }
      int rows_left = dy_ok ? (r_end - r_begin) : 0;

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
        {
          float own[Geo::ADV][VI];
#pragma unroll
          for (int i = 0; i < Geo::ADV; ++i) load_own_row<T, VI>(own[i], a, row_bytes, q, lim, zaddr);
#pragma unroll
          for (int i = 0; i < Geo::ADV; ++i)
            build_window_row<Geo, VI, MASK>(rows[Geo::KR - Geo::ADV + i], own[i], src_lane, halo_mask);
        }
        float dys[U][VO];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          SmemLd<T, VO>::ld((EXACT || u < rows_left) ? da : zaddr, dys[u]);
          da += dpitch;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (EXACT || u < rows_left) {  // rows past the task's end must not contribute
            const float (&dyv)[VO] = dys[u];
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

    // item done: sum over the segment's lanes, then over the channel's row blocks
#pragma unroll
    for (int ty = 0; ty < K; ++ty)
#pragma unroll
      for (int tx = 0; tx < K; ++tx) {
        float v = acc[ty][tx];
        for (int off = LW >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (j == 0 && seg < ntasks) red[seg * KK + ty * K + tx] = v;
      }
    consumer_sync();
    for (int idx = threadIdx.x; idx < gcount * KK; idx += ROWS_CWARPS * 32) {
      const int gg = idx / KK;
      const int tap = idx - gg * KK;
      float s = 0.f;
      for (int b = 0; b < p.NRB; ++b) s += red[(gg * p.NRB + b) * KK + tap];
      p.partial[((size_t)(c0 + gg) * p.SL + slice) * KK + tap] = s;
    }
    consumer_sync();  // red is rewritten by the next item
  }
}

}  // namespace dwb
