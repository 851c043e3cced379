// Fused backward for SMALL maps (7, 14 or 28 columns wide), stride 1, padding k/2, fp32 and fp16:
// "a lane owns a row".
//
// rows_backward_kernel gives a lane a few columns of a row and fetches the halo columns from
// its neighbours by shuffle; on maps this narrow the shuffles, the per-row address selects and
// the per-task set-up outweigh the multiply-adds (profiled: FFMA is 20-36 % of the issued
// instructions).  Here a lane owns a whole row of W columns (W is a template parameter, so
// every column index and every tap that falls off the map edge is resolved at compile time):
//
//   * no shuffles: the K dy rows a dx row needs are read from shared memory by the lane itself
//     (rows above / below the plane come from a block of zero bytes), one row at a time, each
//     used at once for dx (tap row ty, all columns) and for the K filter-gradient sums of that
//     tap row, then dropped: registers hold one dy row, the x row, the dx row, K*K taps and
//     K*K gradient sums;
//   * consumer lane L of the CTA owns row L of the tile (planes * rows, plane-major): with
//     14-row planes the 224 consumer lanes hold exactly 16 planes;
//   * the dx rows are written to a staging area in shared memory laid out like the tensor, and
//     the whole tile (one contiguous byte range of dx) leaves with ONE bulk asynchronous store
//     (cp.async.bulk shared -> global), issued by one elected lane after the consumer warps have
//     met; the staging area of a stage is reused only after that store has read it.
//
// Work decomposition, producer, ring, bounded waits and the two-pass deterministic reduction of
// the filter gradient are those of rows_backward_kernel.  dx: taps applied ty-major / tx-minor
// into one accumulator per output with one FMA per tap that lies inside the map (the products
// with padding zeros, which leave the sum unchanged, are not issued), so the bits equal the
// other kernels' and the reference's (torch_dwconv/dwconv_kernel.cu:164-172).
#pragma once

#include "rows_backward.cuh"

namespace dwb {

constexpr int LANEROW_ZERO_BYTES = 128;  // >= one row of zeros (W <= 32 fp32 columns)

struct LaneRowParams {
  const void *x;
  const void *dy;
  const void *w;
  void *dx;
  float *partial;  // [C][SL][K*K]
  int N, C, H;     // map height (the width is a template parameter)
  int G;           // planes (consecutive channels of one image) per tile: G * H <= consumer lanes
  int NST;         // stages in the ring
  int NCG;         // channel groups = ceil(C / G)
  int SL;          // work items (slices of the image list) per channel group
  int DYOFF, XOFF, OUTOFF;  // byte offsets inside a stage (16-byte aligned); the stage starts
                            // with LANEROW_ZERO_BYTES zero bytes
  void *dw_direct;  // not null: one item per CTA, SL CTAs per cluster, dW written here (see
                    // cluster_finalize in rows_backward.cuh); `partial` is then unused
};

__device__ __forceinline__ void bulk_store_s2g(void *dst, const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk-store groups still have to READ their source.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One lane stores `n` elements that sit at src16 + slot_phase(dst) in shared memory to global
// `dst`: the 16-byte aligned interior as one bulk store (committed as a group), ragged head and
// tail (< 16 bytes each) with plain stores.
template <typename T>
__device__ __forceinline__ void store_range(T *dst, const T *src16, int n) {
  constexpr int EPB = 16 / (int)sizeof(T);
  const int phase = slot_phase(dst);
  const T *src = src16 + phase;
  int head = (EPB - phase) & (EPB - 1);
  if (head > n) head = n;
  const int interior = (n - head) & ~(EPB - 1);
  const int tail = n - head - interior;
  if (interior > 0) bulk_store_s2g(dst + head, src + head, (uint32_t)interior * (uint32_t)sizeof(T));
  bulk_commit();
  for (int i = 0; i < head; ++i) dst[i] = src[i];
  for (int i = 0; i < tail; ++i) dst[head + interior + i] = src[head + interior + i];
}

// A row of W elements of T between shared memory and fp32 registers.  Rows start on a multiple
// of their own length in bytes behind a 16-byte aligned base, so they are 8-byte aligned when that
// length is a multiple of 8, else 4-byte aligned (W even) or element aligned.
template <typename T, int W> struct RowIO;
template <int W> struct RowIO<float, W> {
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[W]) {
    if constexpr (W % 2 == 0) {
#pragma unroll
      for (int i = 0; i < W / 2; ++i)
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v[2 * i]), "=f"(v[2 * i + 1]) : "r"(a + 8u * i));
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[i]) : "r"(a + 4u * i));
    }
  }
  static __device__ __forceinline__ void st(uint32_t a, const float (&v)[W]) {
    if constexpr (W % 2 == 0) {
#pragma unroll
      for (int i = 0; i < W / 2; ++i)
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(a + 8u * i), "f"(v[2 * i]), "f"(v[2 * i + 1]) : "memory");
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i) asm volatile("st.shared.f32 [%0], %1;" ::"r"(a + 4u * i), "f"(v[i]) : "memory");
    }
  }
};
// 16-bit types (fp16, bf16), converted through Pack16<T>.
template <typename T, int W> struct RowIO16 {
  static __device__ __forceinline__ float2 unpack(uint32_t r) { return Pack16<T>::unpack(r); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) { return Pack16<T>::pack(a, b); }
  static __device__ __forceinline__ void ld(uint32_t a, float (&v)[W]) {
    if constexpr (W % 4 == 0) {  // rows of a multiple of 8 bytes
#pragma unroll
      for (int i = 0; i < W / 4; ++i) {
        uint32_t r0, r1;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a + 8u * i));
        const float2 x = unpack(r0), y = unpack(r1);
        v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = y.x; v[4 * i + 3] = y.y;
      }
    } else if constexpr (W % 2 == 0) {
#pragma unroll
      for (int i = 0; i < W / 2; ++i) {
        uint32_t r0;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(r0) : "r"(a + 4u * i));
        const float2 x = unpack(r0);
        v[2 * i] = x.x; v[2 * i + 1] = x.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i) {
        unsigned short h;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(a + 2u * i));
        v[i] = Pack16<T>::from_bits(h);
      }
    }
  }
  static __device__ __forceinline__ void st(uint32_t a, const float (&v)[W]) {
    if constexpr (W % 4 == 0) {
#pragma unroll
      for (int i = 0; i < W / 4; ++i)
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a + 8u * i), "r"(pack(v[4 * i], v[4 * i + 1])),
                     "r"(pack(v[4 * i + 2], v[4 * i + 3]))
                     : "memory");
    } else if constexpr (W % 2 == 0) {
#pragma unroll
      for (int i = 0; i < W / 2; ++i)
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(a + 4u * i), "r"(pack(v[2 * i], v[2 * i + 1])) : "memory");
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i)
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(a + 2u * i), "h"(Pack16<T>::to_bits(v[i]))
                     : "memory");
    }
  }
};

template <int W> struct RowIO<__half, W> : RowIO16<__half, W> {};
template <int W> struct RowIO<__nv_bfloat16, W> : RowIO16<__nv_bfloat16, W> {};

template <typename T, int K, int W, int MINB>
__global__ void __launch_bounds__(ROWS_THREADS, MINB)
lanerow_backward_kernel(const LaneRowParams p, int *__restrict__ error_flag) {
  constexpr int KK = K * K;
  constexpr int P = K / 2;
  constexpr int ES = (int)sizeof(T);
  constexpr uint32_t ROWB = W * ES;
  static_assert(ROWB <= LANEROW_ZERO_BYTES, "a row of zeros must fit the zero block");
  extern __shared__ __align__(128) unsigned char rows_smem[];
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  RowsRing ring = rows_ring_init(rows_smem, 0, p.NST);
  // rows_ring_init clears 16 bytes per stage; the zero block here is longer
  if (threadIdx.x < p.NST * (LANEROW_ZERO_BYTES / 16))
    *reinterpret_cast<uint4 *>(rows_smem + (threadIdx.x / (LANEROW_ZERO_BYTES / 16)) * ring.stage_bytes +
                               (threadIdx.x % (LANEROW_ZERO_BYTES / 16)) * 16) = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  pdl_wait();  // everything earlier in the stream has completed; global memory may be touched

  const T *__restrict__ gx = static_cast<const T *>(p.x);
  const T *__restrict__ gdy = static_cast<const T *>(p.dy);
  const T *__restrict__ gw = static_cast<const T *>(p.w);
  T *__restrict__ gdx = static_cast<T *>(p.dx);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int plane_elems = p.H * W;
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
      const int n_begin = (int)(((long long)slice * p.N) / p.SL);
      const int n_end = (int)(((long long)(slice + 1) * p.N) / p.SL);
      for (int n = n_begin; n < n_end; ++n) {
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
          tx = stage_range(reinterpret_cast<T *>(sb + p.DYOFF), gdy + pl0 * plane_elems,
                           gcount * plane_elems, &ring.full[stage]);
        } else if (lane == 1) {
          fence_proxy_async_smem();
          tx = stage_range(reinterpret_cast<T *>(sb + p.XOFF), gx + pl0 * plane_elems,
                           gcount * plane_elems, &ring.full[stage]);
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
  const int L = warp * 32 + lane;       // this lane's row of the tile (plane-major)
  const int g = L / p.H;                // plane inside the tile
  const int r = L - g * p.H;            // row inside the plane
  const bool elected = (L == 0);
  float *red = ring.scratch;            // [consumer lanes][K] at a time
  bool aborted = false;
  int stage = -1, use = 0;
  for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
    const int cg = item / p.SL;
    const int slice = item - cg * p.SL;
    const int c0 = cg * p.G;
    const int gcount = min(p.G, p.C - c0);
    const int n_begin = (int)(((long long)slice * p.N) / p.SL);
    const int n_end = (int)(((long long)(slice + 1) * p.N) / p.SL);
    const bool active = g < gcount;

    // the channel's taps, flipped in both axes, for the whole item
    float taps[K][K];
    {
      const T *tp = gw + (size_t)(c0 + (active ? g : 0)) * KK;
#pragma unroll
      for (int ty = 0; ty < K; ++ty)
#pragma unroll
        for (int tx = 0; tx < K; ++tx) taps[ty][tx] = active ? Elem<T>::ld(tp + (KK - 1 - (ty * K + tx))) : 0.f;
    }
    float dwacc[K][K];
#pragma unroll
    for (int ty = 0; ty < K; ++ty)
#pragma unroll
      for (int tx = 0; tx < K; ++tx) dwacc[ty][tx] = 0.f;

    for (int n = n_begin; n < n_end; ++n) {
      if (++stage == p.NST) {
        stage = 0;
        ++use;
      }
      if (!aborted && (*ring.abort_flag || !mbar_wait_bounded(&ring.full[stage], use & 1))) {
        aborted = true;
        *ring.abort_flag = 1;
        atomicExch(error_flag, 2);
      }
      if (!aborted) {
        unsigned char *sb = ring.stage(stage);
        const size_t pl0 = (size_t)n * p.C + c0;
        const uint32_t zaddr = smem_u32(sb);
        const int dphase = slot_phase(gdy + pl0 * plane_elems);
        const int xphase = slot_phase(gx + pl0 * plane_elems);
        const int ophase = slot_phase(gdx + pl0 * plane_elems);
        const uint32_t dybase = smem_u32(sb + p.DYOFF) + (uint32_t)((dphase + g * plane_elems) * ES);
        float xr[W], acc[W];
        RowIO<T, W>::ld(active ? smem_u32(sb + p.XOFF) + (uint32_t)((xphase + g * plane_elems + r * W) * ES) : zaddr, xr);
#pragma unroll
        for (int c = 0; c < W; ++c) acc[c] = 0.f;
#pragma unroll
        for (int ty = 0; ty < K; ++ty) {
          const int rr = r - P + ty;  // dy row under tap row ty
          float d[W];
          RowIO<T, W>::ld((active && (unsigned)rr < (unsigned)p.H) ? dybase + (uint32_t)rr * ROWB : zaddr, d);
#pragma unroll
          for (int tx = 0; tx < K; ++tx) {
#pragma unroll
            for (int c = 0; c < W; ++c) {
              const int cc = c - P + tx;  // dy column under tap column tx
              if (cc < 0 || cc >= W) continue;  // off the map: a zero that adds nothing
              acc[c] = fmaf(d[cc], taps[ty][tx], acc[c]);
              dwacc[ty][tx] = fmaf(d[cc], xr[c], dwacc[ty][tx]);
            }
          }
        }
        if (active)
          RowIO<T, W>::st(smem_u32(sb + p.OUTOFF) + (uint32_t)((ophase + g * plane_elems + r * W) * ES), acc);
        fence_proxy_async_smem();  // the rows just written are read by the bulk store below
        __syncwarp();
        if (lane == 0) mbar_arrive(&ring.empty[stage]);  // dy and x of this stage are consumed
      }
      // The elected lane makes sure the staging area the NEXT tile will write is free (its store,
      // NST tiles ago, has read it), then everybody meets: after the barrier this tile's dx rows
      // are all in the staging area and the next one's is free.
      if (elected) {
        if (p.NST == 2)
          bulk_wait_read<0>();
        else
          bulk_wait_read<1>();
      }
      consumer_sync();
      if (elected && !aborted) {
        unsigned char *sb = ring.stage(stage);
        const size_t pl0 = (size_t)n * p.C + c0;
        store_range(gdx + pl0 * plane_elems, reinterpret_cast<const T *>(sb + p.OUTOFF),
                    gcount * plane_elems);
      }
    }

    // item done: per channel, the rows' sums are added in row order, one tap row at a time.
    // Direct mode: the sums stay in shared memory (the dy area of the first stage: this CTA's
    // only item is done, and the bulk stores still in flight read the staging areas only).
    float *fin = reinterpret_cast<float *>(ring.stage(0) + p.DYOFF);
#pragma unroll
    for (int ty = 0; ty < K; ++ty) {
      consumer_sync();  // the previous tap row's readers are done with `red`
#pragma unroll
      for (int tx = 0; tx < K; ++tx) red[L * K + tx] = dwacc[ty][tx];
      consumer_sync();
      for (int idx = threadIdx.x; idx < gcount * K; idx += ROWS_CWARPS * 32) {
        const int gg = idx / K;
        const int tx = idx - gg * K;
        float s = 0.f;
        for (int rr = 0; rr < p.H; ++rr) s += red[(gg * p.H + rr) * K + tx];
        // window position (ty, tx) is the gradient of tap (K-1-ty, K-1-tx)
        const int tap = KK - 1 - (ty * K + tx);
        if (p.dw_direct != nullptr)
          fin[gg * KK + tap] = s;
        else
          p.partial[((size_t)(c0 + gg) * p.SL + slice) * KK + tap] = s;
      }
    }
    if (p.dw_direct != nullptr) {
      consumer_sync();  // fin is complete
      cluster_finalize<T>(fin, gcount * KK, static_cast<T *>(p.dw_direct) + (size_t)c0 * KK, p.SL, true);
    }
  }
  if (elected) bulk_wait_all();  // every dx tile has left shared memory and reached global memory
}

}  // namespace dwb
