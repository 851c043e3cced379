// "Direct" kernel family: one thread per output element, runtime filter extent.
// Serves every shape, stride, padding and dtype (fp32, fp16, fp64); the faster
// families fall back to it for what they do not cover.
#pragma once

#include "common.cuh"

namespace dwb {

// y[n,c,oy,ox] = sum_{ky,kx} x[n,c,oy*sh-ph+ky,ox*sw-pw+kx] * w[c,ky,kx].
// Taps are added ky-major / kx-minor into one accumulator (out-of-range taps add
// fma(0, w, acc)), the order of torch_dwconv/dwconv_kernel.cu:164-172.
template <typename T>
__global__ void __launch_bounds__(256)
direct_forward_kernel(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ y,
                      const Shape s, const long long total, const EpilogueArgs ep) {
  using A = typename Elem<T>::acc_t;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const int ox = (int)(idx % s.Wo);
    const long long t = idx / s.Wo;
    const int oy = (int)(t % s.Ho);
    const long long nc = t / s.Ho;
    const int c = (int)(nc % s.C);
    const T *xp = x + nc * (long long)s.H * s.W;
    const T *wp = w + (long long)c * s.kh * s.kw;
    const int iy0 = oy * s.sh - s.ph;
    const int ix0 = ox * s.sw - s.pw;
    A acc = 0;
    for (int ky = 0; ky < s.kh; ++ky) {
      const int iy = iy0 + ky;
      const bool yok = (iy >= 0) & (iy < s.H);
      for (int kx = 0; kx < s.kw; ++kx) {
        const int ix = ix0 + kx;
        A v = 0;
        if (yok & (ix >= 0) & (ix < s.W)) v = Elem<T>::ld(xp + (long long)iy * s.W + ix);
        acc = fma_acc(v, Elem<T>::ld(wp + ky * s.kw + kx), acc);
      }
    }
    if (ep.on) {
      A sc, bi;
      epilogue_coeffs<T>(ep, c, sc, bi);
      acc = apply_epilogue<A>(acc, sc, bi, ep.act);
    }
    y[idx] = Elem<T>::from_acc(acc);
  }
}

// dx[n,c,iy,ix] = sum over taps with (iy+ph-ky) % sh == 0, (ix+pw-kx) % sw == 0 of
// dy[n,c,(iy+ph-ky)/sh,(ix+pw-kx)/sw] * w[c,ky,kx], visiting ky and kx in
// DESCENDING order: the order in which the reference's flipped-filter
// correlation meets them (torch_dwconv/dwconv_kernel.cu:107-114,164-172).
template <typename T>
__global__ void __launch_bounds__(256)
direct_backward_input_kernel(const T *__restrict__ dy, const T *__restrict__ w,
                             T *__restrict__ dx, const Shape s, const long long total) {
  using A = typename Elem<T>::acc_t;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const int ix = (int)(idx % s.W);
    const long long t = idx / s.W;
    const int iy = (int)(t % s.H);
    const long long nc = t / s.H;
    const int c = (int)(nc % s.C);
    const T *gp = dy + nc * (long long)s.Ho * s.Wo;
    const T *wp = w + (long long)c * s.kh * s.kw;
    A acc = 0;
    for (int ky = s.kh - 1; ky >= 0; --ky) {
      const int ny = iy + s.ph - ky;
      if (ny < 0) continue;
      const int oy = ny / s.sh;
      if (oy * s.sh != ny || oy >= s.Ho) continue;
      for (int kx = s.kw - 1; kx >= 0; --kx) {
        const int nx = ix + s.pw - kx;
        if (nx < 0) continue;
        const int ox = nx / s.sw;
        if (ox * s.sw != nx || ox >= s.Wo) continue;
        acc = fma_acc(Elem<T>::ld(gp + (long long)oy * s.Wo + ox),
                      Elem<T>::ld(wp + ky * s.kw + kx), acc);
      }
    }
    dx[idx] = Elem<T>::from_acc(acc);
  }
}

// Backward-filter, first pass.  Block (c, slice) owns the images
// [slice*N/S, (slice+1)*N/S) of channel c; warp `wid` owns taps wid, wid+nwarps, ...
// and writes partial[(c*S + slice)*kh*kw + tap], the sum over its images of
// dy[oy,ox] * x[oy*sh-ph+ky, ox*sw-pw+kx].  No atomics: every partial has one writer.
template <typename T>
__global__ void __launch_bounds__(256)
direct_backward_filter_partial_kernel(const T *__restrict__ x, const T *__restrict__ dy,
                                      typename Elem<T>::acc_t *__restrict__ partial,
                                      const Shape s, const int S) {
  using A = typename Elem<T>::acc_t;
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  const int c = blockIdx.x / S;
  const int slice = blockIdx.x - c * S;
  const int n0 = (int)((long long)slice * s.N / S);
  const int n1 = (int)((long long)(slice + 1) * s.N / S);
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int kk = s.kh * s.kw;
  const int npix = s.Ho * s.Wo;
  for (int tap = wid; tap < kk; tap += nwarps) {
    const int ky = tap / s.kw;
    const int kx = tap - ky * s.kw;
    A acc = 0;
    for (int n = n0; n < n1; ++n) {
      const T *xp = x + ((long long)n * s.C + c) * (long long)s.H * s.W;
      const T *gp = dy + ((long long)n * s.C + c) * (long long)npix;
      for (int pix = lane; pix < npix; pix += 32) {
        const int oy = pix / s.Wo;
        const int ox = pix - oy * s.Wo;
        const int iy = oy * s.sh - s.ph + ky;
        const int ix = ox * s.sw - s.pw + kx;
        if ((iy >= 0) & (iy < s.H) & (ix >= 0) & (ix < s.W))
          acc = fma_acc(Elem<T>::ld(gp + pix), Elem<T>::ld(xp + (long long)iy * s.W + ix), acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) partial[((long long)c * S + slice) * kk + tap] = acc;
  }
}

// Backward-filter, second pass: dw[c,tap] = sum over the S slices of partial[c,sl,tap].
// A warp owns 32 consecutive outputs (coalesced reads of every slice); the block's 8 warps take
// the slices sl = part, part + 8, ... of the same 32 outputs, each adding in ascending order, and
// the 8 part sums are added in part order.  The order is fixed, so the result does not depend on
// scheduling; eight short chains instead of one long one keep the pass from being latency-bound.
constexpr int FINALIZE_OUTPUTS = 32;  // per block
constexpr int FINALIZE_PARTS = 8;

// The sum of output idx's S partial values, in the fixed order described above; valid in the
// threads with part == 0.  Every thread of the block must call it (it synchronises).
template <typename A>
__device__ __forceinline__ A finalize_sum(const A *__restrict__ partial, const int idx, const bool live,
                                          const int kk, const int S,
                                          A (&part_sum)[FINALIZE_PARTS][FINALIZE_OUTPUTS]) {
  const int o = threadIdx.x & (FINALIZE_OUTPUTS - 1);
  const int part = threadIdx.x / FINALIZE_OUTPUTS;
  A acc = 0;
  if (live) {
    const int c = idx / kk;
    const int tap = idx - c * kk;
    const A *src = partial + (long long)c * S * kk + tap;
#pragma unroll 4
    for (int sl = part; sl < S; sl += FINALIZE_PARTS) acc += src[(long long)sl * kk];
  }
  part_sum[part][o] = acc;
  __syncthreads();
  A total = part_sum[0][o];
#pragma unroll
  for (int q = 1; q < FINALIZE_PARTS; ++q) total += part_sum[q][o];
  return total;
}

template <typename T>
__global__ void __launch_bounds__(FINALIZE_OUTPUTS * FINALIZE_PARTS)
backward_filter_finalize_kernel(const typename Elem<T>::acc_t *__restrict__ partial,
                                T *__restrict__ dw, const int C, const int kk, const int S) {
  using A = typename Elem<T>::acc_t;
  __shared__ A part_sum[FINALIZE_PARTS][FINALIZE_OUTPUTS];
  const int idx = blockIdx.x * FINALIZE_OUTPUTS + (threadIdx.x & (FINALIZE_OUTPUTS - 1));
  const bool live = idx < C * kk;
  pdl_launch_dependents();  // the next kernel in the stream may take its place early
  pdl_wait();  // the first pass has finished and its partial sums are visible
  const A total = finalize_sum<A>(partial, idx, live, kk, S, part_sum);
  if (threadIdx.x < FINALIZE_OUTPUTS && live) dw[idx] = Elem<T>::from_acc(total);
}

// The same second pass writing to an accumulator-typed gradient (fp32; fp64 for fp64 data):
// dw_acc = total, or dw_acc += total when `accumulate` is set.  For callers that sum the
// gradient over several calls (a batch processed in chunks) without a pass of their own.
template <typename A>
__global__ void __launch_bounds__(FINALIZE_OUTPUTS * FINALIZE_PARTS)
backward_filter_finalize_acc_kernel(const A *__restrict__ partial, A *__restrict__ dw_acc,
                                    const int C, const int kk, const int S, const int accumulate) {
  __shared__ A part_sum[FINALIZE_PARTS][FINALIZE_OUTPUTS];
  const int idx = blockIdx.x * FINALIZE_OUTPUTS + (threadIdx.x & (FINALIZE_OUTPUTS - 1));
  const bool live = idx < C * kk;
  pdl_launch_dependents();
  pdl_wait();
  const A total = finalize_sum<A>(partial, idx, live, kk, S, part_sum);
  if (threadIdx.x < FINALIZE_OUTPUTS && live) dw_acc[idx] = accumulate ? dw_acc[idx] + total : total;
}

// Launch geometry of the second pass.
inline int finalize_blocks(int C, int kk) { return ceil_div(C * kk, FINALIZE_OUTPUTS); }
constexpr int FINALIZE_THREADS = FINALIZE_OUTPUTS * FINALIZE_PARTS;

}  // namespace dwb
