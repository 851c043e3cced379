// Channels-last (NHWC) kernels: x[n][h][w][c], the layout PyTorch calls torch.channels_last.
//
// The reference makes every operand contiguous NCHW before it runs
// (torch_dwconv/dwconv_kernel.cu:741-742,855-856,1023-1024), which costs a channels-last caller
// a full extra read and write of each map.  These kernels read and write NHWC directly.
//
// Depthwise convolution in NHWC has the channel as the unit-stride axis, so a warp takes 32
// consecutive channels (lane = channel: every global access of a warp is one 128-byte line)
// and a CTA takes a spatial tile of R rows x TW columns of outputs for those 32 channels: the input tile
// with its halo is copied to shared memory as [row][column][channel] (zeros outside the map:
// the padding), a thread owns (channel, output column) and a strip of R output rows, walks the
// strip's input rows once and reads the K values under its column of each row (consecutive
// lanes read consecutive words: no bank conflicts).  Taps are applied ky-major / kx-minor into
// one accumulator per output with one fused multiply-add each, so results are bit-identical to
// the NCHW kernels on the same values.  3x3 / 5x5 / 7x7, stride 1 or 2, any padding,
// fp32 / fp16 / bf16.
#pragma once

#include "common.cuh"

namespace dwb {

constexpr int NHWC_CB = 32;  // channels per CTA: one lane each

// Output rows per tile (= per thread).  The filter-gradient kernel stages a dy tile beside the x
// tile, so its 7x7 stride-1 variant takes shorter tiles to stay inside 48 KB of shared memory.
constexpr int nhwc_rows(int K, int S, bool filter) { return S == 2 ? 4 : (filter && K == 7) ? 4 : 8; }

template <int K, int S, bool FILTER = false> struct NhwcGeo {
  static constexpr int TW = S == 1 ? 16 : 8;      // output columns per tile = warps per CTA
  static constexpr int R = nhwc_rows(K, S, FILTER);
  static constexpr int THREADS = NHWC_CB * TW;
  static constexpr int IH = (R - 1) * S + K;      // input rows per tile
  static constexpr int IW = (TW - 1) * S + K;     // input columns per tile
};

struct NhwcParams {
  int N, C;
  int Hin, Win, Hout, Wout;
  int pt, pl;   // rows / columns of zero padding above / left of the input
  int flip;     // apply the filter flipped in both axes (backward-input)
  int tiles_x, tiles_y, cblocks;
  long long ntiles;
  EpilogueArgs ep;
};

// Copies the input tile (IH x IW pixels x 32 channels from channel c0) whose first pixel is
// (gy0, gx0) of image `img` into shared memory; a warp moves one pixel's 32 channels at a time.
// UP > 1: (gy, gx) address the map up-sampled by UP with zeros in between.
template <typename T, int IH, int IW, int NWARPS, int UP>
__device__ __forceinline__ void nhwc_stage(float *sm, const T *__restrict__ img, int Hin, int Win, int C,
                                           int c0, int gy0, int gx0) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const bool c_ok = c0 + lane < C;
  constexpr int TOTAL = IH * IW;
  constexpr int UNROLL = 4;
  for (int base = wid; base < TOTAL; base += NWARPS * UNROLL) {
    float v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int pix = base + u * NWARPS;
      const int iy = pix / IW, ix = pix - iy * IW;
      const int gy = gy0 + iy, gx = gx0 + ix;
      int sy = gy, sx = gx;
      bool ok = pix < TOTAL && c_ok && gy >= 0 && gx >= 0;
      if (UP > 1) {
        sy = gy / UP;
        sx = gx / UP;
        ok = ok && sy * UP == gy && sx * UP == gx;
      }
      ok = ok && sy < Hin && sx < Win;
      v[u] = ok ? Elem<T>::ld(img + ((size_t)sy * Win + sx) * C + c0 + lane) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int pix = base + u * NWARPS;
      if (pix < TOTAL) sm[pix * NHWC_CB + lane] = v[u];
    }
  }
}

// out[n][oy][ox][c] = sum over (ky, kx) of in[n][oy*S - pt + ky][ox*S - pl + kx][c] * tap[c][ky][kx],
// `in` being the map up-sampled by UP (backward-input at stride 2: S = 1, UP = 2, flipped taps).
template <typename T, int K, int S, int UP>
__global__ void __launch_bounds__(NhwcGeo<K, S>::THREADS)
nhwc_conv_kernel(const T *__restrict__ in, const T *__restrict__ w, T *__restrict__ out,
                 const NhwcParams p) {
  using G = NhwcGeo<K, S>;
  constexpr int KK = K * K;
  __shared__ float sm[G::IH * G::IW * NHWC_CB];
  const int lane = threadIdx.x & 31;
  const int col = threadIdx.x >> 5;  // output column inside the tile
  const int per_img = p.tiles_x * p.tiles_y * p.cblocks;
  for (long long tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
    const int n = (int)(tile / per_img);
    int rest = (int)(tile - (long long)n * per_img);
    const int cb = rest % p.cblocks;  // channel blocks innermost: neighbours share input lines
    rest /= p.cblocks;
    const int ty = rest / p.tiles_x, tx = rest - ty * p.tiles_x;
    const int y0 = ty * G::R, x0 = tx * G::TW, c0 = cb * NHWC_CB;
    const int c = c0 + lane;
    __syncthreads();
    nhwc_stage<T, G::IH, G::IW, G::TW, UP>(sm, in + (size_t)n * p.Hin * p.Win * p.C, p.Hin, p.Win, p.C, c0,
                                           y0 * S - p.pt, x0 * S - p.pl);
    float tap[K][K];
#pragma unroll
    for (int ky = 0; ky < K; ++ky)
#pragma unroll
      for (int kx = 0; kx < K; ++kx)
        tap[ky][kx] = c < p.C ? Elem<T>::ld(w + (size_t)c * KK + (p.flip ? KK - 1 - (ky * K + kx) : ky * K + kx))
                              : 0.f;
    __syncthreads();
    float acc[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) acc[o] = 0.f;
#pragma unroll
    for (int ir = 0; ir < G::IH; ++ir) {
      float v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx) v[kx] = sm[(ir * G::IW + col * S + kx) * NHWC_CB + lane];
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        const int ky = ir - o * S;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc[o] = fmaf(v[kx], tap[ky][kx], acc[o]);
        }
      }
    }
    if (p.ep.on && c < p.C) {
      float sc, bi;
      epilogue_coeffs<T>(p.ep, c, sc, bi);
#pragma unroll
      for (int o = 0; o < G::R; ++o) acc[o] = apply_epilogue<float>(acc[o], sc, bi, p.ep.act);
    }
    const int ox = x0 + col;
    if (ox < p.Wout && c < p.C) {
#pragma unroll
      for (int o = 0; o < G::R; ++o)
        if (y0 + o < p.Hout)
          out[(((size_t)n * p.Hout + y0 + o) * p.Wout + ox) * p.C + c] = Elem<T>::from_acc(acc[o]);
    }
  }
}

// Backward-filter, first pass, NHWC.  Block (channel block, slice) walks the slice's share of the
// (image, tile) list; x tile (with halo) and dy tile are staged; thread (channel, dy column)
// keeps K*K accumulators.  At the end the block adds, per channel and tap, its TW columns in
// order and writes partial[(c*SL + slice)*K*K + tap].
struct NhwcFilterParams {
  int N, C, H, W, Ho, Wo;
  int pt, pl;
  int SL;
  int tiles_x, tiles_y, cblocks;
};

template <typename T, int K, int S>
__global__ void __launch_bounds__(NhwcGeo<K, S, true>::THREADS)
nhwc_filter_kernel(const T *__restrict__ x, const T *__restrict__ dy, float *__restrict__ partial,
                   const NhwcFilterParams p) {
  using G = NhwcGeo<K, S, true>;
  constexpr int KK = K * K;
  // the tiles and, after the walk, one tap row of per-warp sums at a time share the buffer
  constexpr int TILE_FLOATS = (G::IH * G::IW + G::R * G::TW) * NHWC_CB;
  constexpr int RED_FLOATS = G::TW * K * NHWC_CB;
  static_assert(TILE_FLOATS >= RED_FLOATS, "the tile buffer doubles as the reduction buffer");
  __shared__ float sm[TILE_FLOATS];
  float *sx = sm, *sdy = sm + G::IH * G::IW * NHWC_CB;
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  const int lane = threadIdx.x & 31, col = threadIdx.x >> 5;
  const int cb = blockIdx.x / p.SL;
  const int slice = blockIdx.x - cb * p.SL;
  const int c0 = cb * NHWC_CB, c = c0 + lane;
  const long long total = (long long)p.N * p.tiles_y * p.tiles_x;
  const long long t_begin = slice * total / p.SL, t_end = (slice + 1) * total / p.SL;
  float acc[K][K];
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx) acc[ky][kx] = 0.f;
  for (long long t = t_begin; t < t_end; ++t) {
    const int n = (int)(t / (p.tiles_y * p.tiles_x));
    const int rest = (int)(t - (long long)n * p.tiles_y * p.tiles_x);
    const int ty = rest / p.tiles_x, tx = rest - ty * p.tiles_x;
    const int y0 = ty * G::R, x0 = tx * G::TW;
    __syncthreads();
    nhwc_stage<T, G::IH, G::IW, G::TW, 1>(sx, x + (size_t)n * p.H * p.W * p.C, p.H, p.W, p.C, c0,
                                          y0 * S - p.pt, x0 * S - p.pl);
    nhwc_stage<T, G::R, G::TW, G::TW, 1>(sdy, dy + (size_t)n * p.Ho * p.Wo * p.C, p.Ho, p.Wo, p.C, c0, y0, x0);
    __syncthreads();
    float g[G::R];
#pragma unroll
    for (int o = 0; o < G::R; ++o) g[o] = sdy[(o * G::TW + col) * NHWC_CB + lane];
#pragma unroll
    for (int ir = 0; ir < G::IH; ++ir) {
      float v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx) v[kx] = sx[(ir * G::IW + col * S + kx) * NHWC_CB + lane];
#pragma unroll
      for (int o = 0; o < G::R; ++o) {
        const int ky = ir - o * S;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc[ky][kx] = fmaf(g[o], v[kx], acc[ky][kx]);
        }
      }
    }
  }
  // the tiles are dead: per tap row, the buffer holds [column][kx][channel] and the columns
  // are added in order
#pragma unroll
  for (int ky = 0; ky < K; ++ky) {
    __syncthreads();
#pragma unroll
    for (int kx = 0; kx < K; ++kx) sm[(col * K + kx) * NHWC_CB + lane] = acc[ky][kx];
    __syncthreads();
    for (int idx = threadIdx.x; idx < K * NHWC_CB; idx += G::THREADS) {
      const int kx = idx / NHWC_CB, ln = idx - kx * NHWC_CB;
      float s = 0.f;
#pragma unroll
      for (int q = 0; q < G::TW; ++q) s += sm[(q * K + kx) * NHWC_CB + ln];
      if (c0 + ln < p.C) partial[((size_t)(c0 + ln) * p.SL + slice) * KK + ky * K + kx] = s;
    }
  }
}

}  // namespace dwb
