// "Tiles" kernel family: the general fast path for what the rows family declines.
//
// Serves 3x3 / 5x5 / 7x7 filters with ANY padding (top / left given, bottom / right implied by
// the output extent), any map size (odd widths, maps wider than 128 columns), fp32 / fp16 /
// bf16: forward, backward-input and backward-filter at stride 1 or 2.
// It covers the rest of the domain of the reference's large-map kernel
// (torch_dwconv/dwconv_kernel.cu:69-181: any map size, any padding below k), whose own tests
// use exactly such shapes (padding 0; 63x65 and 33x35 maps).
//
// A CTA takes a tile of TW x 32 (or 32 x 64) outputs of one plane.  All threads copy the input
// tile with its halo from global to shared memory (elements outside the map become zero, which
// is the padding), converting to fp32 on the way.  Two forms of that copy: 16-byte loads and
// stores when every row of the map starts on a 16-byte boundary (width a multiple of 4 fp32 /
// 8 fp16 elements, aligned base): the staged region then starts at the 16-byte boundary at or
// left of the halo, a 16-byte chunk is either wholly inside the map or wholly padding, and the
// copy costs about 3 instructions per element; coalesced scalar loads with one bounds test per
// element for everything else (odd widths, misaligned views, the up-sampled gradient).
// A thread then owns ONE output column and a strip of R = 8 output rows: it walks the strip's
// input rows once, reads the K values of a row under its column from shared memory (consecutive
// threads read consecutive words: no bank conflicts; stride 2 keeps even and odd columns in
// separate halves of a row for the same reason), and adds that row's contribution to every
// output row it touches.  Per accumulator the taps arrive ky-major / kx-minor with one fused
// multiply-add each: the reference's order (dwconv_kernel.cu:164-172), so fp32 results are
// bit-identical to it and to the other families.  No bulk copies, no pipeline: latency is
// hidden by several resident CTAs per SM.
//
// Backward-input at stride 2 has a kernel of its own (tile_bwd2_kernel below): the reference's
// formulation (dy up-sampled with zeros, correlated at stride 1 with the flipped filter,
// torch_dwconv/dwconv.py:57-64) with the products by the inserted zeros left out.
#pragma once

#include <atomic>

#include "common.cuh"

namespace dwb {

constexpr int TILE_THREADS = 256;
constexpr int TILE_R = 8;  // output rows per thread

struct TileParams {
  int NC, C;
  int Hin, Win, Hout, Wout;
  int pt, pl;    // rows / columns of zero padding above / left of the input
  int flip;      // apply the filter flipped in both axes (backward-input)
  int off;       // 16-byte staging: columns between the staged region's start and the halo's
  int tiles_x, tiles_y;
  long long ntiles;
  EpilogueArgs ep;  // forward with a fused epilogue (ep.on)
};

// Position of input-tile column x inside a shared-memory row: stride 2 separates even and odd
// columns so that threads c, c+1, ... (which read columns 2c + kx) hit consecutive words.
template <int S, int HALF> __device__ __forceinline__ int tile_col(int x) {
  return S == 1 ? x : (x & 1) * HALF + (x >> 1);
}

// VEC = 0: scalar staging, the staged region starts at the halo.  VEC = 16 / sizeof(T): staging
// in 16-byte chunks, the staged region starts up to VEC-1 columns left of the halo (`off`).
template <typename T, int K, int S, int TW, int VEC = 0>
struct TileGeo {
  static constexpr int TH = TILE_THREADS / TW * TILE_R;     // output rows per tile
  static constexpr int IH = (TH - 1) * S + K;               // input rows per tile
  static constexpr int IW = (TW - 1) * S + K;               // input columns per tile
  static constexpr int NCH = VEC ? (IW + 2 * VEC - 2) / VEC : 0;  // chunks per staged row
  static constexpr int IWA = VEC ? NCH * VEC : IW;          // staged columns
  static constexpr int HALF = (IWA + 1) / 2;
  static constexpr int PITCH = S == 1 ? IWA : 2 * HALF;
  static constexpr int IR = (TILE_R - 1) * S + K;           // input rows under one thread's strip
};

// 16 bytes of T from global memory (16-byte aligned) as floats.
__device__ __forceinline__ void ld16(const float *p, float (&v)[4]) {
  const float4 q = __ldg(reinterpret_cast<const float4 *>(p));
  v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
__device__ __forceinline__ void ld16(const __half *p, float (&v)[8]) {
  const uint4 q = __ldg(reinterpret_cast<const uint4 *>(p));
  const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void ld16(const __nv_bfloat16 *p, float (&v)[8]) {
  const uint4 q = __ldg(reinterpret_cast<const uint4 *>(p));
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

// The input tile in 16-byte chunks: row iy of the tile is map row gy0 + iy, chunk cx of a row
// holds map columns ax0 + cx*V .. + V-1 with ax0 a multiple of V (so is the map's width: a chunk
// never straddles the edge).  `sm` is 16-byte aligned, PITCH (and HALF) a multiple of 4 words.
template <typename T, int S, int IH, int NCH, int HALF, int PITCH>
__device__ __forceinline__ void tile_stage_vec(float *sm, const T *__restrict__ plane, int Hin, int Win,
                                               int gy0, int ax0) {
  constexpr int V = 16 / (int)sizeof(T);
  constexpr int TOTAL = IH * NCH;
  constexpr int UNROLL = V == 4 ? 4 : 2;
  for (int base = threadIdx.x; base < TOTAL; base += TILE_THREADS * UNROLL) {
    float v[UNROLL][V];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int idx = base + u * TILE_THREADS;
      const int iy = idx / NCH, cx = idx - iy * NCH;
      const int gy = gy0 + iy, gx = ax0 + cx * V;
#pragma unroll
      for (int e = 0; e < V; ++e) v[u][e] = 0.f;
      if (idx < TOTAL && (unsigned)gy < (unsigned)Hin && gx >= 0 && gx + V <= Win)
        ld16(plane + (size_t)gy * Win + gx, v[u]);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int idx = base + u * TILE_THREADS;
      const int iy = idx / NCH, cx = idx - iy * NCH;
      if (idx < TOTAL) {
        if (S == 1) {
          float4 *d = reinterpret_cast<float4 *>(sm + iy * PITCH + cx * V);
#pragma unroll
          for (int q = 0; q < V / 4; ++q)
            d[q] = make_float4(v[u][4 * q], v[u][4 * q + 1], v[u][4 * q + 2], v[u][4 * q + 3]);
        } else if (V == 4) {  // even columns in the first half of the row, odd ones in the second
          float2 *d = reinterpret_cast<float2 *>(sm + iy * PITCH + cx * 2);
          d[0] = make_float2(v[u][0], v[u][2]);
          d[HALF / 2] = make_float2(v[u][1], v[u][3]);
        } else {
          float4 *d = reinterpret_cast<float4 *>(sm + iy * PITCH + cx * 4);
          d[0] = make_float4(v[u][0], v[u][2], v[u][4], v[u][6]);
          d[HALF / 4] = make_float4(v[u][1], v[u][3], v[u][5], v[u][7]);
        }
      }
    }
  }
}

// Copies the input tile whose first element is (gy0, gx0) of `plane` into shared memory,
// element by element with a bounds test each (any alignment).
template <typename T, int S, int IH, int IW, int HALF, int PITCH>
__device__ __forceinline__ void tile_stage(float *sm, const T *__restrict__ plane, int Hin, int Win,
                                           int gy0, int gx0) {
  constexpr int TOTAL = IH * IW;
  constexpr int UNROLL = 4;
  // element idx = base + u*TILE_THREADS sits at (iy, ix); both advance by constants, so the one
  // division is outside the loop
  constexpr int DY = TILE_THREADS / IW, DX = TILE_THREADS % IW;
  int iy = threadIdx.x / IW, ix = threadIdx.x - iy * IW;
  for (int base = threadIdx.x; base < TOTAL; base += TILE_THREADS * UNROLL) {
    float v[UNROLL];
    int pos[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int idx = base + u * TILE_THREADS;
      const int gy = gy0 + iy, gx = gx0 + ix;
      pos[u] = iy * PITCH + tile_col<S, HALF>(ix);
      ix += DX; iy += DY;
      if (ix >= IW) { ix -= IW; ++iy; }
      v[u] = 0.f;
      if (idx < TOTAL && (unsigned)gy < (unsigned)Hin && (unsigned)gx < (unsigned)Win)
        v[u] = Elem<T>::ld(plane + (size_t)gy * Win + gx);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (base + u * TILE_THREADS < TOTAL) sm[pos[u]] = v[u];
  }
}

// out[oy][ox] = sum over (ky, kx) of in[oy*S - pt + ky][ox*S - pl + kx] * tap[ky][kx].
// (Four CTAs per SM, two for 7x7, as the register target: left to itself the compiler aims at
// eight, with 32 registers per thread.)
template <typename T, int K, int S, int TW, int VEC = 0>
__global__ void __launch_bounds__(TILE_THREADS, K == 7 ? 2 : 4)
tile_conv_kernel(const T *__restrict__ in, const T *__restrict__ w, T *__restrict__ out,
                 const TileParams p) {
  using G = TileGeo<T, K, S, TW, VEC>;
  constexpr int KK = K * K;
  __shared__ __align__(16) float sm[G::IH * G::PITCH];
  // position, inside a staged row, of the K columns under this thread's output column
  int cpos[K];
#pragma unroll
  for (int kx = 0; kx < K; ++kx)
    cpos[kx] = tile_col<S, G::HALF>((VEC ? p.off : 0) + (int)(threadIdx.x % TW) * S + kx);
  const int tc = threadIdx.x % TW;   // output column inside the tile
  const int tr = threadIdx.x / TW;   // strip of TILE_R output rows
  const size_t plane_in = (size_t)p.Hin * p.Win, plane_out = (size_t)p.Hout * p.Wout;
  // grid: x = the tile's position inside a plane, y = first plane; a CTA keeps its position and
  // walks the planes y, y + gridDim.y, ... (no division inside the loop; neighbouring CTAs
  // work on neighbouring tiles of one plane, so halo columns and rows are re-read from L2)
  const int ty = (int)blockIdx.x / p.tiles_x, tx = (int)blockIdx.x - ty * p.tiles_x;
  const int y0 = ty * G::TH, x0 = tx * TW;  // first output of the tile
  int chan = (int)blockIdx.y % p.C;
  const int chan_step = (int)gridDim.y % p.C;
  for (int plane = blockIdx.y; plane < p.NC; plane += gridDim.y) {
    __syncthreads();                         // the previous tile's readers are done
    if constexpr (VEC != 0)
      tile_stage_vec<T, S, G::IH, G::NCH, G::HALF, G::PITCH>(sm, in + (size_t)plane * plane_in, p.Hin,
                                                             p.Win, y0 * S - p.pt,
                                                             x0 * S - p.pl - p.off);
    else
      tile_stage<T, S, G::IH, G::IW, G::HALF, G::PITCH>(sm, in + (size_t)plane * plane_in, p.Hin,
                                                            p.Win, y0 * S - p.pt, x0 * S - p.pl);
    float tap[K][K];
    {
      const T *tp = w + (size_t)chan * KK;
      if (p.flip) {  // (two copies of the loop: constant offsets in each, no select per tap)
#pragma unroll
        for (int ky = 0; ky < K; ++ky)
#pragma unroll
          for (int kx = 0; kx < K; ++kx) tap[ky][kx] = Elem<T>::ld(tp + (KK - 1 - (ky * K + kx)));
      } else {
#pragma unroll
        for (int ky = 0; ky < K; ++ky)
#pragma unroll
          for (int kx = 0; kx < K; ++kx) tap[ky][kx] = Elem<T>::ld(tp + (ky * K + kx));
      }
    }
    __syncthreads();
    float acc[TILE_R];
#pragma unroll
    for (int o = 0; o < TILE_R; ++o) acc[o] = 0.f;
    const float *row = sm + (tr * TILE_R * S) * G::PITCH;
#pragma unroll
    for (int ir = 0; ir < G::IR; ++ir) {
      float v[K];
#pragma unroll
      for (int kx = 0; kx < K; ++kx) v[kx] = row[ir * G::PITCH + cpos[kx]];
#pragma unroll
      for (int o = 0; o < TILE_R; ++o) {
        const int ky = ir - o * S;
        if (ky >= 0 && ky < K) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc[o] = fmaf(v[kx], tap[ky][kx], acc[o]);
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
    chan += chan_step;
    if (chan >= p.C) chan -= p.C;
  }
}

// Backward-input at stride 2, polyphase.  The transposed operation is the stride-1 correlation of
// dy, up-sampled by 2 with zeros in between, with the flipped filter (torch_dwconv/dwconv.py:57-64,
// dwconv_kernel.cu:107-114): out[oy][ox] = sum over (ky, kx) of U[oy - pt + ky][ox - pl + kx] *
// wf[ky][kx], U[2a][2b] = dy[a][b] and zero elsewhere.  Three quarters of those products are with
// the inserted zeros; this kernel stages dy as it is (dense) and issues only the others, in the
// same ky-major / kx-minor order, so the sums keep their bits.  For an output column only the kx
// of one parity meet data: a thread picks its ceil(K/2) taps per filter row once per plane
// (`tsel`); for an output row only the ky of one parity do, and which is a compile-time fact once
// the parity of pt is a template argument.  Staged row d of a strip is dy row
// floor((ys - pt) / 2) + d (ys = the strip's first output row, even), and then ky = 2d - P - o for
// output row ys + o (P = pt & 1); columns likewise with pl.
template <int K, int TW, int VEC>
struct Bwd2Geo {
  static constexpr int TH = TILE_THREADS / TW * TILE_R;       // output rows per tile
  static constexpr int KH = (K + 1) / 2;                      // taps of one parity per filter row
  static constexpr int ND = (K + TILE_R - 1) / 2 + 1;         // dy rows under one strip
  static constexpr int IH = (TH / TILE_R - 1) * (TILE_R / 2) + ND;  // dy rows per tile
  static constexpr int IW = TW / 2 + KH;                      // dy columns per tile
  static constexpr int NCH = VEC ? (IW + 2 * VEC - 2) / VEC : 0;
  static constexpr int PITCH = VEC ? NCH * VEC : IW;
};

template <typename T, int K, int TW, int VEC, bool PODD>
__device__ __forceinline__ void bwd2_strip(const float *__restrict__ rows, int pitch, int col0,
                                           const float (&tsel)[K][(K + 1) / 2], float (&acc)[TILE_R]) {
  constexpr int KH = (K + 1) / 2;
  constexpr int ND = Bwd2Geo<K, TW, VEC>::ND;
  constexpr int P = PODD ? 1 : 0;
#pragma unroll
  for (int d = 0; d < ND; ++d) {
    float v[KH];
#pragma unroll
    for (int j = 0; j < KH; ++j) v[j] = rows[d * pitch + col0 + j];
#pragma unroll
    for (int o = 0; o < TILE_R; ++o) {
      const int ky = 2 * d - P - o;
      if (ky >= 0 && ky < K) {
#pragma unroll
        for (int j = 0; j < KH; ++j) acc[o] = fmaf(v[j], tsel[ky][j], acc[o]);
      }
    }
  }
}

// p: Hin x Win = dy, Hout x Wout = dx, pt / pl = k-1-padding, off as in TileParams for the dense
// dy tile (its first column is floor((x0 - pl) / 2)).
template <typename T, int K, int TW, int VEC = 0>
__global__ void __launch_bounds__(TILE_THREADS)
tile_bwd2_kernel(const T *__restrict__ dy, const T *__restrict__ w, T *__restrict__ out,
                 const TileParams p) {
  using G = Bwd2Geo<K, TW, VEC>;
  constexpr int KK = K * K;
  __shared__ __align__(16) float sm[G::IH * G::PITCH];
  const int tc = threadIdx.x % TW, tr = threadIdx.x / TW;
  const int ty = (int)blockIdx.x / p.tiles_x, tx = (int)blockIdx.x - ty * p.tiles_x;
  const int y0 = ty * G::TH, x0 = tx * TW;  // first output of the tile (both even)
  const int px = p.pl & 1;
  const int qx = (px + tc) & 1;             // parity of the kx that meet data under this column
  const int col0 = (VEC ? p.off : 0) + ((tc + qx + px) >> 1);
  // floor((y0 - pt) / 2), floor((x0 - pl) / 2): first dy row / column of the tile
  const int gy0 = (y0 - p.pt - (p.pt & 1)) / 2, gx0 = (x0 - p.pl - px) / 2;
  const size_t plane_in = (size_t)p.Hin * p.Win, plane_out = (size_t)p.Hout * p.Wout;
  int chan = (int)blockIdx.y % p.C;
  const int chan_step = (int)gridDim.y % p.C;
  for (int plane = blockIdx.y; plane < p.NC; plane += gridDim.y) {
    __syncthreads();  // the previous tile's readers are done
    if constexpr (VEC != 0)
      tile_stage_vec<T, 1, G::IH, G::NCH, 0, G::PITCH>(sm, dy + (size_t)plane * plane_in, p.Hin, p.Win,
                                                       gy0, gx0 - p.off);
    else
      tile_stage<T, 1, G::IH, G::IW, 0, G::PITCH>(sm, dy + (size_t)plane * plane_in, p.Hin, p.Win, gy0,
                                                  gx0);
    float tsel[K][G::KH];
    {
      const T *tp = w + (size_t)chan * KK;
#pragma unroll
      for (int ky = 0; ky < K; ++ky)
#pragma unroll
        for (int j = 0; j < G::KH; ++j) {
          const int kx = qx + 2 * j;  // flipped filter: wf[ky][kx] = w[K-1-ky][K-1-kx]
          tsel[ky][j] = kx < K ? Elem<T>::ld(tp + (K - 1 - ky) * K + (K - 1 - kx)) : 0.f;
        }
    }
    __syncthreads();
    float acc[TILE_R];
#pragma unroll
    for (int o = 0; o < TILE_R; ++o) acc[o] = 0.f;
    const float *rows = sm + (tr * (TILE_R / 2)) * G::PITCH;
    if (p.pt & 1)
      bwd2_strip<T, K, TW, VEC, true>(rows, G::PITCH, col0, tsel, acc);
    else
      bwd2_strip<T, K, TW, VEC, false>(rows, G::PITCH, col0, tsel, acc);
    const int ox = x0 + tc;
    if (ox < p.Wout) {
      T *op = out + (size_t)plane * plane_out + (size_t)(y0 + tr * TILE_R) * p.Wout + ox;
      const int nrows = p.Hout - (y0 + tr * TILE_R);
#pragma unroll
      for (int o = 0; o < TILE_R; ++o) {
        if (o < nrows) *op = Elem<T>::from_acc(acc[o]);
        op += p.Wout;
      }
    }
    chan += chan_step;
    if (chan >= p.C) chan -= p.C;
  }
}

// Backward-filter, first pass.  Block (c, slice) owns one of SL equal ranges of channel c's tiles
// (all images, image-major; SL may exceed the batch size) and walks them: the x tile (with halo)
// and the dy tile are staged in shared
// memory; a thread owns one dy column and a strip of dy rows, keeps K*K accumulators, walks the
// strip's x rows once and adds dy[o] * x-row values to the tap row each (x row, dy row) pair
// belongs to.  At the end the block adds its threads' accumulators in a fixed order (warp
// shuffle, then the warps in order) and writes partial[(c*SL + slice)*K*K + tap].
struct TileFilterParams {
  int N, C, H, W, Ho, Wo;
  int pt, pl;
  int off;  // as in TileParams
  int SL;
  int tiles_x, tiles_y;
};

template <typename T, int K, int S, int TW, int VEC = 0>
__global__ void __launch_bounds__(TILE_THREADS)
tile_filter_kernel(const T *__restrict__ x, const T *__restrict__ dy, float *__restrict__ partial,
                   const TileFilterParams p) {
  using G = TileGeo<T, K, S, TW, VEC>;
  constexpr int KK = K * K;
  __shared__ __align__(16) float sx[G::IH * G::PITCH];
  __shared__ __align__(16) float sdy[G::TH * TW];
  int cpos[K];
#pragma unroll
  for (int kx = 0; kx < K; ++kx)
    cpos[kx] = tile_col<S, G::HALF>((VEC ? p.off : 0) + (int)(threadIdx.x % TW) * S + kx);
  __shared__ float red[TILE_THREADS / 32][KK];
  pdl_launch_dependents();  // the second pass may take its place on the SMs early
  const int c = blockIdx.x / p.SL;
  const int slice = blockIdx.x - c * p.SL;
  // the channel's tiles, image-major, in SL contiguous ranges of equal length (+-1)
  const int per_img = p.tiles_x * p.tiles_y;
  const long long total = (long long)p.N * per_img;
  const long long t0 = slice * total / p.SL, t1 = (slice + 1) * total / p.SL;
  int n = (int)(t0 / per_img);
  int ty = (int)(t0 - (long long)n * per_img) / p.tiles_x;
  int tx = (int)(t0 - (long long)n * per_img) - ty * p.tiles_x;
  const int tc = threadIdx.x % TW, tr = threadIdx.x / TW;
  const size_t plane_x = (size_t)p.H * p.W, plane_dy = (size_t)p.Ho * p.Wo;
  float acc[K][K];
#pragma unroll
  for (int ky = 0; ky < K; ++ky)
#pragma unroll
    for (int kx = 0; kx < K; ++kx) acc[ky][kx] = 0.f;

  for (long long t = t0; t < t1; ++t) {
    const T *xp = x + ((size_t)n * p.C + c) * plane_x;
    const T *gp = dy + ((size_t)n * p.C + c) * plane_dy;
    {
      {
        const int y0 = ty * G::TH, x0 = tx * TW;
        __syncthreads();
        if constexpr (VEC != 0) {
          tile_stage_vec<T, S, G::IH, G::NCH, G::HALF, G::PITCH>(sx, xp, p.H, p.W, y0 * S - p.pt,
                                                                 x0 * S - p.pl - p.off);
          tile_stage_vec<T, 1, G::TH, TW / VEC, 0, TW>(sdy, gp, p.Ho, p.Wo, y0, x0);
        } else {
          tile_stage<T, S, G::IH, G::IW, G::HALF, G::PITCH>(sx, xp, p.H, p.W, y0 * S - p.pt,
                                                            x0 * S - p.pl);
          tile_stage<T, 1, G::TH, TW, 0, TW>(sdy, gp, p.Ho, p.Wo, y0, x0);
        }
        __syncthreads();
        float g[TILE_R];
#pragma unroll
        for (int o = 0; o < TILE_R; ++o) g[o] = sdy[(tr * TILE_R + o) * TW + tc];
        const float *row = sx + (tr * TILE_R * S) * G::PITCH;
#pragma unroll
        for (int ir = 0; ir < G::IR; ++ir) {
          float v[K];
#pragma unroll
          for (int kx = 0; kx < K; ++kx) v[kx] = row[ir * G::PITCH + cpos[kx]];
#pragma unroll
          for (int o = 0; o < TILE_R; ++o) {
            const int ky = ir - o * S;
            if (ky >= 0 && ky < K) {
#pragma unroll
              for (int kx = 0; kx < K; ++kx) acc[ky][kx] = fmaf(g[o], v[kx], acc[ky][kx]);
            }
          }
        }
      }
    }
    if (++tx == p.tiles_x) {
      tx = 0;
      if (++ty == p.tiles_y) { ty = 0; ++n; }
    }
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
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < TILE_THREADS / 32; ++q) s += red[q][threadIdx.x];
    partial[((size_t)c * p.SL + slice) * KK + threadIdx.x] = s;
  }
}

// Resident CTAs of a kernel on the whole device (asked once per instantiation).
// (The kernel is a template ARGUMENT: kernels of one signature share a function type, and a
// cache per type would be shared among them.)
template <auto kernel> inline int resident_ctas() {
  static std::atomic<int> cached{0};
  int v = cached.load(std::memory_order_relaxed);
  if (v == 0) {
    int per_sm = 0, dev = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, TILE_THREADS, 0) != cudaSuccess ||
        cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      return 148;
    }
    v = per_sm * sms;
    if (v < 1) v = 1;
    cached.store(v, std::memory_order_relaxed);
  }
  return v;
}

// Slices per channel: as many as give every CTA a place on the device at once (one wave of
// CTAs with equal tile counts), within the bound the workspace was sized for.
template <auto kernel>
inline int filter_slices_for(const TileFilterParams &p, int bound) {
  int S = resident_ctas<kernel>() / p.C;
  if (S > bound) S = bound;
  const long long total = (long long)p.N * p.tiles_x * p.tiles_y;
  if (S > total) S = (int)total;
  return S < 1 ? 1 : S;
}

}  // namespace dwb
