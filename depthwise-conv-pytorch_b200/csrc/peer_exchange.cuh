// Backward-filter second pass fused with the sum over the GPUs of a node.
//
// Every rank adds its partial sums and stores the results straight into every peer's exchange
// buffer over NVLink (plain peer stores, no multimem).  Each 32-bit word of a value travels in
// one 8-byte store together with the number of the call it belongs to, so a word that can be
// read with the right call number is complete: no fences, no separate flags.  The receiving side
// adds the world's values in rank order, so every rank gets the same bits, run after run.
//
// A store takes several microseconds to become visible on the peer (NVSwitch), so the exchange
// is pipelined: call i sends call i's values and completes call i-1's, whose words have long
// arrived by then.  finish() completes the latest call.
//
// Exchange buffer of one rank (n = C*kh*kw, W = 32-bit words per accumulator, B = CTAs):
//   uint32 calls[B]                  exchanges CTA b of THIS rank has started
//   uint64 words[3][world][n*W]      words[call % 3][r][j] = {call, word j of rank r's values}
// Nothing is ever reset: call numbers only grow.  A CTA reads call i-1 and only then sends call i;
// a peer cannot finish call i+1 (where it reads call i) before that, so when it sends call i+2
// into the slot call i-1 used, nobody reads that slot any more: three slots are enough.  A CTA
// depends only on the same-numbered CTA of the other ranks.
#pragma once

#include "common.cuh"
#include "direct_kernels.cuh"

namespace dwb {

constexpr int EXCHANGE_MAX_WORLD = 8;
constexpr int EXCHANGE_SLOTS = 3;
constexpr unsigned EXCHANGE_MAX_POLLS = 1u << 21;  // each poll is about 1 us: gives up after about 2 s

struct ExchangePeers {
  unsigned char *buf[EXCHANGE_MAX_WORLD];  // every rank's buffer as mapped on this GPU
  int world, rank;
};

__host__ __device__ inline size_t exchange_header_bytes(int blocks) {
  return ((size_t)4 * blocks + 15) / 16 * 16;
}
template <typename A>
__host__ __device__ inline size_t exchange_bytes(int world, int n, int blocks) {
  return exchange_header_bytes(blocks) +
         (size_t)EXCHANGE_SLOTS * world * n * (sizeof(A) / 4) * sizeof(unsigned long long);
}

__device__ __forceinline__ void st_word_sys(unsigned long long *p, unsigned call, unsigned word) {
  const unsigned long long v = ((unsigned long long)call << 32) | word;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

template <typename A> struct ExchangeWords;
template <> struct ExchangeWords<float> {
  static constexpr int W = 1;
  static __device__ __forceinline__ void split(float v, unsigned (&w)[1]) { w[0] = __float_as_uint(v); }
  static __device__ __forceinline__ float join(const unsigned (&w)[1]) { return __uint_as_float(w[0]); }
};
template <> struct ExchangeWords<double> {
  static constexpr int W = 2;
  static __device__ __forceinline__ void split(double v, unsigned (&w)[2]) {
    w[0] = (unsigned)__double2loint(v);
    w[1] = (unsigned)__double2hiint(v);
  }
  static __device__ __forceinline__ double join(const unsigned (&w)[2]) {
    return __hiloint2double((int)w[1], (int)w[0]);
  }
};

// Sends value idx of call `call` to every rank.
template <typename A>
__device__ __forceinline__ void exchange_send(const ExchangePeers &px, size_t header, int n, int idx,
                                              unsigned call, A value) {
  constexpr int W = ExchangeWords<A>::W;
  unsigned w[W];
  ExchangeWords<A>::split(value, w);
  const size_t at = ((size_t)(call % EXCHANGE_SLOTS) * px.world + px.rank) * n * W + (size_t)idx * W;
  for (int r = 0; r < px.world; ++r) {
    unsigned long long *words = reinterpret_cast<unsigned long long *>(px.buf[r] + header) + at;
#pragma unroll
    for (int k = 0; k < W; ++k) st_word_sys(words + k, call, w[k]);
  }
}

// The words of value idx of call `call`, one load each, all in flight together (a system-scope
// load takes about a microsecond; eight in a row would take eight).
template <typename A>
__device__ __forceinline__ void exchange_preload(const ExchangePeers &px, size_t header, int n, int idx,
                                                 unsigned call,
                                                 unsigned long long (&v)[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W]) {
  constexpr int W = ExchangeWords<A>::W;
  const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(px.buf[px.rank] + header);
#pragma unroll
  for (int r = 0; r < EXCHANGE_MAX_WORLD; ++r) {
    if (r < px.world) {
      const unsigned long long *words =
          mine + ((size_t)(call % EXCHANGE_SLOTS) * px.world + r) * n * W + (size_t)idx * W;
#pragma unroll
      for (int k = 0; k < W; ++k) v[r][k] = ld_word_sys(words + k);
    }
  }
}

// Adds value idx of call `call` over the ranks, in rank order, from the preloaded words; a word
// that had not arrived yet is polled (bounded).  false: a word did not arrive.
template <typename A>
__device__ __forceinline__ bool exchange_receive(const ExchangePeers &px, size_t header, int n,
                                                 int idx, unsigned call,
                                                 unsigned long long (&v)[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W],
                                                 A &sum) {
  constexpr int W = ExchangeWords<A>::W;
  const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(px.buf[px.rank] + header);
  sum = 0;
#pragma unroll
  for (int r = 0; r < EXCHANGE_MAX_WORLD; ++r) {
    if (r < px.world) {
      const unsigned long long *words =
          mine + ((size_t)(call % EXCHANGE_SLOTS) * px.world + r) * n * W + (size_t)idx * W;
      unsigned w[W];
#pragma unroll
      for (int k = 0; k < W; ++k) {
        unsigned polls = 0;
        unsigned long long word = v[r][k];
        while ((unsigned)(word >> 32) != call) {
          if (++polls > EXCHANGE_MAX_POLLS) return false;
          __nanosleep(200);
          word = ld_word_sys(words + k);
        }
        w[k] = (unsigned)word;
      }
      sum += ExchangeWords<A>::join(w);
    }
  }
  return true;
}

// dw_prev: where the PREVIOUS call's world sum goes (may be null: not wanted).
// (Measured alternative, not kept: staging the sums and sending them from a small kernel on a
// second stream, to hide the time the peer stores take to be acknowledged, was slower on two
// GPUs: 80.8 against 78.3 us per step.)
template <typename T>
__global__ void __launch_bounds__(FINALIZE_THREADS)
backward_filter_finalize_exchange_kernel(const typename Elem<T>::acc_t *__restrict__ partial,
                                         T *__restrict__ dw_prev, const int C, const int kk,
                                         const int S, const ExchangePeers px,
                                         int *__restrict__ error_flag) {
  using A = typename Elem<T>::acc_t;
  __shared__ A part_sum[FINALIZE_PARTS][FINALIZE_OUTPUTS];
  const int o = threadIdx.x & (FINALIZE_OUTPUTS - 1);
  const int part = threadIdx.x / FINALIZE_OUTPUTS;
  const int b = blockIdx.x;
  const int n = C * kk;
  const int idx = b * FINALIZE_OUTPUTS + o;
  const bool live = idx < n;
  A acc = 0;
  pdl_launch_dependents();  // the next kernel in the stream may take its place early
  // The previous call's words do not depend on this call's first pass: warp 0 starts loading
  // them before waiting for it (reads of this rank's own exchange buffer only).
  const size_t header = exchange_header_bytes(gridDim.x);
  unsigned *my_calls = reinterpret_cast<unsigned *>(px.buf[px.rank]);
  unsigned call = 0;
  unsigned long long words[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W];
  if (part == 0) {
    call = my_calls[b] + 1u;  // the same on every rank: all ranks make the same calls
    if (live && call > 1u) exchange_preload<A>(px, header, n, idx, call - 1u, words);
  }
  pdl_wait();  // the first pass has finished and its partial sums are visible
  if (live) {
    const int c = idx / kk;
    const int tap = idx - c * kk;
    const A *src = partial + (long long)c * S * kk + tap;
#pragma unroll 4
    for (int sl = part; sl < S; sl += FINALIZE_PARTS) acc += src[(long long)sl * kk];
  }
  part_sum[part][o] = acc;
  __syncthreads();
  if (part != 0) return;  // the exchange is warp 0's job: lane o owns output idx
  A total = part_sum[0][o];
#pragma unroll
  for (int q = 1; q < FINALIZE_PARTS; ++q) total += part_sum[q][o];

  bool ok = true;
  if (live) {
    // receive before sending: a peer that sees this call's words knows that this rank is done
    // reading the previous call's, which is what makes three slots enough (see the top)
    if (call > 1u) {
      A sum;
      ok = exchange_receive<A>(px, header, n, idx, call - 1u, words, sum);
      if (ok && dw_prev != nullptr) dw_prev[idx] = Elem<T>::from_acc(sum);
    }
    exchange_send<A>(px, header, n, idx, call, total);
  }
  ok = __all_sync(0xffffffffu, ok);
  if (o == 0) {
    my_calls[b] = call;
    if (!ok) atomicExch(error_flag, 1);
  }
}

// Completes the latest call: dw = its world sum.
template <typename T>
__global__ void __launch_bounds__(FINALIZE_OUTPUTS)
exchange_finish_kernel(T *__restrict__ dw, const int n, const ExchangePeers px,
                       int *__restrict__ error_flag) {
  using A = typename Elem<T>::acc_t;
  const int o = threadIdx.x, b = blockIdx.x;
  const int idx = b * FINALIZE_OUTPUTS + o;
  const size_t header = exchange_header_bytes(gridDim.x);
  const unsigned call = reinterpret_cast<const unsigned *>(px.buf[px.rank])[b];
  bool ok = true;
  if (idx < n && call > 0u) {
    A sum;
    unsigned long long words[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W];
    exchange_preload<A>(px, header, n, idx, call, words);
    ok = exchange_receive<A>(px, header, n, idx, call, words, sum);
    if (ok) dw[idx] = Elem<T>::from_acc(sum);
  }
  ok = __all_sync(0xffffffffu, ok);
  if (o == 0 && !ok) atomicExch(error_flag, 1);
}

}  // namespace dwb
