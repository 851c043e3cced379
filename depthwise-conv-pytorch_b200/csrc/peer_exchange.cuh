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
// A kernel stops waiting for its peers' words this long after it started (whatever the world
// size and however many words are late), or after this many polls of one word.
constexpr unsigned long long EXCHANGE_WAIT_NS = 2000000000ull;  // 2 s
constexpr unsigned EXCHANGE_MAX_POLLS = 1u << 22;

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

// The call counter of a CTA is written by one exchange kernel and read by the next; both go
// around the L1 cache (a kernel that became resident early may have read the line before its
// predecessor wrote it).
__device__ __forceinline__ unsigned ld_counter(const unsigned *p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_counter(unsigned *p, unsigned v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
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
// that does not carry the call's number (not arrived yet, or preloaded for another call) is
// polled until `deadline` (global timer, ns).  false: a word did not arrive in time.
template <typename A>
__device__ __forceinline__ bool exchange_receive(const ExchangePeers &px, size_t header, int n,
                                                 int idx, unsigned call,
                                                 unsigned long long (&v)[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W],
                                                 unsigned long long deadline, A &sum) {
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
          if (++polls > EXCHANGE_MAX_POLLS || global_timer_ns() > deadline) return false;
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

// Two forms, chosen per call:
//   same_call == 0 (pipelined): dw_out receives the PREVIOUS call's world sum (may be null: not
//     wanted); this call's sum is completed by the next call or by exchange_finish_kernel, after
//     whatever the stream runs in between has hidden the stores' flight.
//   same_call != 0 (all-reduce inside the kernel): after sending, the kernel waits for the other
//     ranks' words of THIS call and writes this call's world sum to dw_out.  For a step with
//     nothing left to run behind the gradient: one kernel instead of a send plus a finish, and
//     the wait starts while the stores are still in flight.
// Slot safety in both forms and any mix of them: a CTA reads call c-3's words (whose slot call c
// re-uses) before it sends call c-2, and it sends call c only after it has every rank's call
// c-2 or c-1 (pipelined: it receives c-1 before sending c; all-reduce: it received c-1 inside
// call c-1), so every rank is done with the slot by then.
// (Measured alternative, not kept: staging the sums and sending them from a small kernel on a
// second stream, to hide the time the peer stores take to be acknowledged, was slower on two
// GPUs: 80.8 against 78.3 us per step.)
template <typename T>
__global__ void __launch_bounds__(FINALIZE_THREADS)
backward_filter_finalize_exchange_kernel(const typename Elem<T>::acc_t *__restrict__ partial,
                                         T *__restrict__ dw_out, const int C, const int kk,
                                         const int S, const ExchangePeers px,
                                         int *__restrict__ error_flag, const int same_call) {
  using A = typename Elem<T>::acc_t;
  __shared__ A part_sum[FINALIZE_PARTS][FINALIZE_OUTPUTS];
  const int o = threadIdx.x & (FINALIZE_OUTPUTS - 1);
  const int part = threadIdx.x / FINALIZE_OUTPUTS;
  const int b = blockIdx.x;
  const int n = C * kk;
  const int idx = b * FINALIZE_OUTPUTS + o;
  const bool live = idx < n;
  pdl_launch_dependents();  // the next kernel in the stream may take its place early
  // The previous call's words do not depend on this call's first pass, so warp 0 starts loading
  // them before waiting for it (reads of this rank's own exchange buffer only).  Which call is
  // "the previous one" is only known for certain after the wait: this CTA's counter is written
  // at the end of the previous exchange kernel, which may still be running while this kernel is
  // already resident (the kernels between the two start their dependents early).  So the early
  // load goes by the counter as it reads now, a guess; the counter is read again after the wait,
  // and every word is checked against the call number it must carry (exchange_receive), so a
  // word loaded for the wrong call is simply loaded again.
  const size_t header = exchange_header_bytes(gridDim.x);
  unsigned *my_calls = reinterpret_cast<unsigned *>(px.buf[px.rank]);
  unsigned long long words[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W];
  unsigned guess = 0;
  if (part == 0 && !same_call) {
    guess = ld_counter(my_calls + b);
    if (live && guess > 0u) exchange_preload<A>(px, header, n, idx, guess, words);
  }
  pdl_wait();  // the first pass has finished, and with it everything earlier in the stream
  const unsigned long long deadline = global_timer_ns() + EXCHANGE_WAIT_NS;
  unsigned call = 0;
  if (part == 0) {
    call = ld_counter(my_calls + b) + 1u;  // the same on every rank: all ranks make the same calls
    if (!same_call && live && call > 1u && call - 1u != guess)
      exchange_preload<A>(px, header, n, idx, call - 1u, words);
  }
  const A total = finalize_sum<A>(partial, idx, live, kk, S, part_sum);
  if (part != 0) return;  // the exchange is warp 0's job: lane o owns output idx

  bool ok = true;
  if (live) {
    if (!same_call) {
      // receive before sending: a peer that sees this call's words knows that this rank is done
      // reading the previous call's
      if (call > 1u) {
        A sum;
        ok = exchange_receive<A>(px, header, n, idx, call - 1u, words, deadline, sum);
        if (ok && dw_out != nullptr) dw_out[idx] = Elem<T>::from_acc(sum);
      }
      exchange_send<A>(px, header, n, idx, call, total);
    } else {
      exchange_send<A>(px, header, n, idx, call, total);
      A sum;
      exchange_preload<A>(px, header, n, idx, call, words);
      ok = exchange_receive<A>(px, header, n, idx, call, words, deadline, sum);
      if (ok && dw_out != nullptr) dw_out[idx] = Elem<T>::from_acc(sum);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (o == 0) {
    st_counter(my_calls + b, call);
    if (!ok) atomicExch(error_flag, 1);
  }
}

// Completes the latest call: dw = its world sum.  Launched as a programmatic dependent: it
// may be resident while the kernel before it drains, and touches memory only after the wait.
template <typename T>
__global__ void __launch_bounds__(FINALIZE_OUTPUTS)
exchange_finish_kernel(T *__restrict__ dw, const int n, const ExchangePeers px,
                       int *__restrict__ error_flag) {
  using A = typename Elem<T>::acc_t;
  const int o = threadIdx.x, b = blockIdx.x;
  const int idx = b * FINALIZE_OUTPUTS + o;
  const size_t header = exchange_header_bytes(gridDim.x);
  pdl_launch_dependents();
  pdl_wait();  // the exchange kernel that made the latest call has stored its counter
  const unsigned long long deadline = global_timer_ns() + EXCHANGE_WAIT_NS;
  const unsigned call = ld_counter(reinterpret_cast<const unsigned *>(px.buf[px.rank]) + b);
  bool ok = true;
  if (idx < n && call > 0u) {
    A sum;
    unsigned long long words[EXCHANGE_MAX_WORLD][ExchangeWords<A>::W];
    exchange_preload<A>(px, header, n, idx, call, words);
    ok = exchange_receive<A>(px, header, n, idx, call, words, deadline, sum);
    if (ok) dw[idx] = Elem<T>::from_acc(sum);
  }
  ok = __all_sync(0xffffffffu, ok);
  if (o == 0 && !ok) atomicExch(error_flag, 1);
}

}  // namespace dwb
