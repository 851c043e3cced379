// Shared device/host helpers of libdwconv_b200: element traits, status plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dwconv_b200.h"

namespace dwb {

using Shape = dwconv_b200_shape;

// Accumulator type per element type: fp16 and fp32 accumulate in fp32, fp64 in fp64.
template <typename T> struct Elem;
template <> struct Elem<float> {
  using acc_t = float;
  static __device__ __forceinline__ float ld(const float *p) { return __ldg(p); }
  static __device__ __forceinline__ float to_acc(float v) { return v; }
  static __device__ __forceinline__ float from_acc(float v) { return v; }
};
template <> struct Elem<__half> {
  using acc_t = float;
  static __device__ __forceinline__ float ld(const __half *p) { return __half2float(__ldg(p)); }
  static __device__ __forceinline__ float to_acc(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_acc(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {  // not a reference dtype; fp32 accumulation, every family
  using acc_t = float;
  static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(__ldg(p)); }
  static __device__ __forceinline__ float to_acc(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_acc(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<double> {
  using acc_t = double;
  static __device__ __forceinline__ double ld(const double *p) { return __ldg(p); }
  static __device__ __forceinline__ double to_acc(double v) { return v; }
  static __device__ __forceinline__ double from_acc(double v) { return v; }
};

// acc + a * b with ONE rounding, a and b in the tensors' storage type.  For the 16-bit types
// this is the mixed-precision multiply-add of sm_100 (fma.rn.f32.f16 / .bf16): the product of
// two 11-bit (8-bit) significands is exact in fp32, so the result equals
// fmaf(float(a), float(b), acc) bit for bit, without the two conversions.
__device__ __forceinline__ float fma_mix(float a, float b, float acc) { return fmaf(a, b, acc); }
__device__ __forceinline__ float fma_mix(__half a, __half b, float acc) {
  float d;
  asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)), "f"(acc));
  return d;
}
__device__ __forceinline__ float fma_mix(__nv_bfloat16 a, __nv_bfloat16 b, float acc) {
  float d;
  asm("fma.rn.f32.bf16 %0, %1, %2, %3;"
      : "=f"(d)
      : "h"(__bfloat16_as_ushort(a)), "h"(__bfloat16_as_ushort(b)), "f"(acc));
  return d;
}

// Two 16-bit elements in one 32-bit word, and single elements as bit patterns: what the vector
// loads and stores of the 16-bit kernels need, for fp16 and bf16 alike.
template <typename T> struct Pack16;
template <> struct Pack16<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t r) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&r));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __halves2half2(__float2half_rn(a), __float2half_rn(b));
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float from_bits(unsigned short h) { return __half2float(__ushort_as_half(h)); }
  static __device__ __forceinline__ unsigned short to_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
};
template <> struct Pack16<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t r) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __halves2bfloat162(__float2bfloat16_rn(a), __float2bfloat16_rn(b));
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float from_bits(unsigned short h) {
    return __bfloat162float(__ushort_as_bfloat16(h));
  }
  static __device__ __forceinline__ unsigned short to_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
};

// One fused multiply-add, never split by the compiler.
__device__ __forceinline__ float fma_acc(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double fma_acc(double a, double b, double c) { return fma(a, b, c); }

// Optional epilogue of the forward operator, applied to the accumulator before the one rounding
// to the storage type: v = act(acc * scale[c] + bias[c]).  The reference has no such thing (it
// rejects a bias outright, torch_dwconv/dwconv.py:108-109); the blocks that use depthwise
// convolutions follow them with exactly this (folded batch-norm scale and shift, activation),
// which otherwise costs another read and write of the output map.
struct EpilogueArgs {
  const void *scale;  // [C] in the tensors' element type, or null (1)
  const void *bias;   // [C] or null (0)
  int act;            // dwconv_b200_activation
  int on;             // 0: plain forward
};
template <typename A> __device__ __forceinline__ A apply_activation(A v, int act) {
  switch (act) {
    case DWCONV_B200_ACT_RELU: return v > A(0) ? v : A(0);
    case DWCONV_B200_ACT_RELU6: return v < A(0) ? A(0) : (v > A(6) ? A(6) : v);
    case DWCONV_B200_ACT_SILU: return v / (A(1) + exp(-v));
    case DWCONV_B200_ACT_HARDSWISH: {
      const A t = v + A(3);
      return v * (t < A(0) ? A(0) : (t > A(6) ? A(6) : t)) / A(6);
    }
    default: return v;
  }
}
template <typename A> __device__ __forceinline__ A apply_epilogue(A acc, A sc, A bi, int act) {
  return apply_activation<A>(fma_acc(acc, sc, bi), act);
}
// scale and bias of channel c as accumulator values
template <typename T>
__device__ __forceinline__ void epilogue_coeffs(const EpilogueArgs &ep, int c,
                                                typename Elem<T>::acc_t &sc, typename Elem<T>::acc_t &bi) {
  sc = ep.scale ? Elem<T>::ld(static_cast<const T *>(ep.scale) + c) : typename Elem<T>::acc_t(1);
  bi = ep.bias ? Elem<T>::ld(static_cast<const T *>(ep.bias) + c) : typename Elem<T>::acc_t(0);
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization
// attribute may become resident while the kernel before it in the stream is still running (as soon
// as every CTA of that kernel has called pdl_launch_dependents() or exited); it must call
// pdl_wait() before it touches global memory, which returns once the earlier kernel has
// completed and its writes are visible.  Both are no-ops when the launch has no such attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Grid shaping for kernels whose CTAs keep a tile position and walk the planes (or images)
// g-th by g-th: how many CTAs share one of `positions` positions over `units` planes, on a device
// that holds `resident` CTAs of the kernel at once.  One full wave of long-lived CTAs when that
// fills at least 85 % of the device; otherwise about four waves of shorter-lived ones, so that
// no large part of the device idles behind a fixed assignment.
inline int walk_groups(long long resident, long long positions, long long units) {
  long long g = resident / positions;
  if (g < 1 || g * positions * 100 < resident * 85) g = (4 * resident + positions - 1) / positions;
  if (g > units) g = units;
  return g < 1 ? 1 : (int)g;
}
__host__ __device__ __forceinline__ long long ceil_div_ll(long long a, long long b) {
  return (a + b - 1) / b;
}

// Sum over the 32 lanes of a warp in a fixed butterfly order (deterministic).
template <typename A> __device__ __forceinline__ A warp_sum(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace dwb
