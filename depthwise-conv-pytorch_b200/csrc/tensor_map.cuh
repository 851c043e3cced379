// Tensor maps for the copy engine (TMA): the encoder is a driver function, looked up at run
// time so that the library does not link libcuda.
#pragma once

#include <cuda.h>  // CUtensorMap and its enums (types only)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

namespace dwb {

using TensorMapEncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                          const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                          const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                          CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, or null when the driver has none (the callers then stage another way).
inline TensorMapEncodeTiled tensor_map_encoder() {
  static std::atomic<int> state{0};  // 0 not asked yet, 1 found, 2 absent
  static std::atomic<void *> fn{nullptr};
  int s = state.load(std::memory_order_acquire);
  if (s == 0) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess) (void)cudaGetLastError();
    const bool ok = e == cudaSuccess && q == cudaDriverEntryPointSuccess && p != nullptr;
    fn.store(ok ? p : nullptr, std::memory_order_relaxed);
    s = ok ? 1 : 2;
    state.store(s, std::memory_order_release);
  }
  return s == 1 ? reinterpret_cast<TensorMapEncodeTiled>(fn.load(std::memory_order_relaxed)) : nullptr;
}

template <typename T> struct TensorMapType;
template <> struct TensorMapType<float> {
  static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
};
template <> struct TensorMapType<__half> {
  static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
};
template <> struct TensorMapType<__nv_bfloat16> {
  static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
};

// A dense tensor of `rank` dimensions (innermost first; dims in elements, strides of dimensions
// 1.. in bytes, multiples of 16; base 16-byte aligned) read in boxes of `box` elements (inner
// extent a multiple of 16 bytes, every extent at most 256).  What a box holds outside the tensor
// reads as zero.
template <typename T>
inline bool encode_tensor_map(CUtensorMap *map, const T *base, int rank, const cuuint64_t *dims,
                              const cuuint64_t *strides, const cuuint32_t *box) {
  TensorMapEncodeTiled enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  const cuuint32_t elem[5] = {1u, 1u, 1u, 1u, 1u};
  return enc(map, TensorMapType<T>::v, (cuuint32_t)rank, const_cast<T *>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace dwb
