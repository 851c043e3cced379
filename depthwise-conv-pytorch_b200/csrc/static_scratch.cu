// Backward-filter entry point that allocates nothing: its scratch is a fixed array in the
// library's device image.  Declaration and contract: include/dwconv_b200.h.
#include <mutex>

#include "api_checks.cuh"
#include "direct_kernels.cuh"

using namespace dwb;

namespace {

// Partial sums of the two-pass reduction.  One copy per GPU that loads the library,
// resident until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[DWCONV_B200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// The array's name is only a host-side handle; kernels need its device address, which
// differs per device.  Looked up once per device, with that device current.
int scratch_address(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return DWCONV_B200_CUDA_ERROR;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return DWCONV_B200_CUDA_ERROR;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return DWCONV_B200_OK;
}

inline int static_slices(const Shape &s) {
  int S = ceil_div(4 * 148, s.C);
  if (S > s.N) S = s.N;
  return S < 1 ? 1 : S;
}

template <typename T>
int run(const void *x, const void *dy, void *dw, const Shape &s, cudaStream_t st) {
  using A = typename Elem<T>::acc_t;
  const int kk = s.kh * s.kw;
  int S = static_slices(s);
  // shrink the batch split until the partials fit the fixed array
  while (S > 1 && (size_t)s.C * S * kk * sizeof(A) > DWCONV_B200_STATIC_SCRATCH_BYTES) --S;
  if ((size_t)s.C * S * kk * sizeof(A) > DWCONV_B200_STATIC_SCRATCH_BYTES)
    return DWCONV_B200_TOO_LARGE;
  void *scratch = nullptr;
  int e = scratch_address(&scratch);
  if (e != DWCONV_B200_OK) return e;
  direct_backward_filter_partial_kernel<T><<<s.C * S, 256, 0, st>>>((const T *)x, (const T *)dy,
                                                                    (A *)scratch, s, S);
  e = api_launch_status();
  if (e != DWCONV_B200_OK) return e;
  backward_filter_finalize_kernel<T><<<finalize_blocks(s.C, kk), FINALIZE_THREADS, 0, st>>>(
      (const A *)scratch, (T *)dw, s.C, kk, S);
  api_note_path(DWCONV_B200_PATH_DIRECT);
  return api_launch_status();
}

}  // namespace

extern "C" {

size_t dwconv_b200_static_scratch_bytes(void) { return DWCONV_B200_STATIC_SCRATCH_BYTES; }

int dwconv_b200_backward_filter_static(const void *x, const void *dy, void *dw, int dtype,
                                       const dwconv_b200_shape *s, void *stream) {
  if (x == nullptr || dy == nullptr || dw == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  int e = check_shape(s);
  if (e) return e;
  const size_t es = elem_size(dtype);
  if (es == 0) return DWCONV_B200_UNSUPPORTED_DTYPE;
  if (!aligned_to(x, es) || !aligned_to(dy, es) || !aligned_to(dw, es)) return DWCONV_B200_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DWCONV_B200_F32: return run<float>(x, dy, dw, *s, st);
    case DWCONV_B200_F16: return run<__half>(x, dy, dw, *s, st);
    case DWCONV_B200_BF16: return run<__nv_bfloat16>(x, dy, dw, *s, st);
    default: return run<double>(x, dy, dw, *s, st);
  }
}

}  // extern "C"
