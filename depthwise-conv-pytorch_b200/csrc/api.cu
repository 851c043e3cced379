// C ABI of libdwconv_b200.so: argument validation, kernel-family selection, launches.
// Declarations and the reference interfaces they replace: include/dwconv_b200.h.
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "direct_kernels.cuh"
#include "peer_exchange.cuh"
#include "api_checks.cuh"
#include "rows_api.cuh"

using namespace dwb;

namespace {

// The rows family is compiled for fp32, fp16 and bf16; fp64 declines there and runs on the direct family.
template <typename T> constexpr bool kRowsCompiled = true;  // every type is instantiated (fp64 declines)

std::atomic<int> g_forced_path{DWCONV_B200_PATH_AUTO};
thread_local int t_last_path = DWCONV_B200_PATH_AUTO;
thread_local int t_last_cuda_error = 0;

int launch_status() {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    t_last_cuda_error = (int)e;
    (void)cudaGetLastError();  // clear the non-sticky error so later calls start clean
    return DWCONV_B200_CUDA_ERROR;
  }
  return DWCONV_B200_OK;
}

}  // namespace

namespace dwb {
// For the entry points that live in other translation units (static_scratch.cu): the same
// per-thread records dwconv_b200_last_cuda_error / dwconv_b200_last_path report.
int api_launch_status() { return launch_status(); }
void api_note_path(int path) { t_last_path = path; }
}  // namespace dwb

namespace {

inline int grid_for(long long total, int block) {
  long long g = ceil_div_ll(total, block);
  const long long cap = 148ll * 64;  // grid-stride beyond this
  return (int)(g < cap ? g : cap);
}

// Number of batch slices the direct backward-filter first pass uses.
inline int direct_filter_slices(const Shape &s) {
  int S = ceil_div(4 * 148, s.C);
  if (S > s.N) S = s.N;
  if (S < 1) S = 1;
  return S;
}

template <typename T>
int try_rows_forward(const T *x, const T *w, T *y, const Shape &s, cudaStream_t st) {
  if constexpr (kRowsCompiled<T>) return rows_forward<T>(x, w, y, s, st);
  return ROWS_DECLINED;
}
template <typename T>
int try_rows_backward_input(const T *dy, const T *w, T *dx, const Shape &s, cudaStream_t st) {
  if constexpr (kRowsCompiled<T>) return rows_backward_input<T>(dy, w, dx, s, st);
  return ROWS_DECLINED;
}
template <typename T> int try_rows_backward_filter_slices(const Shape &s) {
  if constexpr (kRowsCompiled<T>) return rows_backward_filter_slices<T>(s);
  return 0;
}
template <typename T>
int try_rows_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                             cudaStream_t st, int *slices_out) {
  if constexpr (kRowsCompiled<T>) return rows_backward_filter<T>(x, dy, partial, s, st, slices_out);
  return ROWS_DECLINED;
}

template <typename T> int try_rows_backward_slices(const Shape &s) {
  if constexpr (kRowsCompiled<T>) return rows_backward_slices<T>(s);
  return 0;
}
template <typename T>
int try_rows_backward(const T *x, const T *dy, const T *w, T *dx, typename Elem<T>::acc_t *partial,
                      const Shape &s, cudaStream_t st, int *slices_out, T *dw_direct) {
  if constexpr (kRowsCompiled<T>) return rows_backward<T>(x, dy, w, dx, partial, s, st, slices_out, dw_direct);
  return ROWS_DECLINED;
}

template <typename T>
int try_rows_forward_epilogue(const T *x, const T *w, T *y, const Shape &s, const EpilogueArgs &ep,
                              cudaStream_t st) {
  if constexpr (kRowsCompiled<T>) return rows_forward_epilogue<T>(x, w, y, s, ep, st);
  return ROWS_DECLINED;
}

template <typename T>
int forward_t(const void *x, const void *w, void *y, const Shape &s, cudaStream_t st, int forced,
              const EpilogueArgs &ep) {
  if (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_ROWS) {
    // large filters have no epilogue variant in the rows family: they go on to the general kernels
    int r = ep.on ? try_rows_forward_epilogue<T>((const T *)x, (const T *)w, (T *)y, s, ep, st)
                  : try_rows_forward<T>((const T *)x, (const T *)w, (T *)y, s, st);
    if (r == ROWS_SERVED) {
      t_last_path = DWCONV_B200_PATH_ROWS;
      return launch_status();
    }
    if (forced == DWCONV_B200_PATH_ROWS) return DWCONV_B200_UNSUPPORTED_SHAPE;
  }
  if (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_TILES) {
    if (tiles_forward<T>((const T *)x, (const T *)w, (T *)y, s, ep, st) == ROWS_SERVED) {
      t_last_path = DWCONV_B200_PATH_TILES;
      return launch_status();
    }
    if (forced == DWCONV_B200_PATH_TILES) return DWCONV_B200_UNSUPPORTED_SHAPE;
  }
  const long long total = (long long)s.N * s.C * s.Ho * s.Wo;
  direct_forward_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T *)x, (const T *)w,
                                                                 (T *)y, s, total, ep);
  t_last_path = DWCONV_B200_PATH_DIRECT;
  return launch_status();
}

template <typename T>
int backward_input_t(const void *dy, const void *w, void *dx, const Shape &s, cudaStream_t st,
                     int forced) {
  if (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_ROWS) {
    int r = try_rows_backward_input<T>((const T *)dy, (const T *)w, (T *)dx, s, st);
    if (r == ROWS_SERVED) {
      t_last_path = DWCONV_B200_PATH_ROWS;
      return launch_status();
    }
    if (forced == DWCONV_B200_PATH_ROWS) return DWCONV_B200_UNSUPPORTED_SHAPE;
  }
  if (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_TILES) {
    if (tiles_backward_input<T>((const T *)dy, (const T *)w, (T *)dx, s, st) == ROWS_SERVED) {
      t_last_path = DWCONV_B200_PATH_TILES;
      return launch_status();
    }
    if (forced == DWCONV_B200_PATH_TILES) return DWCONV_B200_UNSUPPORTED_SHAPE;
  }
  const long long total = (long long)s.N * s.C * s.H * s.W;
  direct_backward_input_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(
      (const T *)dy, (const T *)w, (T *)dx, s, total);
  t_last_path = DWCONV_B200_PATH_DIRECT;
  return launch_status();
}

template <typename T>
size_t filter_workspace_t(const Shape &s) {
  using A = typename Elem<T>::acc_t;
  const size_t kk = (size_t)s.kh * s.kw;
  size_t slices = (size_t)direct_filter_slices(s);
  const size_t rs = (size_t)try_rows_backward_filter_slices<T>(s);
  if (rs > slices) slices = rs;
  const size_t fs = (size_t)try_rows_backward_slices<T>(s);  // the fused backward shares the workspace
  if (fs > slices) slices = fs;
  const size_t ns = (size_t)nhwc_filter_slices(s);  // and so do the channels-last kernels
  if (ns > slices) slices = ns;
  const size_t ts = (size_t)tiles_filter_slices(s);  // and the tiles family
  if (ts > slices) slices = ts;
  size_t b = (size_t)s.C * slices * kk * sizeof(A);
  return b < 16 ? 16 : ((b + 15) / 16) * 16;
}

// First pass of the filter gradient: partial sums per (channel, slice, tap) into ws.
template <typename T>
int filter_first_pass_t(const void *x, const void *dy, void *ws, size_t ws_bytes, const Shape &s,
                        cudaStream_t st, int forced, int *slices) {
  using A = typename Elem<T>::acc_t;
  if (ws_bytes < filter_workspace_t<T>(s)) return DWCONV_B200_WORKSPACE_TOO_SMALL;
  int S = 0;
  if (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_ROWS) {
    int r = try_rows_backward_filter<T>((const T *)x, (const T *)dy, (A *)ws, s, st, &S);
    if (r == ROWS_SERVED) {
      t_last_path = DWCONV_B200_PATH_ROWS;
      int e = launch_status();
      if (e != DWCONV_B200_OK) return e;
    } else {
      if (forced == DWCONV_B200_PATH_ROWS) return DWCONV_B200_UNSUPPORTED_SHAPE;
      S = 0;
    }
  }
  if (S == 0 && (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_TILES)) {
    int used = 0;
    if (tiles_backward_filter<T>((const T *)x, (const T *)dy, (A *)ws, s, tiles_filter_slices(s), st,
                                 &used) == ROWS_SERVED) {
      S = used;
      t_last_path = DWCONV_B200_PATH_TILES;
      int e = launch_status();
      if (e != DWCONV_B200_OK) return e;
    } else if (forced == DWCONV_B200_PATH_TILES) {
      return DWCONV_B200_UNSUPPORTED_SHAPE;
    }
  }
  if (S == 0) {
    S = direct_filter_slices(s);
    direct_backward_filter_partial_kernel<T><<<s.C * S, 256, 0, st>>>((const T *)x, (const T *)dy,
                                                                      (A *)ws, s, S);
    t_last_path = DWCONV_B200_PATH_DIRECT;
    int e = launch_status();
    if (e != DWCONV_B200_OK) return e;
  }
  *slices = S;
  return DWCONV_B200_OK;
}

// Second-pass launches can be resident before the first pass has drained.
inline cudaLaunchConfig_t finalize_config(int blocks, cudaStream_t st, cudaLaunchAttribute *attr) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(FINALIZE_THREADS);
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cfg;
}

template <typename T>
int backward_filter_t(const void *x, const void *dy, void *dw, void *ws, size_t ws_bytes,
                      const Shape &s, cudaStream_t st, int forced) {
  using A = typename Elem<T>::acc_t;
  int S = 0;
  int e = filter_first_pass_t<T>(x, dy, ws, ws_bytes, s, st, forced, &S);
  if (e != DWCONV_B200_OK) return e;
  const int kk = s.kh * s.kw;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = finalize_config(finalize_blocks(s.C, kk), st, attr);
  (void)cudaLaunchKernelEx(&cfg, backward_filter_finalize_kernel<T>, (const A *)ws, (T *)dw, s.C, kk, S);
  return launch_status();
}

// First pass of the fused backward: dx, and the partial sums of dW into ws.  One kernel when
// the rows family serves the shape (dy is read once); otherwise backward-input followed by the
// filter gradient's own first pass.
// dw_direct (optional): where the kernel may write the finished filter gradient itself; *slices
// is then 0 and no second pass is due.
template <typename T>
int backward_first_pass_t(const void *x, const void *dy, const void *w, void *dx, void *ws,
                          size_t ws_bytes, const Shape &s, cudaStream_t st, int forced, int *slices,
                          void *dw_direct = nullptr) {
  using A = typename Elem<T>::acc_t;
  if (ws_bytes < filter_workspace_t<T>(s)) return DWCONV_B200_WORKSPACE_TOO_SMALL;
  if (forced == DWCONV_B200_PATH_AUTO || forced == DWCONV_B200_PATH_ROWS) {
    int S = 0;
    int r = try_rows_backward<T>((const T *)x, (const T *)dy, (const T *)w, (T *)dx, (A *)ws, s, st, &S,
                                 (T *)dw_direct);
    if (r != ROWS_DECLINED) {
      t_last_path = DWCONV_B200_PATH_ROWS;
      *slices = (r == ROWS_SERVED_DW) ? 0 : S;
      return launch_status();
    }
  }
  int e = backward_input_t<T>(dy, w, dx, s, st, forced);
  if (e != DWCONV_B200_OK) return e;
  return filter_first_pass_t<T>(x, dy, ws, ws_bytes, s, st, forced, slices);
}

// dw_is_acc: dw is an accumulator-typed buffer (fp32, fp64 for fp64 data); accumulate: add to it.
template <typename T>
int backward_t(const void *x, const void *dy, const void *w, void *dx, void *dw, void *ws,
               size_t ws_bytes, const Shape &s, cudaStream_t st, int forced, bool dw_is_acc,
               int accumulate) {
  using A = typename Elem<T>::acc_t;
  int S = 0;
  int e = dx != nullptr ? backward_first_pass_t<T>(x, dy, w, dx, ws, ws_bytes, s, st, forced, &S,
                                                   dw_is_acc ? nullptr : dw)
                        : filter_first_pass_t<T>(x, dy, ws, ws_bytes, s, st, forced, &S);
  if (e != DWCONV_B200_OK) return e;
  if (S == 0) return DWCONV_B200_OK;  // the first pass finished dW itself
  const int kk = s.kh * s.kw;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = finalize_config(finalize_blocks(s.C, kk), st, attr);
  if (dw_is_acc)
    (void)cudaLaunchKernelEx(&cfg, backward_filter_finalize_acc_kernel<A>, (const A *)ws, (A *)dw, s.C,
                             kk, S, accumulate);
  else
    (void)cudaLaunchKernelEx(&cfg, backward_filter_finalize_kernel<T>, (const A *)ws, (T *)dw, s.C, kk, S);
  return launch_status();
}

// ---- filter gradient summed over the GPUs of one node (peer_exchange.cuh) ----
__device__ int g_exchange_error_flag = 0;

}  // namespace

struct dwconv_b200_exchange {
  int world, rank, device;
  int dtype, C, kh, kw;  // the one layer geometry this buffer is laid out for
  size_t bytes;
  unsigned char *local;                       // cudaMalloc'ed here, zeroed
  unsigned char *peer[EXCHANGE_MAX_WORLD];    // peer[rank] == local; others opened by IPC
  bool connected;
  int *error_flag;
};

namespace {

inline ExchangePeers exchange_peers(const dwconv_b200_exchange *ex) {
  ExchangePeers px;
  for (int r = 0; r < EXCHANGE_MAX_WORLD; ++r) px.buf[r] = r < ex->world ? ex->peer[r] : nullptr;
  px.world = ex->world;
  px.rank = ex->rank;
  return px;
}

template <typename T>
int exchange_finish_t(void *dw, dwconv_b200_exchange *ex, cudaStream_t st) {
  const int kk = ex->kh * ex->kw;
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = finalize_config(finalize_blocks(ex->C, kk), st, attr);
  cfg.blockDim = dim3(FINALIZE_OUTPUTS);
  (void)cudaLaunchKernelEx(&cfg, exchange_finish_kernel<T>, (T *)dw, ex->C * kk, exchange_peers(ex),
                           ex->error_flag);
  return launch_status();
}

// w and dx null: filter gradient only; otherwise the fused backward's first pass.
template <typename T>
int backward_filter_exchange_t(const void *x, const void *dy, const void *w, void *dx, void *dw,
                               void *ws, size_t ws_bytes, const Shape &s, dwconv_b200_exchange *ex,
                               cudaStream_t st, int forced, int same_call) {
  using A = typename Elem<T>::acc_t;
  const int kk = s.kh * s.kw;
  const int blocks = finalize_blocks(s.C, kk);
  if (ex->C != s.C || ex->kh != s.kh || ex->kw != s.kw || sizeof(A) != (ex->dtype == DWCONV_B200_F64 ? 8 : 4) ||
      ex->bytes < exchange_bytes<A>(ex->world, s.C * kk, blocks))
    return DWCONV_B200_BAD_ARGUMENT;
  int S = 0;
  int e = dx != nullptr ? backward_first_pass_t<T>(x, dy, w, dx, ws, ws_bytes, s, st, forced, &S)
                        : filter_first_pass_t<T>(x, dy, ws, ws_bytes, s, st, forced, &S);
  if (e != DWCONV_B200_OK) return e;
  const ExchangePeers px = exchange_peers(ex);
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = finalize_config(blocks, st, attr);
  (void)cudaLaunchKernelEx(&cfg, backward_filter_finalize_exchange_kernel<T>, (const A *)ws, (T *)dw,
                           s.C, kk, S, px, ex->error_flag, same_call);
  return launch_status();
}

int check_ptrs(int dtype, const void *a, const void *b, const void *c) {
  const size_t es = elem_size(dtype);
  if (es == 0) return DWCONV_B200_UNSUPPORTED_DTYPE;
  if (a == nullptr || b == nullptr || c == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (!aligned_to(a, es) || !aligned_to(b, es) || !aligned_to(c, es)) return DWCONV_B200_MISALIGNED;
  return DWCONV_B200_OK;
}

}  // namespace

extern "C" {

int dwconv_b200_version(void) { return DWCONV_B200_VERSION; }

const char *dwconv_b200_status_string(int status) {
  switch (status) {
    case DWCONV_B200_OK: return "ok";
    case DWCONV_B200_BAD_ARGUMENT: return "bad argument (null pointer, non-positive extent, or an exchange object made for another layer)";
    case DWCONV_B200_UNSUPPORTED_DTYPE: return "unsupported dtype (expected f32, f16 or f64)";
    case DWCONV_B200_MISALIGNED: return "pointer not aligned to its element size (workspace: 16 bytes)";
    case DWCONV_B200_WORKSPACE_TOO_SMALL: return "workspace smaller than dwconv_b200_backward_filter_workspace_bytes";
    case DWCONV_B200_CUDA_ERROR: return "CUDA launch failed (see dwconv_b200_last_cuda_error)";
    case DWCONV_B200_UNSUPPORTED_SHAPE: return "the forced kernel family does not serve this shape";
    case DWCONV_B200_TOO_LARGE: return "an extent exceeds what this entry point accepts";
    default: return "unknown status";
  }
}

int dwconv_b200_last_cuda_error(void) { return t_last_cuda_error; }

int dwconv_b200_set_path(int path) {
  if (path < DWCONV_B200_PATH_AUTO || path > DWCONV_B200_PATH_TILES) return -1;
  return g_forced_path.exchange(path);
}

int dwconv_b200_last_path(void) { return t_last_path; }

int dwconv_b200_debug_plan(int op, int dtype, const dwconv_b200_shape *shape, int aligned16,
                           int *out24) {
  if (shape == nullptr || out24 == nullptr || check_shape(shape) != DWCONV_B200_OK) return 0;
  const int es = (int)elem_size(dtype);
  if (es != 4 && es != 2) return 0;
  if (op == 2) return rows_debug_filter_plan(es, *shape, aligned16, out24);
  if (op == 3) return rows_debug_backward_plan(es, *shape, aligned16, out24);
  return rows_debug_conv_plan(op, es, *shape, aligned16, out24);
}

int dwconv_b200_device_status(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) {
    t_last_cuda_error = (int)cudaGetLastError();
    return -1;
  }
  int v = rows_take_device_error();
  int ex = 0;
  if (cudaMemcpyFromSymbol(&ex, g_exchange_error_flag, sizeof(int)) == cudaSuccess && ex != 0) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_exchange_error_flag, &zero, sizeof(int));
    v |= 4;
  } else {
    (void)cudaGetLastError();
  }
  return v;
}

size_t dwconv_b200_exchange_bytes(int dtype, int C, int kh, int kw, int world) {
  if (C <= 0 || kh <= 0 || kw <= 0 || world <= 0 || world > EXCHANGE_MAX_WORLD) return 0;
  const int n = C * kh * kw, blocks = finalize_blocks(C, kh * kw);
  if ((long long)C * kh * kw > (1ll << 26)) return 0;
  if (dtype == DWCONV_B200_F64) return exchange_bytes<double>(world, n, blocks);
  if (dtype == DWCONV_B200_F32 || dtype == DWCONV_B200_F16 || dtype == DWCONV_B200_BF16)
    return exchange_bytes<float>(world, n, blocks);
  return 0;
}

int dwconv_b200_exchange_create(int dtype, int C, int kh, int kw, int world, int rank,
                                dwconv_b200_exchange **out, unsigned char *handle64) {
  const size_t bytes = dwconv_b200_exchange_bytes(dtype, C, kh, kw, world);
  if (out == nullptr || handle64 == nullptr || bytes == 0 || rank < 0 || rank >= world)
    return DWCONV_B200_BAD_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  dwconv_b200_exchange *ex = new dwconv_b200_exchange();
  ex->world = world;
  ex->rank = rank;
  ex->dtype = dtype;
  ex->C = C;
  ex->kh = kh;
  ex->kw = kw;
  ex->bytes = bytes;
  ex->local = nullptr;
  ex->connected = (world == 1);
  for (int r = 0; r < EXCHANGE_MAX_WORLD; ++r) ex->peer[r] = nullptr;
  cudaIpcMemHandle_t h;
  if (cudaGetDevice(&ex->device) != cudaSuccess ||
      cudaMalloc((void **)&ex->local, bytes) != cudaSuccess ||
      cudaMemset(ex->local, 0, bytes) != cudaSuccess ||
      cudaDeviceSynchronize() != cudaSuccess ||
      cudaGetSymbolAddress((void **)&ex->error_flag, g_exchange_error_flag) != cudaSuccess ||
      (world > 1 && cudaIpcGetMemHandle(&h, ex->local) != cudaSuccess)) {
    t_last_cuda_error = (int)cudaGetLastError();
    if (ex->local) (void)cudaFree(ex->local);
    delete ex;
    return DWCONV_B200_CUDA_ERROR;
  }
  ex->peer[rank] = ex->local;
  if (world > 1) memcpy(handle64, &h, 64); else memset(handle64, 0, 64);
  *out = ex;
  return DWCONV_B200_OK;
}

int dwconv_b200_exchange_connect(dwconv_b200_exchange *ex, const unsigned char *handles) {
  if (ex == nullptr || (ex->world > 1 && handles == nullptr)) return DWCONV_B200_BAD_ARGUMENT;
  if (ex->connected) return DWCONV_B200_OK;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != ex->device) return DWCONV_B200_BAD_ARGUMENT;
  for (int r = 0; r < ex->world; ++r) {
    if (r == ex->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)64 * r, 64);
    void *p = nullptr;
    // opened with this rank's GPU current: maps the peer's buffer here and enables peer access
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      t_last_cuda_error = (int)cudaGetLastError();
      return DWCONV_B200_CUDA_ERROR;
    }
    ex->peer[r] = (unsigned char *)p;
  }
  ex->connected = true;
  return DWCONV_B200_OK;
}

int dwconv_b200_exchange_destroy(dwconv_b200_exchange *ex) {
  if (ex == nullptr) return DWCONV_B200_OK;
  (void)cudaDeviceSynchronize();
  for (int r = 0; r < ex->world; ++r)
    if (r != ex->rank && ex->peer[r] != nullptr) (void)cudaIpcCloseMemHandle(ex->peer[r]);
  if (ex->local) (void)cudaFree(ex->local);
  (void)cudaGetLastError();
  delete ex;
  return DWCONV_B200_OK;
}

int dwconv_b200_exchange_finish(void *dw, dwconv_b200_exchange *ex, void *stream) {
  if (ex == nullptr || !ex->connected || dw == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (!aligned_to(dw, elem_size(ex->dtype))) return DWCONV_B200_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (ex->dtype) {
    case DWCONV_B200_F32: return exchange_finish_t<float>(dw, ex, st);
    case DWCONV_B200_F16: return exchange_finish_t<__half>(dw, ex, st);
    case DWCONV_B200_BF16: return exchange_finish_t<__nv_bfloat16>(dw, ex, st);
    default: return exchange_finish_t<double>(dw, ex, st);
  }
}

static int exchange_call(const void *x, const void *dy, const void *w, void *dx, void *dw_prev,
                         void *workspace, size_t workspace_bytes, int dtype,
                         const dwconv_b200_shape *shape, dwconv_b200_exchange *ex, void *stream,
                         int same_call) {
  const void *dw = dw_prev != nullptr ? dw_prev : x;  // dw_prev is optional
  int e = check_ptrs(dtype, x, dy, dw);
  if (e) return e;
  if (dx != nullptr) {
    e = check_ptrs(dtype, w, dx, dx);
    if (e) return e;
  }
  e = check_shape(shape);
  if (e) return e;
  if (ex == nullptr || !ex->connected || workspace == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (!aligned_to(workspace, 16)) return DWCONV_B200_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  const int forced = g_forced_path.load();
  switch (dtype) {
    case DWCONV_B200_F32:
      return backward_filter_exchange_t<float>(x, dy, w, dx, dw_prev, workspace, workspace_bytes, *shape, ex, st, forced, same_call);
    case DWCONV_B200_F16:
      return backward_filter_exchange_t<__half>(x, dy, w, dx, dw_prev, workspace, workspace_bytes, *shape, ex, st, forced, same_call);
    case DWCONV_B200_BF16:
      return backward_filter_exchange_t<__nv_bfloat16>(x, dy, w, dx, dw_prev, workspace, workspace_bytes, *shape, ex, st, forced, same_call);
    default:
      return backward_filter_exchange_t<double>(x, dy, w, dx, dw_prev, workspace, workspace_bytes, *shape, ex, st, forced, same_call);
  }
}

int dwconv_b200_backward_filter_exchange(const void *x, const void *dy, void *dw_prev, void *workspace,
                                         size_t workspace_bytes, int dtype,
                                         const dwconv_b200_shape *shape, dwconv_b200_exchange *ex,
                                         void *stream) {
  return exchange_call(x, dy, nullptr, nullptr, dw_prev, workspace, workspace_bytes, dtype, shape, ex,
                       stream, 0);
}

int dwconv_b200_backward_exchange(const void *x, const void *dy, const void *w, void *dx, void *dw_prev,
                                  void *workspace, size_t workspace_bytes, int dtype,
                                  const dwconv_b200_shape *shape, dwconv_b200_exchange *ex,
                                  void *stream) {
  if (w == nullptr || dx == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  return exchange_call(x, dy, w, dx, dw_prev, workspace, workspace_bytes, dtype, shape, ex, stream, 0);
}

int dwconv_b200_backward_filter_allreduce(const void *x, const void *dy, void *dw, void *workspace,
                                          size_t workspace_bytes, int dtype,
                                          const dwconv_b200_shape *shape, dwconv_b200_exchange *ex,
                                          void *stream) {
  if (dw == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  return exchange_call(x, dy, nullptr, nullptr, dw, workspace, workspace_bytes, dtype, shape, ex, stream, 1);
}

int dwconv_b200_backward_allreduce(const void *x, const void *dy, const void *w, void *dx, void *dw,
                                   void *workspace, size_t workspace_bytes, int dtype,
                                   const dwconv_b200_shape *shape, dwconv_b200_exchange *ex,
                                   void *stream) {
  if (w == nullptr || dx == nullptr || dw == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  return exchange_call(x, dy, w, dx, dw, workspace, workspace_bytes, dtype, shape, ex, stream, 1);
}

int dwconv_b200_copy_async(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return DWCONV_B200_OK;
  if (dst == nullptr || src == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream) != cudaSuccess) {
    t_last_cuda_error = (int)cudaGetLastError();
    return DWCONV_B200_CUDA_ERROR;
  }
  return DWCONV_B200_OK;
}

int dwconv_b200_out_size(int in, int up, int pad0, int pad1, int k, int down) {
  if (down <= 0) return 0;
  const long long num = (long long)in * up + pad0 + pad1 - k + down;
  if (num < 0) return 0;
  return (int)(num / down);
}

static int forward_call(const void *x, const void *w, void *y, int dtype,
                        const dwconv_b200_shape *shape, const EpilogueArgs &ep, void *stream) {
  int e = check_ptrs(dtype, x, w, y);
  if (e) return e;
  e = check_shape(shape);
  if (e) return e;
  cudaStream_t st = (cudaStream_t)stream;
  const int forced = g_forced_path.load();
  switch (dtype) {
    case DWCONV_B200_F32: return forward_t<float>(x, w, y, *shape, st, forced, ep);
    case DWCONV_B200_F16: return forward_t<__half>(x, w, y, *shape, st, forced, ep);
    case DWCONV_B200_BF16: return forward_t<__nv_bfloat16>(x, w, y, *shape, st, forced, ep);
    default: return forward_t<double>(x, w, y, *shape, st, forced, ep);
  }
}

int dwconv_b200_forward(const void *x, const void *w, void *y, int dtype,
                        const dwconv_b200_shape *shape, void *stream) {
  return forward_call(x, w, y, dtype, shape, EpilogueArgs{nullptr, nullptr, 0, 0}, stream);
}

int dwconv_b200_forward_epilogue(const void *x, const void *w, void *y, int dtype,
                                 const dwconv_b200_shape *shape, const dwconv_b200_epilogue *epilogue,
                                 void *stream) {
  EpilogueArgs ep{nullptr, nullptr, 0, 0};
  if (epilogue != nullptr) {
    if (epilogue->activation < DWCONV_B200_ACT_NONE || epilogue->activation > DWCONV_B200_ACT_HARDSWISH)
      return DWCONV_B200_BAD_ARGUMENT;
    const size_t es = elem_size(dtype);
    if (es != 0 && ((epilogue->scale != nullptr && !aligned_to(epilogue->scale, es)) ||
                    (epilogue->bias != nullptr && !aligned_to(epilogue->bias, es))))
      return DWCONV_B200_MISALIGNED;
    ep.scale = epilogue->scale;
    ep.bias = epilogue->bias;
    ep.act = epilogue->activation;
    ep.on = (ep.scale != nullptr || ep.bias != nullptr || ep.act != DWCONV_B200_ACT_NONE) ? 1 : 0;
  }
  return forward_call(x, w, y, dtype, shape, ep, stream);
}

int dwconv_b200_backward_input(const void *dy, const void *w, void *dx, int dtype,
                               const dwconv_b200_shape *shape, void *stream) {
  int e = check_ptrs(dtype, dy, w, dx);
  if (e) return e;
  e = check_shape(shape);
  if (e) return e;
  cudaStream_t st = (cudaStream_t)stream;
  const int forced = g_forced_path.load();
  switch (dtype) {
    case DWCONV_B200_F32: return backward_input_t<float>(dy, w, dx, *shape, st, forced);
    case DWCONV_B200_F16: return backward_input_t<__half>(dy, w, dx, *shape, st, forced);
    case DWCONV_B200_BF16: return backward_input_t<__nv_bfloat16>(dy, w, dx, *shape, st, forced);
    default: return backward_input_t<double>(dy, w, dx, *shape, st, forced);
  }
}

size_t dwconv_b200_backward_filter_workspace_bytes(int dtype, const dwconv_b200_shape *shape) {
  if (elem_size(dtype) == 0 || check_shape(shape) != DWCONV_B200_OK) return 0;
  switch (dtype) {
    case DWCONV_B200_F32: return filter_workspace_t<float>(*shape);
    case DWCONV_B200_F16: return filter_workspace_t<__half>(*shape);
    case DWCONV_B200_BF16: return filter_workspace_t<__nv_bfloat16>(*shape);
    default: return filter_workspace_t<double>(*shape);
  }
}

int dwconv_b200_backward_filter(const void *x, const void *dy, void *dw, void *workspace,
                                size_t workspace_bytes, int dtype,
                                const dwconv_b200_shape *shape, void *stream) {
  int e = check_ptrs(dtype, x, dy, dw);
  if (e) return e;
  e = check_shape(shape);
  if (e) return e;
  if (workspace == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (!aligned_to(workspace, 16)) return DWCONV_B200_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  const int forced = g_forced_path.load();
  switch (dtype) {
    case DWCONV_B200_F32:
      return backward_filter_t<float>(x, dy, dw, workspace, workspace_bytes, *shape, st, forced);
    case DWCONV_B200_F16:
      return backward_filter_t<__half>(x, dy, dw, workspace, workspace_bytes, *shape, st, forced);
    case DWCONV_B200_BF16:
      return backward_filter_t<__nv_bfloat16>(x, dy, dw, workspace, workspace_bytes, *shape, st, forced);
    default:
      return backward_filter_t<double>(x, dy, dw, workspace, workspace_bytes, *shape, st, forced);
  }
}

static int backward_call(const void *x, const void *dy, const void *w, void *dx, void *dw,
                         void *workspace, size_t workspace_bytes, int dtype,
                         const dwconv_b200_shape *shape, void *stream, bool dw_is_acc, int accumulate) {
  int e = check_ptrs(dtype, x, dy, dx != nullptr ? dx : x);
  if (e) return e;
  if (dx != nullptr && w == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (dw == nullptr || workspace == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  const size_t acc_size = dtype == DWCONV_B200_F64 ? 8 : 4;
  if (!aligned_to(dw, dw_is_acc ? acc_size : elem_size(dtype)) || (w != nullptr && !aligned_to(w, elem_size(dtype))))
    return DWCONV_B200_MISALIGNED;
  e = check_shape(shape);
  if (e) return e;
  if (!aligned_to(workspace, 16)) return DWCONV_B200_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  const int forced = g_forced_path.load();
  switch (dtype) {
    case DWCONV_B200_F32:
      return backward_t<float>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st, forced, dw_is_acc, accumulate);
    case DWCONV_B200_F16:
      return backward_t<__half>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st, forced, dw_is_acc, accumulate);
    case DWCONV_B200_BF16:
      return backward_t<__nv_bfloat16>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st, forced, dw_is_acc, accumulate);
    default:
      return backward_t<double>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st, forced, dw_is_acc, accumulate);
  }
}

int dwconv_b200_backward(const void *x, const void *dy, const void *w, void *dx, void *dw,
                         void *workspace, size_t workspace_bytes, int dtype,
                         const dwconv_b200_shape *shape, void *stream) {
  if (dx == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  return backward_call(x, dy, w, dx, dw, workspace, workspace_bytes, dtype, shape, stream, false, 0);
}

int dwconv_b200_backward_accumulate(const void *x, const void *dy, const void *w, void *dx,
                                    void *dw_acc, int accumulate, void *workspace,
                                    size_t workspace_bytes, int dtype,
                                    const dwconv_b200_shape *shape, void *stream) {
  return backward_call(x, dy, w, dx, dw_acc, workspace, workspace_bytes, dtype, shape, stream, true,
                       accumulate ? 1 : 0);
}

}  // extern "C"

// ---- channels-last (NHWC) operators ----
namespace {

template <typename T>
int nhwc_call_t(int op, const void *a, const void *b, void *c, void *ws, size_t ws_bytes, const Shape &s,
                const EpilogueArgs &ep, cudaStream_t st) {
  using A = typename Elem<T>::acc_t;
  int r = ROWS_DECLINED;
  if (op == 0) {
    r = nhwc_forward<T>((const T *)a, (const T *)b, (T *)c, s, ep, st);
  } else if (op == 1) {
    r = nhwc_backward_input<T>((const T *)a, (const T *)b, (T *)c, s, st);
  } else {
    if (ws_bytes < filter_workspace_t<T>(s)) return DWCONV_B200_WORKSPACE_TOO_SMALL;
    int S = 0;
    r = nhwc_backward_filter<T>((const T *)a, (const T *)b, (A *)ws, s, st, &S);
    if (r == ROWS_SERVED) {
      int e = launch_status();
      if (e != DWCONV_B200_OK) return e;
      const int kk = s.kh * s.kw;
      cudaLaunchAttribute attr[1];
      cudaLaunchConfig_t cfg = finalize_config(finalize_blocks(s.C, kk), st, attr);
      (void)cudaLaunchKernelEx(&cfg, backward_filter_finalize_kernel<T>, (const A *)ws, (T *)c, s.C, kk, S);
    }
  }
  if (r != ROWS_SERVED) return DWCONV_B200_UNSUPPORTED_SHAPE;
  return launch_status();
}

// Both gradients on channels-last maps: one pass over dy where the fused kernel serves the
// geometry, the two operators otherwise.
template <typename T>
int nhwc_backward_t(const void *x, const void *dy, const void *w, void *dx, void *dw, void *ws,
                    size_t ws_bytes, const Shape &s, cudaStream_t st) {
  using A = typename Elem<T>::acc_t;
  if (ws_bytes < filter_workspace_t<T>(s)) return DWCONV_B200_WORKSPACE_TOO_SMALL;
  int S = 0;
  if (nhwc_backward<T>((const T *)x, (const T *)dy, (const T *)w, (T *)dx, (A *)ws, s, st, &S) == ROWS_SERVED) {
    int e = launch_status();
    if (e != DWCONV_B200_OK) return e;
    const int kk = s.kh * s.kw;
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = finalize_config(finalize_blocks(s.C, kk), st, attr);
    (void)cudaLaunchKernelEx(&cfg, backward_filter_finalize_kernel<T>, (const A *)ws, (T *)dw, s.C, kk, S);
    return launch_status();
  }
  const EpilogueArgs none{nullptr, nullptr, 0, 0};
  int e = nhwc_call_t<T>(1, dy, w, dx, nullptr, 0, s, none, st);
  if (e != DWCONV_B200_OK) return e;
  return nhwc_call_t<T>(2, x, dy, dw, ws, ws_bytes, s, none, st);
}

int nhwc_call(int op, const void *a, const void *b, void *c, void *ws, size_t ws_bytes, int dtype,
              const dwconv_b200_shape *shape, const EpilogueArgs &ep, void *stream) {
  int e = check_ptrs(dtype, a, b, c);
  if (e) return e;
  e = check_shape(shape);
  if (e) return e;
  if (op == 2) {
    if (ws == nullptr) return DWCONV_B200_BAD_ARGUMENT;
    if (!aligned_to(ws, 16)) return DWCONV_B200_MISALIGNED;
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DWCONV_B200_F32: return nhwc_call_t<float>(op, a, b, c, ws, ws_bytes, *shape, ep, st);
    case DWCONV_B200_F16: return nhwc_call_t<__half>(op, a, b, c, ws, ws_bytes, *shape, ep, st);
    case DWCONV_B200_BF16: return nhwc_call_t<__nv_bfloat16>(op, a, b, c, ws, ws_bytes, *shape, ep, st);
    default: return DWCONV_B200_UNSUPPORTED_SHAPE;  // fp64: make the maps contiguous NCHW
  }
}

}  // namespace

extern "C" {

int dwconv_b200_forward_nhwc(const void *x, const void *w, void *y, int dtype,
                             const dwconv_b200_shape *shape, const dwconv_b200_epilogue *epilogue,
                             void *stream) {
  EpilogueArgs ep{nullptr, nullptr, 0, 0};
  if (epilogue != nullptr) {
    if (epilogue->activation < DWCONV_B200_ACT_NONE || epilogue->activation > DWCONV_B200_ACT_HARDSWISH)
      return DWCONV_B200_BAD_ARGUMENT;
    ep.scale = epilogue->scale;
    ep.bias = epilogue->bias;
    ep.act = epilogue->activation;
    ep.on = (ep.scale != nullptr || ep.bias != nullptr || ep.act != DWCONV_B200_ACT_NONE) ? 1 : 0;
  }
  return nhwc_call(0, x, w, y, nullptr, 0, dtype, shape, ep, stream);
}

int dwconv_b200_backward_input_nhwc(const void *dy, const void *w, void *dx, int dtype,
                                    const dwconv_b200_shape *shape, void *stream) {
  return nhwc_call(1, dy, w, dx, nullptr, 0, dtype, shape, EpilogueArgs{nullptr, nullptr, 0, 0}, stream);
}

int dwconv_b200_backward_filter_nhwc(const void *x, const void *dy, void *dw, void *workspace,
                                     size_t workspace_bytes, int dtype,
                                     const dwconv_b200_shape *shape, void *stream) {
  return nhwc_call(2, x, dy, dw, workspace, workspace_bytes, dtype, shape,
                   EpilogueArgs{nullptr, nullptr, 0, 0}, stream);
}

int dwconv_b200_backward_nhwc(const void *x, const void *dy, const void *w, void *dx, void *dw,
                              void *workspace, size_t workspace_bytes, int dtype,
                              const dwconv_b200_shape *shape, void *stream) {
  int e = check_ptrs(dtype, x, dy, w);
  if (e) return e;
  e = check_ptrs(dtype, dx, dw, workspace);
  if (e) return e;
  e = check_shape(shape);
  if (e) return e;
  if (!aligned_to(workspace, 16)) return DWCONV_B200_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DWCONV_B200_F32:
      return nhwc_backward_t<float>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st);
    case DWCONV_B200_F16:
      return nhwc_backward_t<__half>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st);
    case DWCONV_B200_BF16:
      return nhwc_backward_t<__nv_bfloat16>(x, dy, w, dx, dw, workspace, workspace_bytes, *shape, st);
    default: return DWCONV_B200_UNSUPPORTED_SHAPE;  // fp64: make the maps contiguous NCHW
  }
}

int dwconv_b200_use_dwconv2d_small(int in_h, int in_w, int kh, int kw, int up_h, int up_w,
                                   int down_h, int down_w, int pad_h, int pad_w) {
  const int out_h = dwconv_b200_out_size(in_h, up_h, pad_h, pad_h, kh, down_h);
  const int out_w = dwconv_b200_out_size(in_w, up_w, pad_w, pad_w, kw, down_w);
  return (down_h == 1 && down_w == 1 && in_h <= 32 && in_w <= 32 && in_h == out_h &&
          in_w == out_w && pad_h >= 0 && pad_h < kh && pad_w >= 0 && pad_w < kw &&
          kh * kw <= (in_h + 1) / 2 * in_w)
             ? 1
             : 0;
}

int dwconv_b200_dwconv2d(const void *in, const void *kernel, void *out, int dtype, int N, int C,
                         int in_h, int in_w, int kh, int kw, int up_h, int up_w, int down_h,
                         int down_w, int pad_h0, int pad_h1, int pad_w0, int pad_w1, int forward,
                         void *stream) {
  if (up_h <= 0 || up_w <= 0 || down_h <= 0 || down_w <= 0) return DWCONV_B200_BAD_ARGUMENT;
  const int out_h = dwconv_b200_out_size(in_h, up_h, pad_h0, pad_h1, kh, down_h);
  const int out_w = dwconv_b200_out_size(in_w, up_w, pad_w0, pad_w1, kw, down_w);
  if (out_h <= 0 || out_w <= 0) return DWCONV_B200_BAD_ARGUMENT;
  dwconv_b200_shape s;
  s.N = N; s.C = C; s.kh = kh; s.kw = kw;
  if (forward) {
    // plain strided correlation: in = x, out = y
    if (up_h != 1 || up_w != 1) return DWCONV_B200_UNSUPPORTED_SHAPE;
    s.H = in_h; s.W = in_w; s.sh = down_h; s.sw = down_w; s.ph = pad_h0; s.pw = pad_w0;
    s.Ho = out_h; s.Wo = out_w;
    return dwconv_b200_forward(in, kernel, out, dtype, &s, stream);
  }
  // transposed: in = dy [Ho,Wo], out = dx [H,W], forward stride = up, and the
  // leading padding k-1-p of the flipped correlation gives the forward padding p
  if (down_h != 1 || down_w != 1) return DWCONV_B200_UNSUPPORTED_SHAPE;
  s.H = out_h; s.W = out_w; s.sh = up_h; s.sw = up_w;
  s.ph = kh - 1 - pad_h0; s.pw = kw - 1 - pad_w0;
  s.Ho = in_h; s.Wo = in_w;
  if (s.ph < 0 || s.pw < 0) return DWCONV_B200_UNSUPPORTED_SHAPE;
  return dwconv_b200_backward_input(in, kernel, out, dtype, &s, stream);
}

int dwconv_b200_dwconv2d_small(const void *in, const void *kernel, void *out, int dtype, int N,
                               int C, int in_h, int in_w, int kh, int kw, int up_h, int up_w,
                               int down_h, int down_w, int pad_h, int pad_w, int forward,
                               void *stream) {
  return dwconv_b200_dwconv2d(in, kernel, out, dtype, N, C, in_h, in_w, kh, kw, up_h, up_w,
                              down_h, down_w, pad_h, pad_h, pad_w, pad_w, forward, stream);
}

int dwconv_b200_dwconv2d_backward_kernel(const void *input, const void *out_grad, void *dkernel,
                                         void *workspace, size_t workspace_bytes, int dtype,
                                         int N, int C, int in_h, int in_w, int out_h, int out_w,
                                         int kh, int kw, int up_h, int up_w, int down_h,
                                         int down_w, int pad_h, int pad_w, void *stream) {
  if (up_h != 1 || up_w != 1) return DWCONV_B200_UNSUPPORTED_SHAPE;
  dwconv_b200_shape s;
  s.N = N; s.C = C; s.H = in_h; s.W = in_w; s.kh = kh; s.kw = kw;
  s.sh = down_h; s.sw = down_w; s.ph = pad_h; s.pw = pad_w; s.Ho = out_h; s.Wo = out_w;
  return dwconv_b200_backward_filter(input, out_grad, dkernel, workspace, workspace_bytes, dtype,
                                     &s, stream);
}

}  // extern "C"
