// Compiled tensor-level binding: the counterpart of the reference's pybind11 module
// torch_dwconv._C (torch_dwconv/dwconv.cpp:60-67) for this library.
//
// It owns nothing but the glue a tensor framework needs around the C ABI of
// include/dwconv_b200.h: argument checks with the reference's texts (CHECK_CUDA,
// dwconv.cpp:24-25), result allocation with the caching allocator, the tensor's device made
// current, the current stream of that device.  All arithmetic is in libdwconv_b200.so, which
// this module links to; no kernel lives here.  dwconv_b200/_C.py holds the same functions
// over ctypes and is what runs when this module has not been built; a call costs a few
// microseconds of host time here and 15-20 there.
//
// Four functions have the reference's names and argument order; `forward` and `backward`
// are what the autograd function calls (one call per direction, both gradients from the
// fused kernel).
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <string>
#include <tuple>

#include "dwconv_b200.h"

namespace {

std::string shape_text(const at::Tensor &t) {
  // Python's tuple(t.shape) form, so that messages equal the ctypes mirror's
  std::string s = "(";
  for (int64_t i = 0; i < t.dim(); ++i) {
    s += std::to_string(t.size(i));
    if (i + 1 < t.dim() || t.dim() == 1) s += (i + 1 < t.dim()) ? ", " : ",";
  }
  return s + ")";
}

void check_cuda(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

int dtype_code(const at::Tensor &t) {
  switch (t.scalar_type()) {
    case at::kFloat: return DWCONV_B200_F32;
    case at::kHalf: return DWCONV_B200_F16;
    case at::kDouble: return DWCONV_B200_F64;
    case at::kBFloat16: return DWCONV_B200_BF16;
    default:
      TORCH_CHECK(false, "dwconv_b200: unsupported dtype ", t.dtype(),
                  " (float32, float16, bfloat16, float64)");
  }
  return -1;
}

void check_same(const at::Tensor &t, const at::Tensor &o) {
  TORCH_CHECK(o.scalar_type() == t.scalar_type() && o.device() == t.device(),
              "dwconv_b200: tensors must share dtype and device (", t.dtype(), "/", t.device(),
              " vs ", o.dtype(), "/", o.device(), ")");
}

// The library reads C*kh*kw filter values and N*C planes through raw pointers: a tensor of
// another shape would be read out of bounds, so it is refused here.
void check_filter(const at::Tensor &input, const at::Tensor &kernel) {
  TORCH_CHECK(input.dim() == 4 && kernel.dim() == 4, "dwconv_b200: expected 4-d input and kernel, got ",
              shape_text(input), " and ", shape_text(kernel));
  TORCH_CHECK(kernel.size(0) == input.size(1) && kernel.size(1) == 1,
              "dwconv_b200: kernel must be [C, 1, kh, kw] with C = ", input.size(1), ", got ",
              shape_text(kernel));
}

void check_status(int st, const char *what) {
  if (st == DWCONV_B200_OK) return;
  std::string detail = dwconv_b200_status_string(st);
  if (st == 5) detail += " [cudaError " + std::to_string(dwconv_b200_last_cuda_error()) + "]";
  TORCH_CHECK(false, "dwconv_b200.", what, ": ", detail);
}

void *stream_of(const at::Tensor &t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

bool channels_last(const at::Tensor &t) {
  return t.dim() == 4 && !t.is_contiguous() && t.is_contiguous(at::MemoryFormat::ChannelsLast);
}

// what the channels-last kernels cover (other geometries are made contiguous NCHW)
bool nhwc_served(int code, int kh, int kw, int sh, int sw) {
  return kh == kw && (kh == 3 || kh == 5 || kh == 7) && sh == sw && (sh == 1 || sh == 2) &&
         (code == DWCONV_B200_F32 || code == DWCONV_B200_F16 || code == DWCONV_B200_BF16);
}

dwconv_b200_shape make_shape(const at::Tensor &input, const at::Tensor &kernel, int sh, int sw,
                             int ph, int pw, int Ho, int Wo) {
  dwconv_b200_shape s;
  s.N = (int)input.size(0); s.C = (int)input.size(1); s.H = (int)input.size(2); s.W = (int)input.size(3);
  s.kh = (int)kernel.size(2); s.kw = (int)kernel.size(3);
  s.sh = sh; s.sw = sw; s.ph = ph; s.pw = pw; s.Ho = Ho; s.Wo = Wo;
  return s;
}

// ---- what the autograd function calls ------------------------------------------------

// (out, input as read, kernel as read, channels-last?)  The tensors "as read" are what the
// backward must be given: contiguous copies when the arguments were not.
std::tuple<at::Tensor, at::Tensor, at::Tensor, bool> forward(at::Tensor input, at::Tensor kernel,
                                                             int64_t sh, int64_t sw, int64_t ph,
                                                             int64_t pw) {
  check_cuda(input, "input");
  check_cuda(kernel, "kernel");
  const int code = dtype_code(input);
  check_same(input, kernel);
  check_filter(input, kernel);
  const int kh = (int)kernel.size(2), kw = (int)kernel.size(3);
  const bool nhwc = channels_last(input) && nhwc_served(code, kh, kw, (int)sh, (int)sw);
  if (!nhwc) input = input.contiguous();
  kernel = kernel.contiguous();
  const int H = (int)input.size(2), W = (int)input.size(3);
  const int Ho = dwconv_b200_out_size(H, 1, (int)ph, (int)ph, kh, (int)sh);
  const int Wo = dwconv_b200_out_size(W, 1, (int)pw, (int)pw, kw, (int)sw);
  TORCH_CHECK(Ho > 0 && Wo > 0, "depthwise_conv2d: filter ", kh, "x", kw,
              " does not fit the padded input ", H + 2 * ph, "x", W + 2 * pw);
  const dwconv_b200_shape s = make_shape(input, kernel, (int)sh, (int)sw, (int)ph, (int)pw, Ho, Wo);
  at::Tensor out = at::empty({s.N, s.C, Ho, Wo}, input.options(),
                             nhwc ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
  c10::cuda::CUDAGuard guard(input.device());
  int st;
  if (nhwc)
    st = dwconv_b200_forward_nhwc(input.data_ptr(), kernel.data_ptr(), out.data_ptr(), code, &s,
                                  nullptr, stream_of(input));
  else
    st = dwconv_b200_forward(input.data_ptr(), kernel.data_ptr(), out.data_ptr(), code, &s,
                             stream_of(input));
  check_status(st, "forward");
  return {out, input, kernel, nhwc};
}

// (grad_input or None, grad_kernel or None) for a forward made by `forward` above.
std::tuple<c10::optional<at::Tensor>, c10::optional<at::Tensor>> backward(
    const at::Tensor &input, at::Tensor grad_output, const at::Tensor &kernel, int64_t sh, int64_t sw,
    int64_t ph, int64_t pw, bool nhwc, bool want_dx, bool want_dw) {
  const int code = dtype_code(input);
  check_cuda(grad_output, "grad_output");
  check_same(input, grad_output);
  const int kh = (int)kernel.size(2), kw = (int)kernel.size(3);
  const int Ho = dwconv_b200_out_size((int)input.size(2), 1, (int)ph, (int)ph, kh, (int)sh);
  const int Wo = dwconv_b200_out_size((int)input.size(3), 1, (int)pw, (int)pw, kw, (int)sw);
  TORCH_CHECK(grad_output.dim() == 4 && grad_output.size(0) == input.size(0) &&
                  grad_output.size(1) == input.size(1) && grad_output.size(2) == Ho &&
                  grad_output.size(3) == Wo,
              "depthwise_conv2d backward: grad_output has shape ", shape_text(grad_output),
              ", expected (", input.size(0), ", ", input.size(1), ", ", Ho, ", ", Wo, ")");
  const dwconv_b200_shape s = make_shape(input, kernel, (int)sh, (int)sw, (int)ph, (int)pw, Ho, Wo);
  grad_output = grad_output.contiguous(nhwc ? at::MemoryFormat::ChannelsLast
                                            : at::MemoryFormat::Contiguous);
  c10::optional<at::Tensor> dx, dw;
  at::Tensor ws;
  size_t nbytes = 0;
  if (want_dw) {
    nbytes = dwconv_b200_backward_filter_workspace_bytes(code, &s);
    TORCH_CHECK(nbytes != 0, "dwconv_b200.backward: invalid geometry");
    ws = at::empty({(int64_t)nbytes}, input.options().dtype(at::kByte));
    dw = at::empty_like(kernel);
  }
  if (want_dx)
    dx = at::empty_like(input, nhwc ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
  c10::cuda::CUDAGuard guard(input.device());
  void *stream = stream_of(input);
  if (nhwc && want_dx && want_dw) {
    check_status(dwconv_b200_backward_nhwc(input.data_ptr(), grad_output.data_ptr(), kernel.data_ptr(),
                                           dx->data_ptr(), dw->data_ptr(), ws.data_ptr(), nbytes, code, &s,
                                           stream),
                 "backward_nhwc");
  } else if (nhwc) {
    if (want_dx)
      check_status(dwconv_b200_backward_input_nhwc(grad_output.data_ptr(), kernel.data_ptr(),
                                                   dx->data_ptr(), code, &s, stream),
                   "backward_input_nhwc");
    if (want_dw)
      check_status(dwconv_b200_backward_filter_nhwc(input.data_ptr(), grad_output.data_ptr(),
                                                    dw->data_ptr(), ws.data_ptr(), nbytes, code, &s,
                                                    stream),
                   "backward_filter_nhwc");
  } else if (want_dx && want_dw) {
    // both gradients from one pass over grad_output
    check_status(dwconv_b200_backward(input.data_ptr(), grad_output.data_ptr(), kernel.data_ptr(),
                                      dx->data_ptr(), dw->data_ptr(), ws.data_ptr(), nbytes, code, &s,
                                      stream),
                 "backward");
  } else if (want_dx) {
    check_status(dwconv_b200_backward_input(grad_output.data_ptr(), kernel.data_ptr(), dx->data_ptr(),
                                            code, &s, stream),
                 "backward_input");
  } else if (want_dw) {
    check_status(dwconv_b200_backward_filter(input.data_ptr(), grad_output.data_ptr(), dw->data_ptr(),
                                             ws.data_ptr(), nbytes, code, &s, stream),
                 "backward_filter");
  }
  return {dx, dw};
}

// ---- the reference's four functions (torch_dwconv/dwconv.cpp:27-67) -------------------

bool use_dwconv2d_small(const at::Tensor &input, const at::Tensor &kernel, int64_t up_h, int64_t up_w,
                        int64_t down_h, int64_t down_w, int64_t pad_h, int64_t pad_w) {
  TORCH_CHECK(input.dim() == 4 && kernel.dim() == 4, "dwconv_b200: expected 4-d input and kernel, got ",
              shape_text(input), " and ", shape_text(kernel));
  return dwconv_b200_use_dwconv2d_small((int)input.size(2), (int)input.size(3), (int)kernel.size(2),
                                        (int)kernel.size(3), (int)up_h, (int)up_w, (int)down_h,
                                        (int)down_w, (int)pad_h, (int)pad_w) != 0;
}

at::Tensor dwconv2d(at::Tensor input, at::Tensor kernel, int64_t up_h, int64_t up_w, int64_t down_h,
                    int64_t down_w, int64_t pad_h0, int64_t pad_h1, int64_t pad_w0, int64_t pad_w1,
                    bool forward_op) {
  check_cuda(input, "input");
  check_cuda(kernel, "kernel");
  const int code = dtype_code(input);
  check_same(input, kernel);
  check_filter(input, kernel);
  input = input.contiguous();
  kernel = kernel.contiguous();
  const int N = (int)input.size(0), C = (int)input.size(1), H = (int)input.size(2), W = (int)input.size(3);
  const int kh = (int)kernel.size(2), kw = (int)kernel.size(3);
  const int oh = dwconv_b200_out_size(H, (int)up_h, (int)pad_h0, (int)pad_h1, kh, (int)down_h);
  const int ow = dwconv_b200_out_size(W, (int)up_w, (int)pad_w0, (int)pad_w1, kw, (int)down_w);
  TORCH_CHECK(oh > 0 && ow > 0, "dwconv_b200.dwconv2d: empty output (", oh, " x ", ow, ")");
  at::Tensor out = at::empty({N, C, oh, ow}, input.options());
  c10::cuda::CUDAGuard guard(input.device());
  check_status(dwconv_b200_dwconv2d(input.data_ptr(), kernel.data_ptr(), out.data_ptr(), code, N, C, H,
                                    W, kh, kw, (int)up_h, (int)up_w, (int)down_h, (int)down_w,
                                    (int)pad_h0, (int)pad_h1, (int)pad_w0, (int)pad_w1,
                                    forward_op ? 1 : 0, stream_of(input)),
               "dwconv2d");
  return out;
}

at::Tensor dwconv2d_small(const at::Tensor &input, const at::Tensor &kernel, int64_t up_h, int64_t up_w,
                          int64_t down_h, int64_t down_w, int64_t pad_h, int64_t pad_w,
                          bool forward_op) {
  return dwconv2d(input, kernel, up_h, up_w, down_h, down_w, pad_h, pad_h, pad_w, pad_w, forward_op);
}

at::Tensor dwconv2d_backward_kernel(at::Tensor input, at::Tensor out_grad, const at::Tensor &kernel,
                                    int64_t up_h, int64_t up_w, int64_t down_h, int64_t down_w,
                                    int64_t pad_h, int64_t pad_w) {
  check_cuda(input, "input");
  check_cuda(out_grad, "out_grad");
  const int code = dtype_code(input);
  check_same(input, out_grad);
  TORCH_CHECK(input.dim() == 4 && out_grad.dim() == 4 && kernel.dim() == 4,
              "dwconv_b200.dwconv2d_backward_kernel: expected 4-d tensors");
  TORCH_CHECK(out_grad.size(0) == input.size(0) && out_grad.size(1) == input.size(1),
              "dwconv_b200.dwconv2d_backward_kernel: out_grad is ", shape_text(out_grad),
              " but input is ", shape_text(input), " (batch and channels must agree)");
  input = input.contiguous();
  out_grad = out_grad.contiguous();
  const int N = (int)input.size(0), C = (int)input.size(1), H = (int)input.size(2), W = (int)input.size(3);
  const int kh = (int)kernel.size(2), kw = (int)kernel.size(3);
  const int oh = (int)out_grad.size(2), ow = (int)out_grad.size(3);
  dwconv_b200_shape s;
  s.N = N; s.C = C; s.H = H; s.W = W; s.kh = kh; s.kw = kw; s.sh = (int)down_h; s.sw = (int)down_w;
  s.ph = (int)pad_h; s.pw = (int)pad_w; s.Ho = oh; s.Wo = ow;
  const size_t nbytes = dwconv_b200_backward_filter_workspace_bytes(code, &s);
  TORCH_CHECK(nbytes != 0, "dwconv_b200.dwconv2d_backward_kernel: invalid geometry");
  at::Tensor dkernel = at::empty({C, 1, kh, kw}, input.options());
  at::Tensor ws = at::empty({(int64_t)nbytes}, input.options().dtype(at::kByte));
  c10::cuda::CUDAGuard guard(input.device());
  check_status(dwconv_b200_dwconv2d_backward_kernel(
                   input.data_ptr(), out_grad.data_ptr(), dkernel.data_ptr(), ws.data_ptr(), nbytes,
                   code, N, C, H, W, oh, ow, kh, kw, (int)up_h, (int)up_w, (int)down_h, (int)down_w,
                   (int)pad_h, (int)pad_w, stream_of(input)),
               "dwconv2d_backward_kernel");
  return dkernel;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "dwconv_b200 tensor-level binding (links libdwconv_b200.so)";
  m.def("library_version", []() { return dwconv_b200_version(); });
  m.def("forward", &forward);
  m.def("backward", &backward);
  m.def("use_dwconv2d_small", &use_dwconv2d_small);
  m.def("dwconv2d", &dwconv2d);
  m.def("dwconv2d_small", &dwconv2d_small);
  m.def("dwconv2d_backward_kernel", &dwconv2d_backward_kernel);
}
