"""Operator-level functions with the names, argument order and error behaviour of
the reference's pybind11 module ``torch_dwconv._C`` (torch_dwconv/dwconv.cpp:60-67).

Each function takes torch tensors, allocates the result with torch (the shared
library never allocates) and calls the matching C entry point on the tensor's
device and the current stream of that device.

The four operator functions below are written over ``ctypes``; when the compiled module
``csrc/torch_binding.cpp`` has been built (``_lib.native``), the names are bound to its
functions instead: same arguments, same checks and texts, a few microseconds of host time
per call instead of 15-20.
"""
import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.float64: _lib.F64,
           torch.bfloat16: _lib.BF16}


def _check_cuda(t, name):
    # same text as CHECK_CUDA, torch_dwconv/dwconv.cpp:24-25
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")


def _dtype_code(t, *others):
    code = _DTYPES.get(t.dtype)
    if code is None:
        raise RuntimeError(f"dwconv_b200: unsupported dtype {t.dtype} (float32, float16, bfloat16, float64)")
    for o in others:
        if o.dtype != t.dtype or o.device != t.device:
            raise RuntimeError("dwconv_b200: tensors must share dtype and device "
                               f"({t.dtype}/{t.device} vs {o.dtype}/{o.device})")
    return code


def _check_filter(input, kernel):
    """The library reads C*kh*kw filter values and N*C planes through raw pointers: a tensor
    of another shape would be read out of bounds, so it is refused here."""
    if input.dim() != 4 or kernel.dim() != 4:
        raise RuntimeError(f"dwconv_b200: expected 4-d input and kernel, got {tuple(input.shape)} "
                           f"and {tuple(kernel.shape)}")
    if kernel.shape[0] != input.shape[1] or kernel.shape[1] != 1:
        raise RuntimeError(f"dwconv_b200: kernel must be [C, 1, kh, kw] with C = {input.shape[1]}, "
                           f"got {tuple(kernel.shape)}")


def _stream(t):
    """Raw handle of the current stream of ``t``'s device (no Stream object is built)."""
    return torch._C._cuda_getCurrentRawStream(t.device.index)


class _on_device:
    """``with _on_device(t):`` makes ``t``'s device current for the library call; when it
    already is (the usual case) nothing is switched."""
    __slots__ = ("idx", "prev")

    def __init__(self, t):
        self.idx = t.device.index

    def __enter__(self):
        self.prev = torch.cuda._exchange_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev != self.idx:
            torch.cuda._maybe_exchange_device(self.prev)
        return False


def out_size(n_in, up, pad0, pad1, k, down):
    """``dwconv_b200_out_size`` restated in Python (the hot path calls it per tensor):
    (in*up + pad0 + pad1 - k + down) / down, torch_dwconv/dwconv_kernel.cu:612-615."""
    if down <= 0:
        return 0
    num = n_in * up + pad0 + pad1 - k + down
    return num // down if num >= 0 else 0


def use_dwconv2d_small(input, kernel, up_h, up_w, down_h, down_w, pad_h, pad_w):
    """torch_dwconv/dwconv.cpp:61 -- host-only shape test, works for any device; the same
    predicate as ``dwconv_b200_use_dwconv2d_small`` (dwconv_kernel.cu:652-662), evaluated here
    to spare a library call per forward."""
    in_h, in_w, kh, kw = input.shape[2], input.shape[3], kernel.shape[2], kernel.shape[3]
    return (down_h == 1 and down_w == 1 and in_h <= 32 and in_w <= 32
            and in_h == out_size(in_h, up_h, pad_h, pad_h, kh, down_h)
            and in_w == out_size(in_w, up_w, pad_w, pad_w, kw, down_w)
            and 0 <= pad_h < kh and 0 <= pad_w < kw
            and kh * kw <= (in_h + 1) // 2 * in_w)


def dwconv2d(input, kernel, up_h, up_w, down_h, down_w, pad_h0, pad_h1, pad_w0, pad_w1, forward):
    """torch_dwconv/dwconv.cpp:27-35."""
    _check_cuda(input, "input")
    _check_cuda(kernel, "kernel")
    code = _dtype_code(input, kernel)
    _check_filter(input, kernel)
    input = input.contiguous()
    kernel = kernel.contiguous()
    N, C, H, W = input.shape
    kh, kw = kernel.shape[2], kernel.shape[3]
    oh = out_size(H, up_h, pad_h0, pad_h1, kh, down_h)
    ow = out_size(W, up_w, pad_w0, pad_w1, kw, down_w)
    if oh <= 0 or ow <= 0:
        raise RuntimeError(f"dwconv_b200.dwconv2d: empty output ({oh} x {ow})")
    out = torch.empty((N, C, oh, ow), dtype=input.dtype, device=input.device)
    with _on_device(input):
        st = _lib.lib.dwconv_b200_dwconv2d(
            input.data_ptr(), kernel.data_ptr(), out.data_ptr(), code, N, C, H, W, kh, kw,
            up_h, up_w, down_h, down_w, pad_h0, pad_h1, pad_w0, pad_w1, 1 if forward else 0,
            _stream(input))
    _lib.check(st, "dwconv2d")
    return out


def dwconv2d_small(input, kernel, up_h, up_w, down_h, down_w, pad_h, pad_w, forward):
    """torch_dwconv/dwconv.cpp:37-46 (symmetric padding)."""
    return dwconv2d(input, kernel, up_h, up_w, down_h, down_w, pad_h, pad_h, pad_w, pad_w, forward)


def dwconv2d_backward_kernel(input, out_grad, kernel, up_h, up_w, down_h, down_w, pad_h, pad_w):
    """torch_dwconv/dwconv.cpp:48-58.  ``kernel`` only supplies the filter extent."""
    _check_cuda(input, "input")
    _check_cuda(out_grad, "out_grad")
    code = _dtype_code(input, out_grad)
    if input.dim() != 4 or out_grad.dim() != 4 or kernel.dim() != 4:
        raise RuntimeError("dwconv_b200.dwconv2d_backward_kernel: expected 4-d tensors")
    if tuple(out_grad.shape[:2]) != tuple(input.shape[:2]):
        raise RuntimeError(f"dwconv_b200.dwconv2d_backward_kernel: out_grad is "
                           f"{tuple(out_grad.shape)} but input is {tuple(input.shape)} "
                           "(batch and channels must agree)")
    input = input.contiguous()
    out_grad = out_grad.contiguous()
    N, C, H, W = input.shape
    kh, kw = kernel.shape[2], kernel.shape[3]
    oh, ow = out_grad.shape[2], out_grad.shape[3]
    shape = _lib.Shape(N, C, H, W, kh, kw, down_h, down_w, pad_h, pad_w, oh, ow)
    nbytes = _lib.lib.dwconv_b200_backward_filter_workspace_bytes(code, shape)
    if nbytes == 0:
        raise RuntimeError("dwconv_b200.dwconv2d_backward_kernel: invalid geometry")
    dkernel = torch.empty((C, 1, kh, kw), dtype=input.dtype, device=input.device)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=input.device)
    with _on_device(input):
        st = _lib.lib.dwconv_b200_dwconv2d_backward_kernel(
            input.data_ptr(), out_grad.data_ptr(), dkernel.data_ptr(), ws.data_ptr(), nbytes, code,
            N, C, H, W, oh, ow, kh, kw, up_h, up_w, down_h, down_w, pad_h, pad_w, _stream(input))
    _lib.check(st, "dwconv2d_backward_kernel")
    return dkernel


# the ctypes forms stay reachable (tests compare the two call paths)
CTYPES_FORMS = {"dwconv2d": dwconv2d, "dwconv2d_small": dwconv2d_small,
                "dwconv2d_backward_kernel": dwconv2d_backward_kernel}

if _lib.native is not None:
    dwconv2d = _lib.native.dwconv2d
    dwconv2d_small = _lib.native.dwconv2d_small
    dwconv2d_backward_kernel = _lib.native.dwconv2d_backward_kernel
