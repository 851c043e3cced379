"""Helpers for the GPU parity tests: call the three operators through the C ABI."""
import contextlib

import torch

import oracle
from dwconv_b200 import _lib

CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.float64: _lib.F64,
        torch.bfloat16: _lib.BF16}


def pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def make_shape(x_shape, k_hw, stride, padding):
    N, C, H, W = x_shape
    (sh, sw), (ph, pw) = pair(stride), pair(padding)
    return _lib.Shape(N, C, H, W, k_hw[0], k_hw[1], sh, sw, ph, pw,
                      oracle.conv_out(H, k_hw[0], sh, ph), oracle.conv_out(W, k_hw[1], sw, pw))


@contextlib.contextmanager
def forced_path(path):
    prev = _lib.lib.dwconv_b200_set_path(path)
    try:
        yield
    finally:
        _lib.lib.dwconv_b200_set_path(prev)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def c_forward(x, w, stride, padding):
    s = make_shape(x.shape, w.shape[2:], stride, padding)
    y = torch.full((s.N, s.C, s.Ho, s.Wo), float("nan"), dtype=x.dtype, device=x.device)
    st = _lib.lib.dwconv_b200_forward(x.data_ptr(), w.data_ptr(), y.data_ptr(), CODE[x.dtype], s,
                                      _stream())
    return st, y


def c_backward_input(dy, w, in_hw, stride, padding):
    N, C = dy.shape[:2]
    s = make_shape((N, C, in_hw[0], in_hw[1]), w.shape[2:], stride, padding)
    assert (s.Ho, s.Wo) == tuple(dy.shape[2:])
    dx = torch.full((N, C, in_hw[0], in_hw[1]), float("nan"), dtype=dy.dtype, device=dy.device)
    st = _lib.lib.dwconv_b200_backward_input(dy.data_ptr(), w.data_ptr(), dx.data_ptr(),
                                             CODE[dy.dtype], s, _stream())
    return st, dx


def c_backward_filter(x, dy, k_hw, stride, padding):
    s = make_shape(x.shape, k_hw, stride, padding)
    assert (s.Ho, s.Wo) == tuple(dy.shape[2:])
    nbytes = _lib.lib.dwconv_b200_backward_filter_workspace_bytes(CODE[x.dtype], s)
    # canary bytes after the workspace: the library must stay inside what it asked for
    ws = torch.full((nbytes + 256,), 0xA5, dtype=torch.uint8, device=x.device)
    dw = torch.full((s.C, 1, k_hw[0], k_hw[1]), float("nan"), dtype=x.dtype, device=x.device)
    st = _lib.lib.dwconv_b200_backward_filter(x.data_ptr(), dy.data_ptr(), dw.data_ptr(),
                                              ws.data_ptr(), nbytes, CODE[x.dtype], s, _stream())
    assert bool((ws[nbytes:] == 0xA5).all()), "backward-filter wrote past its workspace"
    return st, dw


def c_backward(x, dy, w, stride, padding):
    """Both gradients through the fused entry point: (status, dx, dw)."""
    s = make_shape(x.shape, w.shape[2:], stride, padding)
    assert (s.Ho, s.Wo) == tuple(dy.shape[2:])
    nbytes = _lib.lib.dwconv_b200_backward_filter_workspace_bytes(CODE[x.dtype], s)
    ws = torch.full((nbytes + 256,), 0xA5, dtype=torch.uint8, device=x.device)
    dx = torch.full(tuple(x.shape), float("nan"), dtype=x.dtype, device=x.device)
    dw = torch.full(tuple(w.shape), float("nan"), dtype=x.dtype, device=x.device)
    st = _lib.lib.dwconv_b200_backward(x.data_ptr(), dy.data_ptr(), w.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), ws.data_ptr(), nbytes, CODE[x.dtype], s,
                                       _stream())
    assert bool((ws[nbytes:] == 0xA5).all()), "fused backward wrote past its workspace"
    return st, dx, dw


def fused_backward_served(x_shape, k_hw, stride, padding, dtype, aligned16=True):
    """Whether the one-kernel first pass of the fused backward serves this geometry."""
    import ctypes
    s = make_shape(x_shape, k_hw, stride, padding)
    out = (ctypes.c_int * 24)()
    return bool(_lib.lib.dwconv_b200_debug_plan(3, CODE[dtype], s, 1 if aligned16 else 0, out))


def last_path():
    return _lib.lib.dwconv_b200_last_path()


def seeded(shape_x, k_hw, stride, padding, dtype, seed, device="cuda"):
    """x ~ N(0,1), w ~ N(0, 1/(kh*kw)), dy ~ N(0,1); drawn on CPU in fp32 in the order
    x, w, dy from one seeded generator, then cast and moved."""
    g = torch.Generator().manual_seed(seed)
    s = make_shape(shape_x, k_hw, stride, padding)
    x = torch.randn(shape_x, generator=g)
    w = torch.randn((shape_x[1], 1, k_hw[0], k_hw[1]), generator=g) / (k_hw[0] * k_hw[1]) ** 0.5
    dy = torch.randn((s.N, s.C, s.Ho, s.Wo), generator=g)
    return tuple(t.to(dtype).to(device) for t in (x, w, dy))
