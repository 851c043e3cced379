"""ctypes front-end of ``dwconv_oracle.c`` (test infrastructure, never shipped).

The C file restates the arithmetic of ``torch_dwconv`` (reference files cited
there function by function).  This wrapper compiles it on demand with ``gcc``
and exposes torch-tensor level helpers:

* ``forward / backward_input / backward_filter``  -- fp64 ground truth; inputs
  of any float dtype are widened to double first.
* ``forward_seq / backward_input_seq``            -- fp32 arithmetic in the
  reference kernels' summation order (``dwconv_kernel.cu:164-172``); fp16 inputs
  are widened to fp32, accumulated in fp32 and rounded to fp16 once, which is
  the accumulation contract of the CUDA library.
* ``upfirdn``                                      -- the reference's general
  operator (``dwconv.cpp:27-35``) in fp64.
* ``out_size / use_small / g_pad``                 -- shape logic
  (``dwconv_kernel.cu:612-615``, ``:652-662``, ``dwconv.py:39-44``).
"""
import ctypes
import os
import subprocess

import torch

__all__ = [
    "build", "lib", "out_size", "use_small", "g_pad", "forward", "backward_input",
    "backward_filter", "upfirdn", "forward_seq", "backward_input_seq",
    "num_threads", "conv_out",
]

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libdwconv_oracle.so")
_SRC = os.path.join(_HERE, "dwconv_oracle.c")
_lib = None


def build(force=False):
    """Compile ``dwconv_oracle.c`` into ``oracle/_build/`` if stale."""
    if (not force and os.path.exists(_SO)
            and os.path.getmtime(_SO) >= os.path.getmtime(_SRC)):
        return _SO
    os.makedirs(os.path.dirname(_SO), exist_ok=True)
    cmd = ["gcc", "-O3", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-fvisibility=hidden", "-o", _SO, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.dwconv_oracle_out_size.restype = ctypes.c_int
        _lib.dwconv_oracle_use_small.restype = ctypes.c_int
        _lib.dwconv_oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads():
    return int(lib().dwconv_oracle_num_threads())


def out_size(n_in, up, pad0, pad1, k, down):
    return int(lib().dwconv_oracle_out_size(n_in, up, pad0, pad1, k, down))


def conv_out(n_in, k, stride, pad):
    """Forward output extent floor((in + 2p - k)/s) + 1."""
    return out_size(n_in, 1, pad, pad, k, stride)


def use_small(in_h, in_w, kh, kw, up, down, pad):
    return bool(lib().dwconv_oracle_use_small(in_h, in_w, kh, kw, up[0], up[1],
                                              down[0], down[1], pad[0], pad[1]))


def g_pad(in_hw, out_hw, k_hw, stride, pad):
    """Padding the reference's backward hands to its operator (dwconv.py:39-44)."""
    return (k_hw[0] - pad[0] - 1, in_hw[0] - out_hw[0] * stride[0] + pad[0],
            k_hw[1] - pad[1] - 1, in_hw[1] - out_hw[1] * stride[1] + pad[1])


def _pair(v):
    return (v, v) if not isinstance(v, (tuple, list)) else tuple(v)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _geom(x_shape, w_shape, stride, padding):
    N, C, H, W = x_shape
    kh, kw = w_shape[2], w_shape[3]
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    return N, C, H, W, kh, kw, sh, sw, ph, pw, conv_out(H, kh, sh, ph), conv_out(W, kw, sw, pw)


def _ints(*v):
    return [ctypes.c_int(int(a)) for a in v]


def forward(x, w, stride=1, padding=0):
    g = _geom(x.shape, w.shape, stride, padding)
    xd = x.detach().cpu().double().contiguous()
    wd = w.detach().cpu().double().contiguous()
    y = torch.empty(g[0], g[1], g[10], g[11], dtype=torch.float64)
    lib().dwconv_oracle_forward_f64(_ptr(xd), _ptr(wd), _ptr(y), *_ints(*g))
    return y


def backward_input(dy, w, in_hw, stride=1, padding=0):
    N, C, Ho, Wo = dy.shape
    g = _geom((N, C, in_hw[0], in_hw[1]), w.shape, stride, padding)
    assert (g[10], g[11]) == (Ho, Wo), "dy does not match the forward geometry"
    gd = dy.detach().cpu().double().contiguous()
    wd = w.detach().cpu().double().contiguous()
    dx = torch.empty(N, C, in_hw[0], in_hw[1], dtype=torch.float64)
    lib().dwconv_oracle_backward_input_f64(_ptr(gd), _ptr(wd), _ptr(dx), *_ints(*g))
    return dx


def backward_filter(x, dy, k_hw, stride=1, padding=0):
    N, C, H, W = x.shape
    g = _geom(x.shape, (C, 1, k_hw[0], k_hw[1]), stride, padding)
    assert (g[10], g[11]) == tuple(dy.shape[2:]), "dy does not match the forward geometry"
    xd = x.detach().cpu().double().contiguous()
    gd = dy.detach().cpu().double().contiguous()
    dw = torch.empty(C, 1, k_hw[0], k_hw[1], dtype=torch.float64)
    lib().dwconv_oracle_backward_filter_f64(_ptr(xd), _ptr(gd), _ptr(dw), *_ints(*g))
    return dw


def upfirdn(inp, w, up, down, pad, forward_dir):
    """pad = (pad_h0, pad_h1, pad_w0, pad_w1); up/down = (h, w)."""
    N, C, H, W = inp.shape
    kh, kw = w.shape[2], w.shape[3]
    oh = out_size(H, up[0], pad[0], pad[1], kh, down[0])
    ow = out_size(W, up[1], pad[2], pad[3], kw, down[1])
    i_d = inp.detach().cpu().double().contiguous()
    wd = w.detach().cpu().double().contiguous()
    out = torch.empty(N, C, oh, ow, dtype=torch.float64)
    lib().dwconv_oracle_upfirdn_f64(
        _ptr(i_d), _ptr(wd), _ptr(out),
        *_ints(N, C, H, W, kh, kw, up[0], up[1], down[0], down[1],
               pad[0], pad[1], pad[2], pad[3], 1 if forward_dir else 0))
    return out


def _seq(fn, a, w, out_shape, g):
    dt = a.dtype
    assert dt in (torch.float32, torch.float16), "sequential-order oracle is fp32/fp16 only"
    af = a.detach().cpu().float().contiguous()
    wf = w.detach().cpu().float().contiguous()
    out = torch.empty(out_shape, dtype=torch.float32)
    fn(_ptr(af), _ptr(wf), _ptr(out), *_ints(*g))
    return out.to(dt)  # fp16: one round-to-nearest-even at the end


def forward_seq(x, w, stride=1, padding=0):
    g = _geom(x.shape, w.shape, stride, padding)
    return _seq(lib().dwconv_oracle_forward_f32seq, x, w, (g[0], g[1], g[10], g[11]), g)


def backward_input_seq(dy, w, in_hw, stride=1, padding=0):
    N, C, Ho, Wo = dy.shape
    g = _geom((N, C, in_hw[0], in_hw[1]), w.shape, stride, padding)
    assert (g[10], g[11]) == (Ho, Wo)
    return _seq(lib().dwconv_oracle_backward_input_f32seq, dy, w,
                (N, C, in_hw[0], in_hw[1]), g)
