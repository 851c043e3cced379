"""The opt-in fused epilogue of the forward operator, act(conv(x, w) * scale[c] + bias[c]),
against the fp64 oracle followed by the same elementwise operations in fp64: every kernel
family, every activation, fp32 / fp16 / bf16 / fp64, and gradients through the activations
whose derivative is a function of the output."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from dwconv_b200 import _lib
from gpu_util import forced_path, last_path, seeded

pytestmark = pytest.mark.gpu

ACTS = {None: lambda v: v, "relu": torch.relu, "relu6": lambda v: v.clamp(0, 6), "silu": F.silu,
        "hardswish": F.hardswish}

# (shape, k, stride, padding, family that must serve it)
CASES = [
    ((4, 12, 14, 14), 3, 1, 1, _lib.PATH_ROWS), ((2, 6, 56, 56), 5, 2, 2, _lib.PATH_ROWS),
    ((2, 4, 28, 28), 7, 1, 3, _lib.PATH_ROWS), ((3, 5, 7, 7), 3, 1, 1, _lib.PATH_ROWS),
    ((2, 3, 64, 64), 3, 1, 0, _lib.PATH_TILES), ((1, 3, 63, 65), 5, 2, 2, _lib.PATH_TILES),
    ((2, 3, 12, 12), (3, 5), (1, 2), (1, 2), _lib.PATH_DIRECT), ((2, 3, 30, 30), 13, 1, 6, _lib.PATH_DIRECT),
]


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


@pytest.mark.parametrize("act", list(ACTS), ids=lambda a: str(a))
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64],
                         ids=["f32", "f16", "bf16", "f64"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c[0])) + f"k{c[1]}")
def test_forward_epilogue_matches_oracle(case, dtype, act):
    import dwconv_b200
    shape, k, s, p, family = case
    x, w, _ = seeded(shape, _pair(k), s, p, dtype, seed=5)
    g = torch.Generator().manual_seed(9)
    C = shape[1]
    scale = (torch.rand(C, generator=g) + 0.5).to(dtype).cuda()
    bias = torch.randn(C, generator=g).to(dtype).cuda()
    y = dwconv_b200.depthwise_conv2d_epilogue(x, w, scale, bias, act, stride=s, padding=p)
    if dtype != torch.float64:  # fp32, fp16 and bf16 share the kernel families; fp64 is direct only
        assert last_path() == family
    assert _lib.lib.dwconv_b200_device_status() == 0
    z = oracle.forward(x, w, s, p)  # fp64, from the storage-rounded inputs
    want = ACTS[act](z * scale.double().cpu().view(1, C, 1, 1) + bias.double().cpu().view(1, C, 1, 1))
    kk = _pair(k)[0] * _pair(k)[1]
    err = (y.double().cpu() - want).abs().max().item()
    mag = max(want.abs().max().item(), 1.0)
    tol = {torch.float32: 2e-5 * kk, torch.float16: 1e-2 * mag, torch.bfloat16: 4e-2 * mag,
           torch.float64: 1e-10 * kk}[dtype]
    assert err <= tol, (err, tol)
    # scale or bias alone, and nothing at all (the plain forward, bit for bit)
    only_b = dwconv_b200.depthwise_conv2d_epilogue(x, w, None, bias, None, stride=s, padding=p)
    wb = z + bias.double().cpu().view(1, C, 1, 1)
    assert (only_b.double().cpu() - wb).abs().max().item() <= tol
    plain = dwconv_b200.depthwise_conv2d_epilogue(x, w, stride=s, padding=p)
    assert torch.equal(plain, dwconv_b200.depthwise_conv2d(x, w, stride=s, padding=p))


@pytest.mark.parametrize("act", [None, "relu", "relu6"], ids=lambda a: str(a))
@pytest.mark.parametrize("case", CASES[:6], ids=lambda c: "x".join(map(str, c[0])) + f"k{c[1]}")
def test_epilogue_gradients(case, act):
    """dx and dW through the fused epilogue against autograd on the CPU in fp64."""
    import dwconv_b200
    shape, k, s, p, _ = case
    x, w, dy = seeded(shape, _pair(k), s, p, torch.float32, seed=6)
    C = shape[1]
    g = torch.Generator().manual_seed(2)
    scale = (torch.rand(C, generator=g) + 0.5).cuda()
    bias = torch.randn(C, generator=g).cuda()
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = dwconv_b200.depthwise_conv2d_epilogue(xr, wr, scale, bias, act, stride=s, padding=p)
    y.backward(dy)
    xd, wd = x.double().cpu().requires_grad_(True), w.double().cpu().requires_grad_(True)
    z = F.conv2d(xd, wd, stride=s, padding=p, groups=C)
    yd = ACTS[act](z * scale.double().cpu().view(1, C, 1, 1) + bias.double().cpu().view(1, C, 1, 1))
    yd.backward(dy.double().cpu())
    kk = _pair(k)[0] * _pair(k)[1]
    # elements that sit exactly on an activation kink in fp32 but not in fp64 are not compared
    assert (xr.grad.double().cpu() - xd.grad).abs().max().item() <= 1e-4 * kk
    scale_w = max(wd.grad.abs().max().item(), 1e-30)
    assert (wr.grad.double().cpu() - wd.grad).abs().max().item() <= 1e-4 * scale_w


def test_epilogue_argument_checks():
    import dwconv_b200
    x, w, _ = seeded((1, 4, 14, 14), (3, 3), 1, 1, torch.float32, seed=1)
    with pytest.raises(ValueError, match="unknown activation"):
        dwconv_b200.depthwise_conv2d_epilogue(x, w, activation="tanh", padding=1)
    with pytest.raises(RuntimeError, match="must have 4 elements"):
        dwconv_b200.depthwise_conv2d_epilogue(x, w, scale=torch.ones(3, device="cuda"), padding=1)
    with pytest.raises(RuntimeError, match="gets no gradient"):
        dwconv_b200.depthwise_conv2d_epilogue(x, w, bias=torch.ones(4, device="cuda", requires_grad=True),
                                              padding=1)
    xr = x.clone().requires_grad_(True)
    y = dwconv_b200.depthwise_conv2d_epilogue(xr, w, activation="silu", padding=1)
    with pytest.raises(RuntimeError, match="forward-only"):
        y.sum().backward()
    # the C entry point validates the activation code and the pointers' alignment
    import ctypes
    s = _lib.Shape(1, 4, 14, 14, 3, 3, 1, 1, 1, 1, 14, 14)
    yb = torch.empty_like(x)
    bad = _lib.Epilogue(None, None, 9)
    assert _lib.lib.dwconv_b200_forward_epilogue(x.data_ptr(), w.data_ptr(), yb.data_ptr(), _lib.F32, s,
                                                 ctypes.byref(bad), None) == 1
    odd = _lib.Epilogue(x.data_ptr() + 2, None, 0)
    assert _lib.lib.dwconv_b200_forward_epilogue(x.data_ptr(), w.data_ptr(), yb.data_ptr(), _lib.F32, s,
                                                 ctypes.byref(odd), None) == 3
