"""Channels-last (NHWC) maps: read and written in place by their own kernels, against the
oracle and against the NCHW path on the same values."""
import pytest
import torch

import oracle
from conftest import NP_DT, assert_dw_close
from dwconv_b200 import _lib
from gpu_util import CODE, make_shape, seeded

pytestmark = pytest.mark.gpu

CASES = [
    # (N, C, H, W, k, stride, padding): channel counts around the 32-channel blocks, odd maps,
    # paddings other than k/2, tiles that end mid-map
    (2, 32, 14, 14, 3, 1, 1), (3, 40, 28, 28, 3, 2, 1), (2, 7, 33, 35, 5, 1, 2), (1, 96, 56, 56, 5, 2, 2),
    (2, 65, 17, 19, 7, 1, 3), (1, 33, 30, 41, 7, 2, 3), (2, 16, 20, 20, 3, 1, 0), (1, 48, 21, 21, 5, 2, 0),
    (1, 3, 64, 64, 3, 1, (2, 0)), (4, 160, 7, 7, 3, 1, 1),
    # enough tiles per CTA for the two-stage tensor-copy pipeline to wrap around (several images
    # per CTA in the forward, several steps per slice in the filter gradient)
    (5, 128, 112, 112, 3, 1, 1), (5, 64, 112, 112, 5, 2, 2), (40, 32, 56, 56, 7, 1, 3), (3, 24, 120, 72, 5, 1, 0),
    # stride 2 with every filter size and paddings of both parities (the polyphase backward-input)
    (2, 16, 30, 41, 7, 2, 3), (2, 8, 33, 35, 3, 2, 0), (1, 24, 20, 20, 5, 2, (1, 2)), (3, 32, 28, 28, 7, 2, (2, 5)),
    (2, 40, 17, 16, 3, 2, 2),
]


@pytest.mark.parametrize("dtn", ["f32", "f16"])
@pytest.mark.parametrize("cfg", CASES, ids=lambda c: "x".join(map(str, c)))
def test_channels_last_through_the_c_abi(cfg, dtn):
    N, C, H, W, k, s, p = cfg
    dt = NP_DT[dtn]
    x, w, dy = seeded((N, C, H, W), (k, k), s, p, dt, seed=C + H + k)
    sh = make_shape((N, C, H, W), (k, k), s, p)
    xl = x.contiguous(memory_format=torch.channels_last)
    dyl = dy.contiguous(memory_format=torch.channels_last)
    L, st0 = _lib.lib, torch.cuda.current_stream().cuda_stream
    y = torch.full_like(dyl, float("nan"))
    dx = torch.full_like(xl, float("nan"))
    assert L.dwconv_b200_forward_nhwc(xl.data_ptr(), w.data_ptr(), y.data_ptr(), CODE[dt], sh, None, st0) == 0
    assert L.dwconv_b200_backward_input_nhwc(dyl.data_ptr(), w.data_ptr(), dx.data_ptr(), CODE[dt], sh, st0) == 0
    nbytes = L.dwconv_b200_backward_filter_workspace_bytes(CODE[dt], sh)
    ws = torch.full((nbytes + 256,), 0xA5, dtype=torch.uint8, device="cuda")
    dw = torch.full_like(w, float("nan"))
    assert L.dwconv_b200_backward_filter_nhwc(xl.data_ptr(), dyl.data_ptr(), dw.data_ptr(), ws.data_ptr(),
                                              nbytes, CODE[dt], sh, st0) == 0
    torch.cuda.synchronize()
    assert bool((ws[nbytes:] == 0xA5).all()), "wrote past the workspace"
    assert y.is_contiguous(memory_format=torch.channels_last)
    assert not torch.isnan(y).any() and not torch.isnan(dx).any() and not torch.isnan(dw).any()
    assert torch.equal(y.cpu(), oracle.forward_seq(x, w, s, p))
    assert torch.equal(dx.cpu(), oracle.backward_input_seq(dy, w, (H, W), s, p))
    assert_dw_close(dw, oracle.backward_filter(x, dy, (k, k), s, p), dt, "NHWC dW")
    # both gradients in one call (one pass over dy at stride 1 with 3x3 / 5x5 filters, the two
    # operators otherwise): dx the same bits, dW the same sums in another order
    dx2 = torch.full_like(xl, float("nan"))
    dw2 = torch.full_like(w, float("nan"))
    ws.fill_(0xA5)
    assert L.dwconv_b200_backward_nhwc(xl.data_ptr(), dyl.data_ptr(), w.data_ptr(), dx2.data_ptr(),
                                       dw2.data_ptr(), ws.data_ptr(), nbytes, CODE[dt], sh, st0) == 0
    torch.cuda.synchronize()
    assert bool((ws[nbytes:] == 0xA5).all()), "wrote past the workspace"
    assert torch.equal(dx2, dx), "fused dx differs from backward-input's"
    assert not torch.isnan(dw2).any()
    assert_dw_close(dw2, oracle.backward_filter(x, dy, (k, k), s, p), dt, "NHWC fused dW")
    assert L.dwconv_b200_device_status() == 0, "a bounded wait expired in a kernel"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["f32", "f16", "bf16"])
def test_channels_last_through_autograd(dtype):
    """``depthwise_conv2d`` on a channels-last tensor: output and input gradient come back
    channels-last, with the values of the NCHW path."""
    import dwconv_b200
    for (N, C, H, W, k, s, p) in [(2, 40, 28, 28, 3, 1, 1), (2, 24, 30, 30, 5, 2, 2)]:
        x, w, dy = seeded((N, C, H, W), (k, k), s, p, dtype, seed=3)
        xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        ya = dwconv_b200.depthwise_conv2d(xa, wa, stride=s, padding=p)
        ya.backward(dy)
        xb = x.contiguous(memory_format=torch.channels_last).requires_grad_(True)
        wb = w.clone().requires_grad_(True)
        yb = dwconv_b200.depthwise_conv2d(xb, wb, stride=s, padding=p)
        assert yb.is_contiguous(memory_format=torch.channels_last) and not yb.is_contiguous()
        yb.backward(dy.contiguous(memory_format=torch.channels_last))
        assert xb.grad.is_contiguous(memory_format=torch.channels_last)
        assert torch.equal(yb, ya)
        assert torch.equal(xb.grad, xa.grad)
        scale = wa.grad.double().abs().max().item()
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert (wb.grad.double() - wa.grad.double()).abs().max().item() <= tol * scale
    assert _lib.lib.dwconv_b200_device_status() == 0


def test_channels_last_outside_the_nhwc_kernels_is_copied():
    """A geometry the channels-last kernels do not cover (rectangular filter) still works: the
    map is made contiguous first, as the reference does for every input."""
    import dwconv_b200
    x, w, _ = seeded((2, 8, 12, 12), (3, 5), 1, (1, 2), torch.float32, seed=8)
    xl = x.contiguous(memory_format=torch.channels_last)
    y = dwconv_b200.depthwise_conv2d(xl, w, stride=1, padding=(1, 2))
    assert y.is_contiguous()
    assert torch.equal(y.cpu(), oracle.forward_seq(x, w, 1, (1, 2)))
    s = make_shape((2, 8, 12, 12), (3, 5), 1, (1, 2))
    assert _lib.lib.dwconv_b200_forward_nhwc(xl.data_ptr(), w.data_ptr(), y.data_ptr(), _lib.F32, s, None,
                                             None) == 6


@pytest.mark.parametrize("layout", ["nhwc", "wide_nchw"])
def test_tensor_copy_kernels_replay_in_a_cuda_graph(layout):
    """The kernels whose tiles arrive by tensor copies take their tensor maps as launch
    arguments, so a captured launch keeps them: after one eager call (one-time set-up), forward
    and both gradients are captured into a CUDA graph and replayed on new values in the same
    buffers; results equal the eager ones bit for bit."""
    if layout == "nhwc":
        N, C, H, W, k, s, p = 6, 64, 28, 28, 3, 1, 1
    else:
        N, C, H, W, k, s, p = 2, 8, 40, 160, 5, 1, 2   # wider than 128 columns: the tile kernels
    dt = torch.float32
    x, w, dy = seeded((N, C, H, W), (k, k), s, p, dt, seed=21)
    sh = make_shape((N, C, H, W), (k, k), s, p)
    fmt = torch.channels_last if layout == "nhwc" else torch.contiguous_format
    xs, dys = x.contiguous(memory_format=fmt), dy.contiguous(memory_format=fmt)
    y, dx, dw = torch.empty_like(dys), torch.empty_like(xs), torch.empty_like(w)
    L = _lib.lib
    nbytes = L.dwconv_b200_backward_filter_workspace_bytes(CODE[dt], sh)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")

    def ops(st):
        if layout == "nhwc":
            a = L.dwconv_b200_forward_nhwc(xs.data_ptr(), w.data_ptr(), y.data_ptr(), CODE[dt], sh, None, st)
            b = L.dwconv_b200_backward_input_nhwc(dys.data_ptr(), w.data_ptr(), dx.data_ptr(), CODE[dt], sh, st)
            c = L.dwconv_b200_backward_filter_nhwc(xs.data_ptr(), dys.data_ptr(), dw.data_ptr(), ws.data_ptr(),
                                                   nbytes, CODE[dt], sh, st)
        else:
            a = L.dwconv_b200_forward(xs.data_ptr(), w.data_ptr(), y.data_ptr(), CODE[dt], sh, st)
            b = L.dwconv_b200_backward_input(dys.data_ptr(), w.data_ptr(), dx.data_ptr(), CODE[dt], sh, st)
            c = L.dwconv_b200_backward_filter(xs.data_ptr(), dys.data_ptr(), dw.data_ptr(), ws.data_ptr(),
                                              nbytes, CODE[dt], sh, st)
        assert (a, b, c) == (0, 0, 0)

    ops(torch.cuda.current_stream().cuda_stream)   # eager: one-time set-up of every kernel
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        ops(torch.cuda.current_stream().cuda_stream)
    for seed in (31, 32):
        x2, _, dy2 = seeded((N, C, H, W), (k, k), s, p, dt, seed=seed)
        xs.copy_(x2.contiguous(memory_format=fmt))
        dys.copy_(dy2.contiguous(memory_format=fmt))
        y.fill_(float("nan")); dx.fill_(float("nan")); dw.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y.cpu(), oracle.forward_seq(x2, w, s, p))
        assert torch.equal(dx.cpu(), oracle.backward_input_seq(dy2, w, (H, W), s, p))
        assert_dw_close(dw, oracle.backward_filter(x2, dy2, (k, k), s, p), dt, "replayed dW")
    assert L.dwconv_b200_device_status() == 0
