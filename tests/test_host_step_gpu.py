"""HostMapsStep (pinned host maps, chunked three-stream pipeline) against the one-call path."""
import pytest
import torch

import dwconv_b200

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,k,s,p,dtype,chunk", [
    ((13, 24, 14, 14), 3, 1, 1, torch.float32, 4),     # ragged last chunk
    ((8, 16, 28, 28), 3, 2, 1, torch.float32, None),   # default chunking: one chunk
    ((9, 8, 17, 17), 5, 1, 2, torch.float16, 2),
    ((6, 4, 12, 12), 7, 1, 3, torch.float64, 1),
    ((5, 32, 56, 56), 3, 1, 1, torch.float32, 1),
    ((40, 64, 28, 28), 3, 1, 1, torch.float32, None),  # default chunking: 11, 11, 11, 7
])
def test_host_step_matches_one_call(shape, k, s, p, dtype, chunk):
    g = torch.Generator().manual_seed(5)
    N, C, H, W = shape
    x = torch.randn(shape, generator=g).to(dtype).pin_memory()
    w = (torch.randn((C, 1, k, k), generator=g) / k).to(dtype).pin_memory()
    step = dwconv_b200.HostMapsStep(shape, k, s, p, dtype=dtype, device="cuda:0", chunk_images=chunk)
    dy = torch.randn(step.y_shape, generator=g).to(dtype).pin_memory()
    y = torch.empty(step.y_shape, dtype=dtype).pin_memory()
    dx = torch.empty(shape, dtype=dtype).pin_memory()
    dw = torch.empty_like(w).pin_memory()

    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    yd = dwconv_b200.depthwise_conv2d(xd, wd, None, s, p)
    yd.backward(dy.cuda())

    for _ in range(3):  # eager, then recorded into a CUDA graph, then replayed
        y.fill_(float("nan")); dx.fill_(float("nan")); dw.fill_(float("nan"))
        step.run(x, w, dy, y, dx, dw)
        step.synchronize()
        assert torch.equal(y, yd.detach().cpu())
        assert torch.equal(dx, xd.grad.cpu())
        ref = wd.grad.double().cpu()
        tol = {torch.float32: 1e-4, torch.float16: 1e-2, torch.float64: 1e-10}[dtype]
        assert (dw.double() - ref).abs().max() <= tol * max(1.0, ref.abs().max().item())


def test_host_step_rejects_pageable_and_wrong_shape():
    step = dwconv_b200.HostMapsStep((2, 4, 8, 8), 3, 1, 1, device="cuda:0")
    mk = lambda s: torch.zeros(s).pin_memory()  # noqa: E731
    x, w, dy, y, dx, dw = mk((2, 4, 8, 8)), mk((4, 1, 3, 3)), mk((2, 4, 8, 8)), mk((2, 4, 8, 8)), \
        mk((2, 4, 8, 8)), mk((4, 1, 3, 3))
    with pytest.raises(RuntimeError, match="pinned"):
        step.run(torch.zeros(2, 4, 8, 8), w, dy, y, dx, dw)
    with pytest.raises(RuntimeError, match="shape"):
        step.run(x, w, mk((2, 4, 7, 7)), y, dx, dw)
    step.run(x, w, dy, y, dx, dw)
    step.synchronize()
    assert float(y.abs().max()) == 0.0


def test_host_pipeline_overlaps_steps_and_keeps_their_results_apart():
    """HostMapsPipeline: consecutive steps on alternating HostMapsStep objects and streams.  Six
    steps with different inputs, two in flight at a time, each with its own host buffers: every
    step's results equal the one-call path's on that step's inputs."""
    shape, k, s, p, dtype = (12, 16, 28, 28), 3, 1, 1, torch.float32
    N, C, H, W = shape
    pipe = dwconv_b200.HostMapsPipeline(shape, k, s, p, depth=2, dtype=dtype, device="cuda:0",
                                        chunk_images=4)
    g = torch.Generator().manual_seed(11)
    steps = []
    for i in range(6):
        x = torch.randn(shape, generator=g).pin_memory()
        w = (torch.randn((C, 1, k, k), generator=g) / k).pin_memory()
        dy = torch.randn(pipe.y_shape, generator=g).pin_memory()
        outs = [torch.full(pipe.y_shape, float("nan")).pin_memory(),
                torch.full(shape, float("nan")).pin_memory(),
                torch.full((C, 1, k, k), float("nan")).pin_memory()]
        steps.append((x, w, dy, outs))
    events = [pipe.run(x, w, dy, *outs) for x, w, dy, outs in steps]
    for ev, (x, w, dy, (y, dx, dw)) in zip(events, steps):
        pipe.wait(ev)
        xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
        yd = dwconv_b200.depthwise_conv2d(xd, wd, None, s, p)
        yd.backward(dy.cuda())
        assert torch.equal(y, yd.detach().cpu())
        assert torch.equal(dx, xd.grad.cpu())
        ref = wd.grad.double().cpu()
        assert (dw.double() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    pipe.synchronize()
    assert dwconv_b200._lib.lib.dwconv_b200_device_status() == 0
