"""StackStep (static buffers, C entry points, CUDA graph) against the modules under autograd."""
import pytest
import torch

import dwconv_b200

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_stack_step_equals_autograd(dtype):
    spec = ((8, 16, 3, 1), (12, 16, 5, 2), (6, 9, 3, 2), (4, 30, 7, 1))
    torch.manual_seed(4)
    stack = dwconv_b200.DepthwiseStack(spec).to(device="cuda", dtype=dtype)
    step = dwconv_b200.StackStep(stack, batch=5, device="cuda:0")
    for x, dy in zip(step.x, step.dy):
        x.copy_(torch.randn(x.shape, device="cuda"))
        dy.copy_(torch.randn(dy.shape, device="cuda"))
    xs = [x.clone().requires_grad_(True) for x in step.x]
    ys = stack(xs)
    torch.autograd.backward(ys, [dy.clone() for dy in step.dy])
    for _ in range(3):  # eager, recorded, replayed
        for t in step.y + step.dx + step.dw:
            t.fill_(float("nan"))
        step.run()
        torch.cuda.synchronize()
        for i, layer in enumerate(stack.layers):
            assert torch.equal(step.y[i], ys[i].detach())
            assert torch.equal(step.dx[i], xs[i].grad)
            assert torch.equal(step.dw[i], layer.weight.grad)
    assert step.images_per_second(steps=5, warmup=2) > 0


def test_from_conv2d_matches_torch_on_gpu():
    conv = torch.nn.Conv2d(10, 10, 3, stride=1, padding=1, groups=10, bias=False).cuda()
    m = dwconv_b200.from_conv2d(conv)
    x = torch.randn(3, 10, 14, 14, device="cuda")
    assert (m(x) - conv(x)).abs().max().item() <= 1e-5 * 9
