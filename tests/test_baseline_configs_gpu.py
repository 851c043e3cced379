"""The BASELINE configurations at full size.  The CPU oracle cannot run them whole in
seconds, so they are checked through properties that do not depend on size:

* sampled planes of y and dx are bit-identical to the sequential-order oracle;
* sampled channels of dW agree with the fp64 oracle over the whole batch;
* the adjoint identity <y, dy> == <x, dx> == <w, dW> ties the three operators together;
* a batch shard computed alone equals the same images inside the full batch (bit for bit).
"""
import pytest
import torch

import oracle
from conftest import assert_close_fp, assert_dw_close
from gpu_util import c_backward, c_backward_filter, c_backward_input, c_forward, make_shape

pytestmark = pytest.mark.gpu

# name: (N, C, H, k, stride, pad, dtype)
CONFIGS = {
    "c1": (8, 32, 56, 3, 1, 1, torch.float32),
    "c2": (128, 576, 14, 3, 1, 1, torch.float32),
    "c3a": (128, 32, 112, 3, 1, 1, torch.float32),
    "c3b": (128, 96, 112, 3, 2, 1, torch.float32),
    "c3c": (128, 144, 56, 5, 2, 2, torch.float32),
    "c3d": (128, 240, 28, 3, 2, 1, torch.float32),
    "c3e": (128, 480, 14, 5, 1, 2, torch.float32),
    "c3f": (128, 672, 14, 5, 2, 2, torch.float32),
    "c3g": (128, 1152, 7, 3, 1, 1, torch.float32),
    "c4a": (64, 96, 56, 7, 1, 3, torch.float16),
    "c4b": (64, 192, 28, 7, 1, 3, torch.float16),
    "c5k3": (32, 256, 32, 3, 1, 1, torch.float32),
    "c5k5": (32, 256, 32, 5, 1, 2, torch.float32),
    "c5k7": (32, 256, 32, 7, 1, 3, torch.float32),
    "c5k13": (32, 256, 32, 13, 1, 6, torch.float32),
    "c5k31": (32, 256, 32, 31, 1, 15, torch.float32),
}


def _draw(N, C, H, k, s, p, dt, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    sh = make_shape((N, C, H, H), (k, k), s, p)
    x = torch.randn((N, C, H, H), generator=g, device="cuda").to(dt)
    w = (torch.randn((C, 1, k, k), generator=g, device="cuda") / k).to(dt)
    dy = torch.randn((N, C, sh.Ho, sh.Wo), generator=g, device="cuda").to(dt)
    return x, w, dy


@pytest.mark.parametrize("name", list(CONFIGS))
def test_full_size_config(name):
    N, C, H, k, s, p, dt = CONFIGS[name]
    x, w, dy = _draw(N, C, H, k, s, p, dt, seed=list(CONFIGS).index(name))
    st, y = c_forward(x, w, s, p)
    assert st == 0
    st, dx = c_backward_input(dy, w, (H, H), s, p)
    assert st == 0
    st, dw = c_backward_filter(x, dy, (k, k), s, p)
    assert st == 0
    torch.cuda.synchronize()
    assert not torch.isnan(y).any() and not torch.isnan(dx).any() and not torch.isnan(dw).any()

    # both gradients from one pass over dy: dx the same bits, dW the same sum to rounding
    st, fdx, fdw = c_backward(x, dy, w, s, p)
    assert st == 0
    assert torch.equal(fdx, dx), f"{name}: fused dx differs"
    assert not torch.isnan(fdw).any()
    scale = dw.double().abs().max().item()
    assert (fdw.double() - dw.double()).abs().max().item() <= (2e-2 if dt == torch.float16 else 2e-4) * scale

    # sampled planes: first, last, and a seeded random handful
    g = torch.Generator().manual_seed(1)
    planes = sorted({0, 1, C - 1, C, N * C - 1, *torch.randint(0, N * C, (12,), generator=g).tolist()})
    for pl in planes:
        n, c = divmod(pl, C)
        xs, ws, dys = x[n:n + 1, c:c + 1], w[c:c + 1], dy[n:n + 1, c:c + 1]
        assert torch.equal(y[n:n + 1, c:c + 1].cpu(), oracle.forward_seq(xs, ws, s, p)), (name, pl)
        assert torch.equal(dx[n:n + 1, c:c + 1].cpu(),
                           oracle.backward_input_seq(dys, ws, (H, H), s, p)), (name, pl)
        assert_close_fp(y[n:n + 1, c:c + 1], oracle.forward(xs, ws, s, p), dt, k, k, "y")
        assert_close_fp(dx[n:n + 1, c:c + 1], oracle.backward_input(dys, ws, (H, H), s, p), dt, k,
                        k, "dx")

    # sampled channels of dW over the whole batch
    for c in sorted({0, C - 1, int(torch.randint(0, C, (1,), generator=g))}):
        truth = oracle.backward_filter(x[:, c:c + 1], dy[:, c:c + 1], (k, k), s, p)
        assert_dw_close(dw[c:c + 1], truth, dt, f"{name} dW[{c}]")

    # adjoint identity in fp64 on the device
    a = (y.double() * dy.double()).sum().item()
    b = (x.double() * dx.double()).sum().item()
    cc = (w.double() * dw.double()).sum().item()
    scale = (y.double().abs() * dy.double().abs()).sum().item()
    rel = 2e-3 if dt == torch.float16 else 1e-5
    assert abs(a - b) <= rel * scale and abs(a - cc) <= rel * scale, (a, b, cc)

    # a shard alone == the same images inside the batch
    if N >= 4:
        n0, n1 = N // 4, N // 2
        st, ys = c_forward(x[n0:n1].contiguous(), w, s, p)
        assert st == 0 and torch.equal(ys, y[n0:n1])
        st, dxs = c_backward_input(dy[n0:n1].contiguous(), w, (H, H), s, p)
        assert st == 0 and torch.equal(dxs, dx[n0:n1])
