"""The CPU oracle against the fixtures produced by running the reference package
(tests/golden/make_golden.py) -- this is what pins the oracle."""
import pytest
import torch

import oracle
from conftest import NP_DT, assert_close_fp, assert_dw_close, case_names, golden


@pytest.mark.parametrize("name", case_names())
def test_oracle_f64_matches_reference_outputs(name):
    g = golden()
    m, t = g.cases[name], g.tensors(name)
    dt = NP_DT[m["dtype"]]
    st, pd = tuple(m["stride"]), tuple(m["padding"])
    y = oracle.forward(t["x"], t["w"], st, pd)
    dx = oracle.backward_input(t["dy"], t["w"], (m["H"], m["W"]), st, pd)
    dw = oracle.backward_filter(t["x"], t["dy"], (m["kh"], m["kw"]), st, pd)
    assert tuple(y.shape) == tuple(t["y"].shape)
    if m["dist"] == "dyadic":
        # all products and partial sums are exact in fp32: equality, not tolerance
        assert torch.equal(y, t["y"].double())
        assert torch.equal(dx, t["dx"].double())
        assert torch.equal(dw, t["dw"].double())
        return
    assert_close_fp(t["y"], y, dt, m["kh"], m["kw"], "y")
    assert_close_fp(t["dx"], dx, dt, m["kh"], m["kw"], "dx")
    # the reference side (F.conv2d on CPU) accumulates dW in the storage dtype
    assert_dw_close(t["dw"], dw, dt, "dw")


@pytest.mark.parametrize("name", [n for n in case_names() if "f64" not in n])
def test_oracle_seq_matches_reference_outputs(name):
    g = golden()
    m, t = g.cases[name], g.tensors(name)
    dt = NP_DT[m["dtype"]]
    st, pd = tuple(m["stride"]), tuple(m["padding"])
    y = oracle.forward_seq(t["x"], t["w"], st, pd)
    dx = oracle.backward_input_seq(t["dy"], t["w"], (m["H"], m["W"]), st, pd)
    assert y.dtype == dt and dx.dtype == dt
    if m["dist"] == "dyadic":
        assert torch.equal(y, t["y"]) and torch.equal(dx, t["dx"])
    else:
        assert_close_fp(y, t["y"], dt, m["kh"], m["kw"], "y")
        assert_close_fp(dx, t["dx"], dt, m["kh"], m["kw"], "dx")
    # and against the fp64 ground truth, at the library's contract tolerance
    assert_close_fp(y, oracle.forward(t["x"], t["w"], st, pd), dt, m["kh"], m["kw"], "y/f64")
    assert_close_fp(dx, oracle.backward_input(t["dy"], t["w"], (m["H"], m["W"]), st, pd), dt,
                    m["kh"], m["kw"], "dx/f64")


@pytest.mark.parametrize("name", case_names())
def test_autograd_calls_of_the_reference_operator(name):
    """forward == operator(up=1, down=stride, pad) and backward-input ==
    operator(up=stride, down=1, g_pad, flipped) -- the two calls of dwconv.py:33-35,62-64."""
    g = golden()
    m, t = g.cases[name], g.tensors(name)
    st, pd = tuple(m["stride"]), tuple(m["padding"])
    k = (m["kh"], m["kw"])
    y = oracle.upfirdn(t["x"], t["w"], (1, 1), st, (pd[0], pd[0], pd[1], pd[1]), True)
    assert torch.equal(y, oracle.forward(t["x"], t["w"], st, pd))
    gp = oracle.g_pad((m["H"], m["W"]), tuple(y.shape[2:]), k, st, pd)
    dx = oracle.upfirdn(t["dy"], t["w"], st, (1, 1), gp, False)
    assert tuple(dx.shape[2:]) == (m["H"], m["W"])
    ref = oracle.backward_input(t["dy"], t["w"], (m["H"], m["W"]), st, pd)
    assert (dx - ref).abs().max().item() <= 1e-12 * max(1.0, ref.abs().max().item())


def test_use_small_truth_table():
    for H, W, kh, kw, sh, sw, ph, pw, want in golden().meta["use_small_table"]:
        assert oracle.use_small(H, W, kh, kw, (1, 1), (sh, sw), (ph, pw)) == bool(want), \
            (H, W, kh, kw, sh, sw, ph, pw)


def test_golden_small_flags_consistent():
    g = golden()
    for m in g.meta["cases"]:
        assert oracle.use_small(m["H"], m["W"], m["kh"], m["kw"], (1, 1), tuple(m["stride"]),
                                tuple(m["padding"])) == m["use_small"], m["name"]


def test_out_size_formula():
    # floor((H + 2p - k)/s) + 1 for every combination the fixtures use, via the
    # reference's expression (in*up + pad0 + pad1 - k + down)/down
    for H in range(1, 40):
        for k in (1, 2, 3, 5, 7):
            for s in (1, 2, 3):
                for p in (0, 1, 2, 3):
                    if H + 2 * p < k:
                        continue
                    assert oracle.conv_out(H, k, s, p) == (H + 2 * p - k) // s + 1


def test_linearity_and_adjoint_identity():
    """<conv(x,w), dy> == <x, dx> == <w, dW>: ties the three operators together."""
    gen = torch.Generator().manual_seed(7)
    for (N, C, H, W, k, s, p) in [(2, 3, 13, 11, 3, 2, 1), (1, 2, 9, 9, 5, 1, 2), (2, 2, 8, 10, 4, 3, 0)]:
        x = torch.randn(N, C, H, W, generator=gen, dtype=torch.float64)
        w = torch.randn(C, 1, k, k, generator=gen, dtype=torch.float64)
        y = oracle.forward(x, w, s, p)
        dy = torch.randn(y.shape, generator=gen, dtype=torch.float64)
        dx = oracle.backward_input(dy, w, (H, W), s, p)
        dw = oracle.backward_filter(x, dy, (k, k), s, p)
        a, b, c = (y * dy).sum().item(), (x * dx).sum().item(), (w * dw).sum().item()
        assert abs(a - b) <= 1e-10 * abs(a) + 1e-12 and abs(a - c) <= 1e-10 * abs(a) + 1e-12
