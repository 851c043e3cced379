import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "depthwise-conv-pytorch_b200")
for p in (ROOT, PKG, os.path.join(PKG, "compat")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")
NP_DT = {"f32": torch.float32, "f16": torch.float16, "f64": torch.float64}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library and the compiled tensor-level module are built from source once per
    session (neither nvcc nor the C++ compiler needs a GPU)."""
    from build_dwconv_b200 import build_binding, build_library
    build_library()
    build_binding()


class Golden:
    def __init__(self):
        with open(os.path.join(GOLDEN, "ref_meta.json")) as f:
            self.meta = json.load(f)
        self.arrays = np.load(os.path.join(GOLDEN, "ref_cases.npz"))
        self.cases = {c["name"]: c for c in self.meta["cases"]}

    def tensors(self, name):
        return {k: torch.from_numpy(self.arrays[f"{name}/{k}"]) for k in
                ("x", "w", "dy", "y", "dx", "dw")}


_golden = None


def golden():
    global _golden
    if _golden is None:
        _golden = Golden()
    return _golden


def case_names():
    with open(os.path.join(GOLDEN, "ref_meta.json")) as f:
        return [c["name"] for c in json.load(f)["cases"]]


def tolerances(dtype, kh, kw):
    """(abs, rel) bounds for forward / backward-input against the fp64 ground truth:
    fp32 max-abs <= 1e-5*kh*kw, fp16 1e-2 relative (to the largest magnitude), fp64 1e-10."""
    if dtype == torch.float32:
        return 1e-5 * kh * kw, 0.0
    if dtype == torch.float16:
        return 0.0, 1e-2
    return 1e-10 * kh * kw, 0.0


def assert_close_fp(actual, truth, dtype, kh, kw, what=""):
    a = actual.detach().double().cpu()
    t = truth.detach().double().cpu()
    assert a.shape == t.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(t.shape)}"
    atol, rtol = tolerances(dtype, kh, kw)
    err = (a - t).abs().max().item() if a.numel() else 0.0
    bound = atol + rtol * max(t.abs().max().item(), 1.0)
    assert err <= bound, f"{what}: max abs err {err:.3e} > {bound:.3e}"


def assert_dw_close(actual, truth, dtype, what=""):
    """Filter gradient: 1e-4 relative to the largest true magnitude (fp16 output: 1e-2,
    its storage rounding alone is 2^-11)."""
    a = actual.detach().double().cpu()
    t = truth.detach().double().cpu()
    assert a.shape == t.shape
    rel = {torch.float32: 1e-4, torch.float16: 1e-2, torch.float64: 1e-10}[dtype]
    err = (a - t).abs().max().item()
    bound = rel * max(t.abs().max().item(), 1e-30)
    assert err <= bound, f"{what}: dW max abs err {err:.3e} > {bound:.3e}"
