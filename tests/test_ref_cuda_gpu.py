"""The library against the reference's own CUDA kernels, run on the same GPU.

The unmodified reference extension (``oracle/_ref``, built by ``oracle/build_ref.py``) runs in a
child process (``oracle/ref_cuda.py``) on the seeded inputs written here; skipped when that
build is not present on this machine.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dwconv_b200
from conftest import ROOT

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(ROOT, "oracle", "_ref", "torch_dwconv", "_C.so")

# (x shape, k, stride, padding, dtype, served by the reference's kernels)
CASES = [
    ((4, 16, 14, 14), 3, 1, 1, np.float32, True),    # small-map kernel, 3x3
    ((2, 8, 7, 7), 3, 1, 1, np.float32, True),       # small-map kernel, odd height
    ((2, 8, 14, 14), 5, 1, 2, np.float32, True),     # small-map kernel, generic filter
    ((2, 8, 32, 32), 7, 1, 3, np.float32, True),
    ((2, 6, 56, 56), 3, 1, 1, np.float32, True),     # tiled kernel
    ((2, 6, 56, 56), 5, 2, 2, np.float32, True),     # tiled kernel, stride 2
    ((2, 4, 112, 112), 3, 2, 1, np.float32, True),
    ((2, 4, 40, 40), 7, 1, 3, np.float32, True),
    ((3, 5, 33, 47), 3, 1, 1, np.float32, True),     # rectangular map
    ((3, 5, 47, 33), 5, 2, 2, np.float32, True),
    ((2, 6, 56, 56), 7, 1, 3, np.float16, True),     # half: the reference accumulates in half
    ((2, 8, 28, 28), 3, 2, 1, np.float32, False),    # the reference sends this one to F.conv2d
]


@pytest.fixture(scope="module")
def reference_outputs(tmp_path_factory):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref is not built on this machine")
    tmp = tmp_path_factory.mktemp("refcuda")
    rng = np.random.default_rng(11)
    arrays = {}
    for i, (shape, k, s, p, dt, _) in enumerate(CASES):
        N, C, H, W = shape
        ho, wo = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        arrays[f"x{i}"] = rng.standard_normal(shape).astype(dt)
        arrays[f"w{i}"] = (rng.standard_normal((C, 1, k, k)) / k).astype(dt)
        arrays[f"dy{i}"] = rng.standard_normal((N, C, ho, wo)).astype(dt)
        arrays[f"sp{i}"] = np.array([s, p])
    fin, fout = str(tmp / "in.npz"), str(tmp / "out.npz")
    np.savez(fin, **arrays)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_cuda.py"),
                        "--cases", fin, "--out", fout], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return arrays, np.load(fout)


@pytest.mark.parametrize("i", range(len(CASES)))
def test_matches_reference_cuda_kernels(reference_outputs, i):
    arrays, ref = reference_outputs
    shape, k, s, p, dt, served = CASES[i]
    assert int(ref[f"served{i}"]) == int(served)
    if not served:
        return
    x = torch.from_numpy(arrays[f"x{i}"]).cuda().requires_grad_(True)
    w = torch.from_numpy(arrays[f"w{i}"]).cuda().requires_grad_(True)
    dy = torch.from_numpy(arrays[f"dy{i}"]).cuda()
    y = dwconv_b200.depthwise_conv2d(x, w, None, s, p)
    y.backward(dy)
    got = {"y": y.detach().cpu().numpy(), "dx": x.grad.cpu().numpy(), "dw": w.grad.cpu().numpy()}
    for name in ("y", "dx", "dw"):
        a, b = got[name].astype(np.float64), ref[f"{name}{i}"].astype(np.float64)
        assert a.shape == b.shape
        scale = max(1.0, np.abs(b).max())
        if dt == np.float16:
            tol = 1e-2 * scale * (4 if name == "dw" else 1)  # the reference adds in half
        elif name == "dw":
            tol = 1e-4 * scale       # the reference adds with float atomics, in any order
        else:
            tol = 0.0                # same taps, same order, one FMA each: identical bits
        err = np.abs(a - b).max()
        assert err <= tol, f"case {i} {name}: max abs diff {err} (tolerance {tol})"
