"""Generate tests/golden/*.npz|json by RUNNING THE REFERENCE PACKAGE on CPU.

Run once in a container that has the reference checkout:

    python oracle/build_ref.py            # builds oracle/_ref/torch_dwconv
    python tests/golden/make_golden.py

The reference's CUDA operators reject CPU tensors (torch_dwconv/dwconv.cpp:24-25),
so its CPU-executable routes are used, each exactly as a caller reaches it:

* route "fallback": ``torch_dwconv.depthwise_conv2d`` on maps <= 32x32 that its
  small-map test refuses (dwconv.py:123-128) -- forward and autograd backward;
* route "module":   ``torch_dwconv.DepthwiseConv2d(custom=False)``
  (dwconv.py:166-173) with its weight overwritten by the seeded filter;
* host logic:       ``torch_dwconv._C.use_dwconv2d_small`` (no device check,
  dwconv.cpp:61) over a grid of shapes, ``make_tuple`` results and the
  ``ValueError`` texts of ``check_options`` / ``make_tuple``.

Inputs are stored with the outputs, so the fixtures do not depend on a torch
RNG stream.  "dyadic" cases draw multiples of 1/8 (filters: 1/4) so that every
product and partial sum is exact in fp32: any summation order must reproduce
them bit for bit.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))

import torch_dwconv  # noqa: E402  (the reference, from oracle/_ref)
from torch_dwconv.dwconv import check_options, make_tuple  # noqa: E402

assert "oracle/_ref" in torch_dwconv.__file__.replace(os.sep, "/")

# name, N, C, H, W, kh, kw, stride, padding, dtype, dist
CASES = [
    # scaled-down BASELINE shapes (same H, W, k, stride, padding; fewer planes)
    ("c1_56_k3s1", 1, 2, 56, 56, 3, 3, 1, 1, "f32", "randn"),
    ("c2_14_k3s1", 2, 4, 14, 14, 3, 3, 1, 1, "f32", "randn"),
    ("c3a_112_k3s1", 1, 1, 112, 112, 3, 3, 1, 1, "f32", "dyadic"),
    ("c3b_112_k3s2", 1, 1, 112, 112, 3, 3, 2, 1, "f32", "dyadic"),
    ("c3c_56_k5s2", 1, 2, 56, 56, 5, 5, 2, 2, "f32", "randn"),
    ("c3d_28_k3s2", 2, 3, 28, 28, 3, 3, 2, 1, "f32", "randn"),
    ("c3e_14_k5s1", 2, 4, 14, 14, 5, 5, 1, 2, "f32", "randn"),
    ("c3f_14_k5s2", 2, 4, 14, 14, 5, 5, 2, 2, "f32", "randn"),
    ("c3g_7_k3s1", 3, 5, 7, 7, 3, 3, 1, 1, "f32", "randn"),
    ("c4a_56_k7_f16", 1, 2, 56, 56, 7, 7, 1, 3, "f16", "randn"),
    ("c4b_28_k7_f16", 2, 2, 28, 28, 7, 7, 1, 3, "f16", "randn"),
    ("c5_32_k3", 1, 3, 32, 32, 3, 3, 1, 1, "f32", "randn"),
    ("c5_32_k5", 1, 3, 32, 32, 5, 5, 1, 2, "f32", "randn"),
    ("c5_32_k7", 1, 3, 32, 32, 7, 7, 1, 3, "f32", "randn"),
    ("c5_32_k13", 1, 3, 32, 32, 13, 13, 1, 6, "f32", "randn"),
    ("c5_32_k31", 1, 2, 32, 32, 31, 31, 1, 15, "f32", "randn"),
    # the shape classes of the reference's own tests (test_forward.py, test_grad.py)
    ("t_64_k3s1p1", 1, 1, 64, 64, 3, 3, 1, 1, "f32", "dyadic"),
    ("t_64_k5s2p2", 1, 1, 64, 64, 5, 5, 2, 2, "f32", "dyadic"),
    ("t_63x65_k3s2p1", 1, 2, 63, 65, 3, 3, 2, 1, "f32", "randn"),
    ("t_63x65_k5s1p2", 1, 2, 63, 65, 5, 5, 1, 2, "f32", "randn"),
    ("t_34_k3s2p0_f64", 2, 2, 34, 34, 3, 3, 2, 0, "f64", "randn"),
    ("t_33x35_k5s2p2_f64", 2, 2, 33, 35, 5, 5, 2, 2, "f64", "randn"),
    ("t_16_k5s1p2_f64", 2, 2, 16, 16, 5, 5, 1, 2, "f64", "randn"),
    # edges: 1x1 filter, filter larger than the map, stride 3, rectangular
    # filter, tuple stride / padding, no padding with a ragged last window
    ("e_k1", 2, 3, 9, 10, 1, 1, 1, 0, "f32", "randn"),
    ("e_k_gt_map", 1, 2, 5, 5, 7, 7, 1, 3, "f32", "randn"),
    ("e_s3", 1, 2, 17, 19, 3, 3, 3, 1, "f32", "randn"),
    ("e_rect_3x5", 1, 2, 12, 13, 3, 5, 1, (1, 2), "f32", "randn"),
    ("e_tuple_s21_p01", 1, 2, 15, 14, 3, 3, (2, 1), (0, 1), "f32", "randn"),
    ("e_ragged_s2p0", 1, 2, 10, 10, 3, 3, 2, 0, "f32", "randn"),
    ("e_pad_ge_k", 1, 1, 6, 6, 3, 3, 1, 3, "f32", "randn"),
    ("e_1x1_map", 3, 2, 1, 1, 3, 3, 1, 1, "f32", "randn"),
]

DT = {"f32": torch.float32, "f16": torch.float16, "f64": torch.float64}


def draw(gen, shape, dist, scale=1.0):
    if dist == "dyadic":
        return torch.randint(-16, 17, shape, generator=gen).float() / 8.0
    return torch.randn(shape, generator=gen) * scale


def run_case(idx, case):
    name, N, C, H, W, kh, kw, stride, padding, dt, dist = case
    gen = torch.Generator().manual_seed(idx)
    x = draw(gen, (N, C, H, W), dist)
    if dist == "dyadic":
        w = torch.randint(-4, 5, (C, 1, kh, kw), generator=gen).float() / 4.0
    else:
        w = torch.randn((C, 1, kh, kw), generator=gen) / (kh * kw) ** 0.5
    x = x.to(DT[dt])
    w = w.to(DT[dt])
    st = make_tuple(stride, 2)
    pd = make_tuple(padding, 2)
    small = torch_dwconv._C.use_dwconv2d_small(x, w, 1, 1, st[0], st[1], pd[0], pd[1])
    xr = x.clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    square = kh == kw
    if (not small) and H <= 32 and W <= 32:
        route = "fallback"
        y = torch_dwconv.depthwise_conv2d(xr, wr, None, stride, padding)
    else:
        route = "module"
        mod = torch_dwconv.DepthwiseConv2d(C, C, kh if square else max(kh, kw), stride=stride,
                                           padding=padding, custom=False)
        mod.weight = torch.nn.Parameter(wr.detach().clone())
        wr = mod.weight
        y = mod(xr)
    dy = draw(gen, tuple(y.shape), dist).to(DT[dt])
    y.backward(dy)
    out = {
        "x": x, "w": w, "dy": dy, "y": y.detach(), "dx": xr.grad, "dw": wr.grad,
    }
    meta = {"name": name, "N": N, "C": C, "H": H, "W": W, "kh": kh, "kw": kw,
            "stride": list(st), "padding": list(pd), "dtype": dt, "dist": dist,
            "route": route, "use_small": bool(small), "seed": idx}
    return meta, out


def small_table():
    """Truth table of the reference's small-map eligibility (host-only logic)."""
    rows = []
    w_cache = {}
    for H in (1, 3, 7, 14, 15, 32, 33):
        for W in (1, 7, 14, 32, 33):
            for k in (1, 2, 3, 5, 7, 13, 31):
                for s in (1, 2):
                    for p in (0, 1, k // 2, k - 1, k):
                        x = torch.empty(1, 1, H, W)
                        w = w_cache.setdefault(k, torch.empty(1, 1, k, k))
                        r = torch_dwconv._C.use_dwconv2d_small(x, w, 1, 1, s, s, p, p)
                        rows.append([H, W, k, k, s, s, p, p, int(r)])
    # rectangular filters / mixed strides / mixed pads
    for (H, W, kh, kw, sh, sw, ph, pw) in [(14, 14, 3, 5, 1, 1, 1, 2), (14, 14, 5, 3, 1, 1, 2, 1),
                                           (14, 28, 3, 3, 1, 2, 1, 1), (32, 32, 7, 3, 1, 1, 3, 1),
                                           (8, 32, 3, 3, 1, 1, 1, 1), (32, 8, 3, 3, 1, 1, 1, 1),
                                           (3, 3, 3, 3, 1, 1, 1, 1), (2, 2, 3, 3, 1, 1, 1, 1)]:
        r = torch_dwconv._C.use_dwconv2d_small(torch.empty(1, 1, H, W), torch.empty(1, 1, kh, kw),
                                               1, 1, sh, sw, ph, pw)
        rows.append([H, W, kh, kw, sh, sw, ph, pw, int(r)])
    return rows


def error_texts():
    out = {}

    def grab(key, fn):
        try:
            fn()
            out[key] = None
        except Exception as e:  # noqa: BLE001
            out[key] = [type(e).__name__, str(e)]

    grab("dilation", lambda: check_options(4, 4, 2, None, None))
    grab("groups", lambda: check_options(4, 4, 1, 2, None))
    grab("channels", lambda: check_options(4, 8, 1, None, None))
    grab("bias", lambda: check_options(4, 4, 1, None, True))
    grab("padding_mode", lambda: check_options(4, 4, 1, None, None, "reflect"))
    grab("tuple_len", lambda: make_tuple((1, 2, 3), 2))
    grab("cpu_tensor", lambda: torch_dwconv.depthwise_conv2d(torch.zeros(1, 2, 40, 40),
                                                             torch.zeros(2, 1, 3, 3)))
    out["make_tuple"] = {
        "int": list(make_tuple(3, 2)), "list1": list(make_tuple([3], 2)),
        "tuple2": list(make_tuple((1, 2), 2)),
    }
    return out


def main():
    arrays, metas = {}, []
    for idx, case in enumerate(CASES):
        meta, out = run_case(idx, case)
        metas.append(meta)
        for k, v in out.items():
            arrays[f"{meta['name']}/{k}"] = v.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_cases.npz"), **arrays)
    with open(os.path.join(HERE, "ref_meta.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": metas, "use_small_table": small_table(),
                   "errors": error_texts()}, f, indent=0, separators=(",", ":"))
    print("cases:", len(metas), "routes:", {m["route"] for m in metas})


if __name__ == "__main__":
    main()
