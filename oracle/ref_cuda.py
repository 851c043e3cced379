"""Runs the reference's own CUDA route (package ``torch_dwconv`` in ``oracle/_ref``) on a GPU.

Test/benchmark infrastructure (never part of the shipped library).  Always run as a child
process, because the reference must be imported under its own name ``torch_dwconv``.

Two uses:

* ``--cases in.npz --out out.npz``: for every case ``i`` in the file (arrays ``x{i}``, ``w{i}``,
  ``dy{i}``, ``sp{i}`` = [stride, padding]) compute ``y``, ``dx``, ``dw`` through
  ``torch_dwconv.depthwise_conv2d`` + autograd (torch_dwconv/dwconv.py:115-131, :15-73) on
  CUDA tensors and store them.  The GPU parity tests compare the library with these.
* ``--time --layers JSON``: CUDA-event timing of the same route (forward alone; forward +
  backward) over rotating buffer sets larger than L2, printed as one JSON object, for context
  beside the library's numbers.

Shapes outside the reference's CUDA kernels are refused here rather than passed on: its
dispatcher serves square filters 3, 5, 7 with stride 1 or 2 (torch_dwconv/dwconv_kernel.cu:808-845)
and sends small maps it cannot serve to ``F.conv2d`` (dwconv.py:125-128), which would not be the
reference's kernels any more.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference():
    ref_dir = os.path.join(HERE, "_ref")
    if not os.path.exists(os.path.join(ref_dir, "torch_dwconv", "_C.so")):
        return None
    sys.path.insert(0, ref_dir)
    import torch_dwconv
    return torch_dwconv


def served_by_reference_kernels(ref, x, w, stride, padding):
    """True when ``depthwise_conv2d`` runs the reference's CUDA kernels for this problem."""
    k = w.shape[2]
    if w.shape[2] != w.shape[3] or k not in (3, 5, 7) or stride not in (1, 2):
        return False
    small = ref.dwconv.use_dwconv2d_small(x, w, (1, 1), (stride, stride), (padding, padding))
    if not small and x.shape[2] <= 32 and x.shape[3] <= 32:
        return False  # the F.conv2d branch
    return True


def run_cases(ref, path_in, path_out):
    import numpy as np
    import torch
    data = np.load(path_in)
    out = {}
    n = len([k for k in data.files if k.startswith("x")])
    for i in range(n):
        stride, padding = (int(v) for v in data[f"sp{i}"])
        x = torch.from_numpy(data[f"x{i}"]).cuda().requires_grad_(True)
        w = torch.from_numpy(data[f"w{i}"]).cuda().requires_grad_(True)
        dy = torch.from_numpy(data[f"dy{i}"]).cuda()
        if not served_by_reference_kernels(ref, x, w, stride, padding):
            out[f"served{i}"] = np.array(0)
            continue
        y = ref.depthwise_conv2d(x, w, None, stride, padding)
        y.backward(dy)
        torch.cuda.synchronize()
        out[f"served{i}"] = np.array(1)
        out[f"y{i}"] = y.detach().cpu().numpy()
        out[f"dx{i}"] = x.grad.cpu().numpy()
        out[f"dw{i}"] = w.grad.cpu().numpy()
    np.savez(path_out, **out)


def time_layers(ref, layers, reps):
    import torch
    dts = {"f32": torch.float32, "f16": torch.float16}
    res = []
    for layer in layers:
        if len(layer) == 8:   # rectangular map: [N, C, H, W, k, stride, pad, dtype]
            N, C, H, W, k, s, p, dt = layer
        else:                 # square map: [N, C, H, k, stride, pad, dtype]
            N, C, H, k, s, p, dt = layer
            W = H
        ho, wo = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        per_set = 2 * N * C * (H * W + ho * wo) * (2 if dt == "f16" else 4)
        n_sets = max(2, min(8, int(2 * 126e6 // per_set) + 2))
        sets = []
        for si in range(n_sets):
            g = torch.Generator(device="cuda").manual_seed(si)
            x = torch.randn((N, C, H, W), generator=g, device="cuda").to(dts[dt]).requires_grad_(True)
            w = (torch.randn((C, 1, k, k), generator=g, device="cuda") / k).to(dts[dt]).requires_grad_(True)
            dy = torch.randn((N, C, ho, wo), generator=g, device="cuda").to(dts[dt])
            sets.append((x, w, dy))
        if not served_by_reference_kernels(ref, sets[0][0], sets[0][1], s, p):
            res.append({"layer": list(layer), "served": False})
            continue

        def fwd(i):
            x, w, dy = sets[i % n_sets]
            with torch.no_grad():
                ref.depthwise_conv2d(x, w, None, s, p)

        def fwd_bwd(i):
            x, w, dy = sets[i % n_sets]
            x.grad = None
            w.grad = None
            ref.depthwise_conv2d(x, w, None, s, p).backward(dy)

        times = {}
        for name, fn in (("forward", fwd), ("forward_backward", fwd_bwd)):
            for i in range(3):
                fn(i)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for i in range(reps):
                fn(i)
            z.record()
            torch.cuda.synchronize()
            times[name] = a.elapsed_time(z) / reps
        res.append({"layer": list(layer), "served": True,
                    "forward_ms": round(times["forward"], 5),
                    "forward_backward_ms": round(times["forward_backward"], 5),
                    "buffer_sets": n_sets})
        del sets
        torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases")
    ap.add_argument("--out")
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--layers", help="JSON list of [N, C, H, k, stride, pad, dtype] or "
                                     "[N, C, H, W, k, stride, pad, dtype]")
    ap.add_argument("--reps", type=int, default=50)
    a = ap.parse_args()
    ref = load_reference()
    if ref is None:
        print(json.dumps({"unavailable": "oracle/_ref/torch_dwconv/_C.so not built"}))
        return 3
    if a.cases:
        run_cases(ref, a.cases, a.out)
        return 0
    if a.time:
        print(json.dumps({"impl": "reference CUDA kernels (torch_dwconv, unmodified, sm_100)",
                          "layers": time_layers(ref, json.loads(a.layers), a.reps)}))
        return 0
    ap.error("nothing to do")


if __name__ == "__main__":
    sys.exit(main())
