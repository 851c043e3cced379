"""Times the reference's CPU route for the depthwise-conv path on the host cores.

Test/benchmark infrastructure (never part of the shipped library).  Run as a script by
``bench.py`` in a child process so that the reference package (import name
``torch_dwconv``, in ``oracle/_ref``) cannot shadow anything in the parent.

kind = "reference": ``torch_dwconv.DepthwiseConv2d(custom=False)`` forward + autograd
       backward on CPU tensors -- the reference's only CPU-executable route
       (torch_dwconv/dwconv.py:166-173; its CUDA operators reject CPU tensors,
       dwconv.cpp:24-25) -- with all host threads torch uses by default.
kind = "port": the C restatement in ``dwconv_oracle.c`` (OpenMP over planes), used when
       the reference extension is not available on this machine.

Prints one JSON object: seconds per step, images per step, threads, kind.
"""
import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def load_reference():
    ref_dir = os.path.join(HERE, "_ref")
    if not os.path.exists(os.path.join(ref_dir, "torch_dwconv", "_C.so")):
        return None
    sys.path.insert(0, ref_dir)
    try:
        import torch_dwconv  # noqa: F401
        return torch_dwconv
    except Exception as e:  # noqa: BLE001
        sys.stderr.write(f"[cpu_baseline] reference not importable: {e}\n")
        sys.path.remove(ref_dir)
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", required=True,
                    help="JSON list of [N, C, H, k, stride, pad, dtype] per layer")
    ap.add_argument("--images", type=int, required=True, help="images per step (sample of N)")
    ap.add_argument("--steps", type=int, default=0, help="timed steps (0: run for --seconds)")
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--seconds", type=float, default=10.0)
    ap.add_argument("--force-port", action="store_true")
    a = ap.parse_args()

    import torch
    # all the host cores, whatever the launcher put into OMP_NUM_THREADS (torchrun sets it to 1
    # for every rank it starts, which would make this a single-threaded figure)
    ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, ncpu))
    layers = json.loads(a.layers)
    ref = None if a.force_port else load_reference()
    dts = {"f32": torch.float32, "f16": torch.float16, "f64": torch.float64}
    work = []
    for i, (N, C, H, k, s, p, dt) in enumerate(layers):
        g = torch.Generator().manual_seed(i)
        n = min(a.images, N)
        x = torch.randn(n, C, H, H, generator=g).to(dts[dt])
        w = (torch.randn(C, 1, k, k, generator=g) / k).to(dts[dt])
        ho = (H + 2 * p - k) // s + 1
        dy = torch.randn(n, C, ho, ho, generator=g).to(dts[dt])
        work.append((x, w, dy, k, s, p, H))

    if ref is not None:
        kind, threads = "reference", torch.get_num_threads()
        mods = []
        for (x, w, dy, k, s, p, H) in work:
            m = ref.DepthwiseConv2d(x.shape[1], x.shape[1], k, stride=s, padding=p, custom=False)
            m.weight = torch.nn.Parameter(w.clone())
            mods.append(m)

        def step():
            for m, (x, w, dy, k, s, p, H) in zip(mods, work):
                xr = x.requires_grad_(True)
                xr.grad = None
                m.weight.grad = None
                m(xr).backward(dy)
    else:
        sys.path.insert(0, ROOT)
        import oracle
        kind, threads = "port", oracle.num_threads()

        def step():
            for (x, w, dy, k, s, p, H) in work:
                oracle.forward_seq(x.float(), w.float(), s, p)
                oracle.backward_input_seq(dy.float(), w.float(), (H, H), s, p)
                oracle.backward_filter(x, dy, (k, k), s, p)

    for _ in range(max(a.warmup, 1)):
        step()
    times = []
    t_end = time.perf_counter() + a.seconds
    while True:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if a.steps > 0 and len(times) >= a.steps:
            break
        if a.steps == 0 and time.perf_counter() >= t_end:
            break
    print(json.dumps({"kind": kind, "threads": threads, "cpu_count": os.cpu_count(),
                      "images": min(a.images, layers[0][0]), "steps": len(times),
                      "mean_s": sum(times) / len(times), "best_s": min(times)}))


if __name__ == "__main__":
    main()
