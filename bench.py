#!/usr/bin/env python
"""Benchmark of the depthwise-conv2d hot path (forward + backward-input + backward-filter).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl b200|reference]

One "step" is one pass of the three operators over one batch of seeded synthetic data of the
named workload (per-GPU batch fixed: weak scaling; with N > 1 each step also sums the filter
gradient over ranks with one all-reduce).  Rank 0 prints ONE JSON line:

* ``value``      algorithmic GB/s, inputs resident in HBM, device-timed (CUDA events), max over
                 ranks; algorithmic bytes per step = 3 * (|x| + |y| + |w|) summed over layers;
* ``e2e``        the same metric through the public Python API with pinned HOST buffers:
                 host->device copies of x, w, dy and device->host copies of y, dx, dW inside
                 the timed region;
* ``roofline``   the slowest of the three operators, timed alone with CUDA events, against
                 the measured HBM copy bandwidth (MEASURED_PEAKS.json);
* ``cpu_baseline`` the reference's CPU route timed on this machine's host cores (rank 0);
* ``clocks``     SM clock / throttle reasons sampled with nvidia-smi while the GPU was loaded;
* ``timing_spread`` median and best of 60 steps timed one by one, and the L2-warm step (one
                 buffer set reused), beside the headline mean over the rotating sets.

``--impl reference`` times only the reference's CPU route (see oracle/cpu_baseline.py) and
prints the same line with ``"impl": "reference"``.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "depthwise-conv-pytorch_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

# layer = (N, C, H(=W), k, stride, pad, dtype); batch sizes are per GPU
WORKLOADS = {
    "c1": [(8, 32, 56, 3, 1, 1, "f32")],
    "c2": [(128, 576, 14, 3, 1, 1, "f32")],
    "c3": [(128, 32, 112, 3, 1, 1, "f32"), (128, 96, 112, 3, 2, 1, "f32"),
           (128, 144, 56, 5, 2, 2, "f32"), (128, 240, 28, 3, 2, 1, "f32"),
           (128, 480, 14, 5, 1, 2, "f32"), (128, 672, 14, 5, 2, 2, "f32"),
           (128, 1152, 7, 3, 1, 1, "f32")],
    "c3a": [(128, 32, 112, 3, 1, 1, "f32")], "c3b": [(128, 96, 112, 3, 2, 1, "f32")],
    "c3c": [(128, 144, 56, 5, 2, 2, "f32")], "c3d": [(128, 240, 28, 3, 2, 1, "f32")],
    "c3e": [(128, 480, 14, 5, 1, 2, "f32")], "c3f": [(128, 672, 14, 5, 2, 2, "f32")],
    "c3g": [(128, 1152, 7, 3, 1, 1, "f32")],
    "c4a": [(64, 96, 56, 7, 1, 3, "f16")],
    "c4b": [(64, 192, 28, 7, 1, 3, "f16")],
    "c5k3": [(32, 256, 32, 3, 1, 1, "f32")],
    "c5k5": [(32, 256, 32, 5, 1, 2, "f32")],
    "c5k7": [(32, 256, 32, 7, 1, 3, "f32")],
    "c5k13": [(32, 256, 32, 13, 1, 6, "f32")],
    "c5k31": [(32, 256, 32, 31, 1, 15, "f32")],
}
DESCR = {
    "c1": "single depthwise conv N8 C32 56x56 k3 s1 p1 fp32",
    "c2": "MobileNetV2-style small-map layer N128 C576 14x14 k3 s1 p1 fp32",
    "c3": "EfficientNet-B0 depthwise stack, 7 layers, N128 fp32",
    "c4a": "ConvNeXt-T-style 7x7 N64 C96 56x56 fp16 (fp32 accumulate)",
    "c4b": "ConvNeXt-T-style 7x7 N64 C192 28x28 fp16 (fp32 accumulate)",
}
ESIZE = {"f32": 4, "f16": 2, "f64": 8}
METRIC = "dwconv_fwd_bwd_achieved_hbm_gbps"
UNIT = "GB/s"
L2_BYTES = 126e6


def out_hw(H, k, s, p):
    return (H + 2 * p - k) // s + 1


def layer_bytes(layer, n=None):
    """(|x|, |y|, |w|) in bytes."""
    N, C, H, k, s, p, dt = layer
    n = N if n is None else n
    ho = out_hw(H, k, s, p)
    b = ESIZE[dt]
    return n * C * H * H * b, n * C * ho * ho * b, C * k * k * b


def step_bytes(layers, n=None):
    return sum(3 * sum(layer_bytes(l, n)) for l in layers)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU route in a child process
# --------------------------------------------------------------------------------------
def run_cpu_route(layers, images, steps, warmup, seconds):
    cmd = [sys.executable, os.path.join(ROOT, "oracle", "cpu_baseline.py"),
           "--layers", json.dumps(layers), "--images", str(images), "--steps", str(steps),
           "--warmup", str(warmup), "--seconds", str(seconds)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=1800)
    if res.returncode != 0:
        raise RuntimeError("cpu_baseline.py failed: " + res.stderr[-400:])
    return json.loads(res.stdout.strip().splitlines()[-1])


def cpu_baseline_entry(layers, r):
    n = r["images"]
    val = step_bytes(layers, n) / r["mean_s"] / 1e9
    what = ("torch_dwconv.DepthwiseConv2d(custom=False) fwd + autograd bwd on CPU tensors"
            if r["kind"] == "reference" else "C oracle port (OpenMP)")
    return {"value": round(val, 3), "unit": UNIT, "cores": r["threads"], "kind": r["kind"],
            "host_cpus": r["cpu_count"], "ms_per_step": round(r["mean_s"] * 1e3, 3),
            "sample": f"{n} of {layers[0][0]} images per layer, {r['steps']} steps, mean; {what}"}


def reference_arm(args, layers):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    N = layers[0][0]
    # calibrate on a few images so that steps+warmup stay within ~2 minutes
    probe = run_cpu_route(layers, min(8, N), 2, 1, 0)
    per_img = probe["mean_s"] / probe["images"]
    budget = 120.0 / max(1, args.steps + args.warmup)
    images = int(max(1, min(N, budget / per_img)))
    r = run_cpu_route(layers, images, args.steps, max(1, args.warmup), 0)
    entry = cpu_baseline_entry(layers, r)
    line = {
        "impl": "reference", "metric": METRIC, "value": entry["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": entry["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": layers[0][6], "data": "synthetic (seeded N(0,1))",
        "config": {"workload": f"{args.workload}: {DESCR.get(args.workload, args.workload)}",
                   "images_per_step": images},
        "cpu_baseline": entry,
        "e2e": {"value": entry["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.samples = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        for t, line in self.samples:
            if not (t0 <= t <= t1):
                continue
            f = [v.strip() for v in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                smax = float(f[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def gpu_arm(args, layers):
    import torch
    import torch.distributed as dist
    import dwconv_b200
    from dwconv_b200 import _lib
    from dwconv_b200.dist import FilterGradReducer, PeerFilterExchange, bind_to_gpu_numa_node

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # before any pinned host buffer exists: keep this rank on its GPU's NUMA node
    numa = bind_to_gpu_numa_node(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=90))
    L = _lib.lib
    tdt = {"f32": torch.float32, "f16": torch.float16, "f64": torch.float64}
    code = {"f32": _lib.F32, "f16": _lib.F16, "f64": _lib.F64}

    # ---- buffers: enough rotating sets that >= 2 x L2 is touched between reuses ----------
    per_set = sum(2 * (bx + by) for bx, by, _ in map(layer_bytes, layers))  # x, dx, y, dy
    n_sets = max(2, min(8, int(2 * L2_BYTES // per_set) + 2))
    sets = []
    for si in range(n_sets):
        bufs = []
        for li, (N, C, H, k, s, p, dt) in enumerate(layers):
            g = torch.Generator(device=dev).manual_seed(1000 * rank + 10 * li + si)
            ho = out_hw(H, k, s, p)
            x = torch.randn((N, C, H, H), generator=g, device=dev).to(tdt[dt])
            w = (torch.randn((C, 1, k, k), generator=g, device=dev) / k).to(tdt[dt])
            dy = torch.randn((N, C, ho, ho), generator=g, device=dev).to(tdt[dt])
            shape = _lib.Shape(N, C, H, H, k, k, s, s, p, p, ho, ho)
            nws = L.dwconv_b200_backward_filter_workspace_bytes(code[dt], shape)
            bufs.append(dict(x=x, w=w, dy=dy, y=torch.empty_like(dy), dx=torch.empty_like(x),
                             dw=torch.empty_like(w), ws=torch.empty(nws, dtype=torch.uint8, device=dev),
                             nws=nws, shape=shape, code=code[dt]))
        sets.append(bufs)

    def op_forward(b, st):
        _lib.check(L.dwconv_b200_forward(b["x"].data_ptr(), b["w"].data_ptr(), b["y"].data_ptr(),
                                         b["code"], b["shape"], st), "forward")

    def op_backward_input(b, st):
        _lib.check(L.dwconv_b200_backward_input(b["dy"].data_ptr(), b["w"].data_ptr(),
                                                b["dx"].data_ptr(), b["code"], b["shape"], st),
                   "backward_input")

    def op_backward_filter(b, st):
        _lib.check(L.dwconv_b200_backward_filter(b["x"].data_ptr(), b["dy"].data_ptr(),
                                                 b["dw"].data_ptr(), b["ws"].data_ptr(), b["nws"],
                                                 b["code"], b["shape"], st), "backward_filter")

    # N > 1: the filter gradient is summed over the GPUs inside its second pass (peer stores over
    # NVLink, one exchange object per layer); if peer mapping is not possible on this machine the
    # step falls back to one NCCL all-reduce of the packed gradients on a side stream
    exchanges = None
    if world > 1 and not args.nccl_reduce:
        try:
            exchanges = [PeerFilterExchange(C, k, tdt[dt], dev) for (N, C, H, k, s, p, dt) in layers]
        except RuntimeError as e:
            if rank == 0:
                sys.stderr.write(f"[bench] peer exchange unavailable ({e}); using NCCL all-reduce\n")
            exchanges = None
        ok = torch.tensor([1 if exchanges is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            exchanges = None

    def op_backward_filter_exchange(li, b, st, prev=None):
        # sends this step's gradient to all ranks; the previous step's world sum lands in the
        # previous buffer set's dw (the exchange is pipelined by one step)
        exchanges[li].launch(b["x"].data_ptr(), b["dy"].data_ptr(),
                             prev["dw"].data_ptr() if prev is not None else None,
                             b["ws"].data_ptr(), b["nws"], b["shape"], st)

    OPS = (("forward", op_forward, 1), ("backward_input", op_backward_input, 1),
           ("backward_filter", op_backward_filter, 2))  # launches per call

    def compute_step(bufs, st, local=False, prev=None):
        for b in bufs:
            op_forward(b, st)
        for li in reversed(range(len(bufs))):
            b = bufs[li]
            op_backward_input(b, st)
            if exchanges is not None and not local:
                op_backward_filter_exchange(li, b, st, prev[li] if prev is not None else None)
            else:
                op_backward_filter(b, st)

    # dW all-reduce: packed into one flat fp32 buffer, on a side stream, overlapped with the
    # next step's kernels; the result is awaited before the next all-reduce starts
    reducer = None
    pending = [None]
    if world > 1 and exchanges is None:
        reducer = FilterGradReducer([b["dw"].shape for b in sets[0]], dev, side_stream=True)

    # ---- one CUDA graph per buffer set (compute only; the collective stays eager) -------
    stream = torch.cuda.Stream(device=dev)
    graphs = None
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for si, bufs in enumerate(sets):  # also every kernel's first-call set-up, outside capture
            compute_step(bufs, stream.cuda_stream, prev=sets[si - 1])
    stream.synchronize()
    if not args.no_graph and args.launch != "eager":
        graphs = []
        for si, bufs in enumerate(sets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                compute_step(bufs, torch.cuda.current_stream().cuda_stream, prev=sets[si - 1])
            graphs.append(g)

    use_graph = [graphs is not None]

    def compute_only(i):
        if use_graph[0]:
            graphs[i % n_sets].replay()
        else:
            compute_step(sets[i % n_sets], torch.cuda.current_stream().cuda_stream,
                         prev=sets[(i - 1) % n_sets])

    def step(i):
        bufs = sets[i % n_sets]
        last_step[0] = i
        compute_only(i)
        if reducer is not None:
            if pending[0] is not None:
                reducer.finish(pending[0])
            pending[0] = [b["dw"] for b in bufs]
            reducer.start(pending[0])

    last_step = [0]

    def drain():
        if reducer is not None and pending[0] is not None:
            reducer.finish(pending[0])
            pending[0] = None
        if exchanges is not None:  # complete the last step's sum
            for ex, b in zip(exchanges, sets[last_step[0] % n_sets]):
                ex.finish(b["dw"], stream=torch.cuda.current_stream().cuda_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    calibration = None
    with torch.cuda.stream(stream):
        if graphs is not None and args.launch == "auto":
            # Replaying a graph saves host time per launch; launching eagerly lets each kernel
            # become resident while the previous step's last kernel drains (programmatic dependent
            # launch does not reach across graph boundaries).  Which wins depends on the step's
            # length, so time a few steps each way and keep the faster (same choice on all ranks).
            calibration = {}
            for mode in (True, False):
                use_graph[0] = mode
                for i in range(10):
                    step(i)
                drain()
                barrier()
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record(stream)
                for i in range(120):
                    step(i)
                drain()
                c1.record(stream)
                barrier()
                t = torch.tensor([c0.elapsed_time(c1) / 120], device=dev, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                calibration["graph_ms" if mode else "eager_ms"] = round(float(t.item()), 5)
            use_graph[0] = calibration["graph_ms"] <= calibration["eager_ms"]
        for i in range(max(args.warmup, 3)):
            step(i)
        drain()
        barrier()
        t_load0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        drain()
        e1.record(stream)
        barrier()
        ms_total = e0.elapsed_time(e1)
        # ---- spread of single steps (each bracketed by its own events, which costs a little
        # overlap), and the same step with L2 warm (one buffer set over and over) ------------
        n_single = 60
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_single + 1)]
        for i in range(n_single):
            marks[i].record(stream)
            step(i)
        drain()
        marks[n_single].record(stream)
        stream.synchronize()
        singles = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(n_single))
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(5):
            compute_step(sets[0], stream.cuda_stream, local=True)
        w0.record(stream)
        for _ in range(n_single):
            compute_step(sets[0], stream.cuda_stream, local=True)
        w1.record(stream)
        stream.synchronize()
        spread = {"single_step_median_ms": round(statistics.median(singles), 5),
                  "single_step_best_ms": round(singles[0], 5),
                  "l2_warm_ms_per_step": round(w0.elapsed_time(w1) / n_single, 5),
                  "l2_warm_note": "same buffer set every step, launched eagerly, no exchange; "
                                  f"one set is {per_set / 1e6:.0f} MB against 126 MB of L2"}
        # ---- per-operator timing (first layer set rotation), same stream, CUDA events ---
        op_ms = {}
        reps = max(20, min(args.steps, 200))
        for name, fn, _ in OPS:
            for i in range(3):
                for b in sets[i % n_sets]:
                    fn(b, stream.cuda_stream)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for i in range(reps):
                for b in sets[i % n_sets]:
                    fn(b, stream.cuda_stream)
            z.record(stream)
            stream.synchronize()
            op_ms[name] = a.elapsed_time(z) / reps
        # N > 1: every rank's step without the exchange, and the filter gradient with it, so that
        # the cost of the exchange can be read off (all ranks run this loop together)
        multi = None
        if world > 1 and exchanges is not None:
            multi = {}
            for name, fn in (("local_step_ms", lambda i: compute_step(sets[i % n_sets], stream.cuda_stream, local=True)),
                             ("filter_exchange_ms", lambda i: [op_backward_filter_exchange(li, b, stream.cuda_stream)
                                                               for li, b in enumerate(sets[i % n_sets])])):
                for i in range(3):
                    fn(i)
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for i in range(reps):
                    fn(i)
                z.record(stream)
                stream.synchronize()
                t = torch.tensor([a.elapsed_time(z) / reps], device=dev, dtype=torch.float64)
                gathered = [torch.zeros_like(t) for _ in range(world)]
                dist.all_gather(gathered, t)
                multi[name] = [round(float(v.item()), 5) for v in gathered]
        # context for the roofline: what a plain device copy of one operator's traffic (read |x|,
        # write |y| of the first layer) achieves at THIS size, same stream and timing
        b0 = sets[0][0]
        cp_a, cp_z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        scratch = [torch.empty_like(sets[i % n_sets][0]["x"]) for i in range(n_sets)]
        for i in range(3):
            scratch[i % n_sets].copy_(sets[i % n_sets][0]["x"])
        cp_a.record(stream)
        for i in range(reps):
            scratch[i % n_sets].copy_(sets[i % n_sets][0]["x"])
        cp_z.record(stream)
        stream.synchronize()
        copy_ms = cp_a.elapsed_time(cp_z) / reps
        copy_gbps = 2 * b0["x"].numel() * b0["x"].element_size() / (copy_ms * 1e-3) / 1e9
        del scratch
        # keep the GPU loaded until the clock sampler has a few samples
        if sampler is not None:
            t_need = t_load0 + 0.8
            i = 0
            while time.perf_counter() < t_need:
                # rank 0 only: nothing in here may wait for another rank
                compute_step(sets[i % n_sets], stream.cuda_stream, local=True)
                i += 1
                if i % 64 == 0:
                    stream.synchronize()
            stream.synchronize()
        t_load1 = time.perf_counter()
    clocks = sampler.stop(t_load0, t_load1) if sampler is not None else None

    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    sb = step_bytes(layers)
    value = sb * world / (ms_step * 1e-3) / 1e9

    # ---- e2e: public Python API, pinned host buffers, copies inside the timed region ----
    host = []
    for (N, C, H, k, s, p, dt) in layers:
        g = torch.Generator().manual_seed(77)
        ho = out_hw(H, k, s, p)
        hx = torch.randn((N, C, H, H), generator=g).to(tdt[dt]).pin_memory()
        hw_ = (torch.randn((C, 1, k, k), generator=g) / k).to(tdt[dt]).pin_memory()
        hdy = torch.randn((N, C, ho, ho), generator=g).to(tdt[dt]).pin_memory()
        outs = [torch.empty_like(hdy).pin_memory(), torch.empty_like(hx).pin_memory(),
                torch.empty_like(hw_).pin_memory()]
        host.append((hx, hw_, hdy, outs, s, p))
    h2d = sum(t.numel() * t.element_size() for h in host for t in h[:3])
    d2h = sum(t.numel() * t.element_size() for h in host for t in h[3])

    pipes = [] if args.no_e2e else [
        dwconv_b200.HostMapsStep(hx.shape, hw_.shape[2], s, p, dtype=hx.dtype, device=dev,
                                 all_reduce=world > 1)
        for hx, hw_, hdy, outs, s, p in host]

    def e2e_step():
        for pipe, (hx, hw_, hdy, outs, s, p) in zip(pipes, host):
            pipe.run(hx, hw_, hdy, outs[0], outs[1], outs[2])

    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 20))
    for _ in range(3 if e2e_steps else 0):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps if e2e_steps else None
    if world > 1 and e2e_s is not None:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = sb * world / e2e_s / 1e9 if e2e_s else None

    if rank == 0:
        peak, peak_src = load_peaks()
        # dominant operator = the slowest of the three; each moves |x|+|y|+|w| bytes per layer
        dom = max(op_ms, key=op_ms.get)
        op_bytes = sb / 3
        achieved = op_bytes / (op_ms[dom] * 1e-3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "dram_traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                traffic = json.load(f).get(args.workload, {}).get(dom)
        cpu_entry = None
        if world == 1 and not args.no_cpu_baseline:
            try:
                r = run_cpu_route(layers, layers[0][0], 0, 1, args.cpu_seconds)
                cpu_entry = cpu_baseline_entry(layers, r)
            except Exception as e:  # noqa: BLE001
                cpu_entry = {"value": None, "unit": UNIT, "cores": None, "kind": "port",
                             "sample": f"failed: {e}"}
        launches = sum(n for _, _, n in OPS) * len(layers) * args.steps
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": layers[0][6], "data": "synthetic (seeded N(0,1); w ~ N(0,1/k^2))",
            "config": {
                "workload": f"{args.workload}: {DESCR.get(args.workload, args.workload)}",
                "per_gpu_batch": layers[0][0],
                "l2": f"rotating {n_sets} buffer sets ({n_sets * per_set / 1e6:.0f} MB touched "
                      f"between reuses; L2 is 126 MB)",
                "cuda_graph": use_graph[0],
                "launch_calibration": calibration,
                "algorithmic_bytes_per_step": sb,
                "parallelism": "single GPU" if world == 1 else (
                    f"dp{world} (batch-sharded; dW summed over the GPUs inside the filter-gradient "
                    "kernel by peer stores over NVLink)" if exchanges is not None else
                    f"dp{world} (batch-sharded; one NCCL all-reduce of dW per step, overlapped)"),
            },
            "frac_of_8TBs": round(value / world / 8000.0, 4),
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 2),
                         "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4),
                         "peak_source": peak_src, "traffic": traffic,
                         "algorithmic_bytes_per_launch": op_bytes,
                         "torch_copy_of_first_layer_x_gbps": round(copy_gbps, 1)},
            "timing_spread": spread,
            "ops_ms": {k: round(v, 5) for k, v in op_ms.items()},
            "ops_gbps": {k: round(op_bytes / (v * 1e-3) / 1e9, 1) for k, v in op_ms.items()},
            "e2e": None if e2e_val is None else {
                "value": round(e2e_val, 3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3, 4),
                "api": "dwconv_b200.HostMapsStep.run: pinned host x, w, dy -> pinned host y, dx, dw; "
                       f"batch cut into chunks of {pipes[0].chunk} images, upload / kernels / "
                       "download on three streams",
                "gpu_launches_per_step": sum(p.launches_per_run for p in pipes)},
            "per_rank": multi,
            "numa_binding": numa,
            "gpu_launches": launches,
            "clocks": clocks,
            "cpu_baseline": cpu_entry,
            "kernel_family": {1: "direct", 2: "rows"}.get(L.dwconv_b200_last_path(), "auto"),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly")
    ap.add_argument("--launch", default="auto", choices=["auto", "graph", "eager"],
                    help="replay one CUDA graph per step, launch eagerly, or time both and keep "
                         "the faster (default)")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="N > 1: sum dW with an NCCL all-reduce instead of the in-kernel exchange")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    args = ap.parse_args()
    layers = [list(l) for l in WORKLOADS[args.workload]]
    if args.impl == "reference":
        reference_arm(args, layers)
    else:
        gpu_arm(args, layers)


if __name__ == "__main__":
    main()
