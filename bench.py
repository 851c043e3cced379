#!/usr/bin/env python
"""Benchmark of the depthwise-conv2d hot path (forward + backward-input + backward-filter).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl b200|reference]

One "step" is one training step's worth of the path over one batch of seeded synthetic data
of the named workload: every layer's forward, then every layer's two gradients (by default
from the fused backward call, which reads dy once).  The per-GPU batch is fixed (weak
scaling).  With N > 1 every step also sums the filter gradient over the ranks, and the step
is SYNCHRONOUS: the world sum of step i's dW is in memory before step i ends (the sum is made
by peer stores inside the kernel that finishes the gradient; an exchange_finish call per layer
closes the step).  Rank 0 prints ONE JSON line:

* ``value``      algorithmic GB/s, inputs resident in HBM, device-timed (CUDA events), max over
                 ranks; algorithmic bytes per step = 3 * (|x| + |y| + |w|) summed over layers
                 (the unfused definition, whether or not the backward is fused);
* ``e2e``        the same metric through the public Python API with pinned HOST buffers:
                 host->device copies of x, w, dy and device->host copies of y, dx, dW inside
                 the timed region, every step, two consecutive steps in flight at a time
                 (``HostMapsPipeline``; ``serial_ms_per_step``: one at a time); ``copy_ceiling_ms``
                 beside it is the same bytes moved both ways at once with no kernel at all;
* ``roofline``   the slowest kernel of the step, timed alone with CUDA events, its own
                 algorithmic bytes against the measured HBM copy bandwidth (MEASURED_PEAKS.json);
* ``cpu_baseline`` the reference's CPU route timed on this machine's host cores (rank 0, N = 1);
* ``clocks``     SM clock / throttle reasons sampled with nvidia-smi while the GPU was loaded;
* ``stack``      the other half of the metric: the EfficientNet-B0 depthwise stack (c3), images/s;
* ``strong``     strong scaling: c4a (global batch 64) and c5k3 (global batch 256) with the
                 batch divided by N, step time and images/s for the whole job;
* ``dw_check``   N > 1: the last step's exchanged dW against an NCCL all-reduce of the ranks'
                 local gradients, and whether all ranks hold identical bits;
* ``timing_spread`` median and best of 60 steps timed one by one, and the L2-warm step.

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
    # maps wider than the 128 columns the row-staged kernels take, and a layer without padding:
    # the tile kernels' ground (not BASELINE configurations; the shapes of the reference's own tests
    # and of a 224x224 stem)
    "t224": [(32, 32, 224, 3, 1, 1, "f32")],
    "t224s2": [(32, 32, 224, 3, 2, 1, "f32")],
    "t224k5h": [(32, 32, 224, 5, 1, 2, "f16")],
    "t64p0": [(32, 32, 64, 3, 1, 0, "f32")],
}
DESCR = {
    "c1": "single depthwise conv N8 C32 56x56 k3 s1 p1 fp32",
    "c2": "MobileNetV2-style small-map layer N128 C576 14x14 k3 s1 p1 fp32",
    "c3": "EfficientNet-B0 depthwise stack, 7 layers, N128 fp32",
    "c4a": "ConvNeXt-T-style 7x7 N64 C96 56x56 fp16 (fp32 accumulate)",
    "c4b": "ConvNeXt-T-style 7x7 N64 C192 28x28 fp16 (fp32 accumulate)",
}
# strong scaling (fixed global batch, divided over the ranks): workload -> global batch
STRONG = {"c4a": 64, "c5k3": 256}
ESIZE = {"f32": 4, "f16": 2, "bf16": 2, "f64": 8}
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


def config_of(args, layers):
    """The keys both arms print under ``config``."""
    return {"workload": f"{args.workload}: {DESCR.get(args.workload, args.workload)}",
            "per_gpu_batch": layers[0][0]}


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU route in a child process
# --------------------------------------------------------------------------------------
def run_cpu_route(layers, images, steps, warmup, seconds):
    cmd = [sys.executable, os.path.join(ROOT, "oracle", "cpu_baseline.py"),
           "--layers", json.dumps(layers), "--images", str(images), "--steps", str(steps),
           "--warmup", str(warmup), "--seconds", str(seconds)]
    # the child uses every host core: a launcher's per-rank thread limits do not apply to it
    env = {k: v for k, v in os.environ.items()
           if k not in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS")}
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=1800, env=env)
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
        "config": config_of(args, layers),
        "sample_images_per_step": images,
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
class Bench:
    """Rotating buffer sets and the step of one workload at one per-GPU batch."""

    def __init__(self, layers, dev, rank, world, exchange, min_sets=2, max_sets=8):
        import torch
        from dwconv_b200 import _lib
        from dwconv_b200.dist import PeerFilterExchange
        self.torch, self._lib, self.L = torch, _lib, _lib.lib
        self.layers, self.dev, self.rank, self.world = layers, dev, rank, world
        tdt = {"f32": torch.float32, "f16": torch.float16, "f64": torch.float64}
        code = {"f32": _lib.F32, "f16": _lib.F16, "f64": _lib.F64}
        # enough rotating sets that >= 2 x L2 is touched between reuses of a set
        self.per_set = sum(2 * (bx + by) for bx, by, _ in map(layer_bytes, layers))  # x, dx, y, dy
        self.n_sets = max(min_sets, min(max_sets, int(2 * L2_BYTES // self.per_set) + 2))
        self.sets = []
        for si in range(self.n_sets):
            bufs = []
            for li, (N, C, H, k, s, p, dt) in enumerate(layers):
                g = torch.Generator(device=dev).manual_seed(1000 * rank + 10 * li + si)
                ho = out_hw(H, k, s, p)
                x = torch.randn((N, C, H, H), generator=g, device=dev).to(tdt[dt])
                w = (torch.randn((C, 1, k, k), generator=g, device=dev) / k).to(tdt[dt])
                dy = torch.randn((N, C, ho, ho), generator=g, device=dev).to(tdt[dt])
                shape = _lib.Shape(N, C, H, H, k, k, s, s, p, p, ho, ho)
                nws = self.L.dwconv_b200_backward_filter_workspace_bytes(code[dt], shape)
                bufs.append(dict(x=x, w=w, dy=dy, y=torch.empty_like(dy), dx=torch.empty_like(x),
                                 dw=torch.empty_like(w),
                                 ws=torch.empty(nws, dtype=torch.uint8, device=dev),
                                 nws=nws, shape=shape, code=code[dt]))
            self.sets.append(bufs)
        self.exchanges = None
        if world > 1 and exchange:
            self.exchanges = [PeerFilterExchange(C, k, tdt[dt], dev) for (N, C, H, k, s, p, dt) in layers]
        self.graphs = {}

    # ---- single operators -------------------------------------------------------------
    def forward(self, b, st):
        self._lib.check(self.L.dwconv_b200_forward(b["x"].data_ptr(), b["w"].data_ptr(),
                                                   b["y"].data_ptr(), b["code"], b["shape"], st),
                        "forward")

    def backward_input(self, b, st):
        self._lib.check(self.L.dwconv_b200_backward_input(b["dy"].data_ptr(), b["w"].data_ptr(),
                                                          b["dx"].data_ptr(), b["code"], b["shape"], st),
                        "backward_input")

    def backward_filter(self, b, st, dw=None):
        self._lib.check(self.L.dwconv_b200_backward_filter(
            b["x"].data_ptr(), b["dy"].data_ptr(), (dw if dw is not None else b["dw"]).data_ptr(),
            b["ws"].data_ptr(), b["nws"], b["code"], b["shape"], st), "backward_filter")

    def backward(self, b, st):
        self._lib.check(self.L.dwconv_b200_backward(
            b["x"].data_ptr(), b["dy"].data_ptr(), b["w"].data_ptr(), b["dx"].data_ptr(),
            b["dw"].data_ptr(), b["ws"].data_ptr(), b["nws"], b["code"], b["shape"], st), "backward")

    # ---- steps ------------------------------------------------------------------------
    def step_local(self, bufs, st, fused=True):
        """Forward of every layer, then both gradients of every layer; no exchange."""
        for b in bufs:
            self.forward(b, st)
        for b in reversed(bufs):
            if fused:
                self.backward(b, st)
            else:
                self.backward_input(b, st)
                self.backward_filter(b, st)

    def step_sync(self, bufs, st, fused=True):
        """N > 1.  The filter gradient's second pass sends each rank's sums to all ranks; the
        kernels that follow in the step hide the stores' flight; one finish call per layer at
        the end of the step leaves the world sum of THIS step in ``dw``."""
        ex = self.exchanges
        for b in bufs:
            self.forward(b, st)
        for li in reversed(range(len(bufs))):
            b = bufs[li]
            if fused:
                ex[li].launch_backward(b["x"].data_ptr(), b["dy"].data_ptr(), b["w"].data_ptr(),
                                       b["dx"].data_ptr(), None, b["ws"].data_ptr(), b["nws"],
                                       b["shape"], st)
            else:
                ex[li].launch(b["x"].data_ptr(), b["dy"].data_ptr(), None, b["ws"].data_ptr(),
                              b["nws"], b["shape"], st)
                self.backward_input(b, st)
        for li in reversed(range(len(bufs))):
            ex[li].finish(bufs[li]["dw"], stream=st)

    def step_sync_kernel(self, bufs, st):
        """N > 1.  The whole sum inside the kernel that finishes the gradient: after sending its
        sums it waits for the other ranks' and writes the world sum of THIS step to ``dw``."""
        for b in bufs:
            self.forward(b, st)
        for li in reversed(range(len(bufs))):
            b = bufs[li]
            self.exchanges[li].launch_allreduce(b["x"].data_ptr(), b["dy"].data_ptr(), b["w"].data_ptr(),
                                                b["dx"].data_ptr(), b["dw"].data_ptr(), b["ws"].data_ptr(),
                                                b["nws"], b["shape"], st)

    def step_pipelined(self, bufs, prev, st):
        """N > 1, for comparison: the sum of a step's dW is completed by the NEXT step's
        exchange call (delayed by one step; no finish kernel)."""
        for b in bufs:
            self.forward(b, st)
        for li in reversed(range(len(bufs))):
            b = bufs[li]
            self.backward_input(b, st)
            self.exchanges[li].launch(b["x"].data_ptr(), b["dy"].data_ptr(), prev[li]["dw"].data_ptr(),
                                      b["ws"].data_ptr(), b["nws"], b["shape"], st)

    def run_step(self, i, mode, st):
        bufs = self.sets[i % self.n_sets]
        if mode == "local":
            self.step_local(bufs, st, True)
        elif mode == "local_unfused":
            self.step_local(bufs, st, False)
        elif mode == "sync":
            self.step_sync(bufs, st, True)
        elif mode == "sync_split":
            self.step_sync(bufs, st, False)
        elif mode == "sync_kernel":
            self.step_sync_kernel(bufs, st)
        elif mode == "pipelined":
            self.step_pipelined(bufs, self.sets[(i - 1) % self.n_sets], st)
        else:
            raise ValueError(mode)

    def launches_per_step(self, mode):
        per_layer = {"local": 3, "local_unfused": 4, "sync": 4, "sync_split": 5, "sync_kernel": 3,
                     "pipelined": 4}[mode]
        return per_layer * len(self.layers)

    def make_graphs(self, mode, stream):
        """One CUDA graph per buffer set for ``mode`` (after an eager pass: kernel set-up)."""
        torch = self.torch
        if mode in self.graphs:
            return self.graphs[mode]
        with torch.cuda.stream(stream):
            for si in range(self.n_sets):
                self.run_step(si, mode, stream.cuda_stream)
        stream.synchronize()
        graphs = []
        for si in range(self.n_sets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                self.run_step(si, mode, torch.cuda.current_stream().cuda_stream)
            graphs.append(g)
        self.graphs[mode] = graphs
        return graphs

    def time_steps(self, mode, steps, warmup, stream, use_graph, barrier):
        """ms per step: CUDA events on ``stream`` around ``steps`` steps, max over ranks."""
        torch = self.torch
        graphs = self.make_graphs(mode, stream) if use_graph else None

        def one(i):
            if graphs is not None:
                graphs[i % self.n_sets].replay()
            else:
                self.run_step(i, mode, stream.cuda_stream)

        with torch.cuda.stream(stream):
            for i in range(warmup):
                one(i)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                one(i)
            e1.record(stream)
            barrier()
        ms = e0.elapsed_time(e1) / steps
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def close(self):
        if self.exchanges is not None:
            for ex in self.exchanges:
                ex.close()
            self.exchanges = None
        self.graphs = {}
        self.sets = []


def gpu_arm(args, layers):
    import torch
    import torch.distributed as dist
    import dwconv_b200
    from dwconv_b200 import _lib
    from dwconv_b200.dist import bind_to_gpu_numa_node

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
        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=120))
    L = _lib.lib
    tdt = {"f32": torch.float32, "f16": torch.float16, "f64": torch.float64}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    wb = Bench(layers, dev, rank, world, exchange=True)
    n_sets, per_set = wb.n_sets, wb.per_set
    stream = torch.cuda.Stream(device=dev)
    head_mode = "local" if world == 1 else "sync"
    if args.unfused:
        head_mode = "local_unfused" if world == 1 else "sync_split"

    sampler = ClockSampler(local) if rank == 0 else None
    # ---- launch calibration: graph replay or eager launches; at N > 1 also which order of
    # the backward kernels hides the exchange better (same choice on all ranks) -------------
    calibration = {}
    candidates = [head_mode]
    if world > 1 and not args.unfused:
        candidates.append("sync_kernel")
    best = None
    for mode in candidates:
        for use_graph in ((True, False) if args.launch == "auto" else
                          ((True,) if args.launch == "graph" else (False,))):
            ms = wb.time_steps(mode, args.calibration_steps, min(10, args.calibration_steps), stream,
                               use_graph, barrier)
            calibration[f"{mode}_{'graph' if use_graph else 'eager'}_ms"] = round(ms, 5)
            if best is None or ms < best[0]:
                best = (ms, mode, use_graph)
    _, head_mode, use_graph = best

    # ---- the headline: exactly --steps steps after >= 3 warm-up steps ---------------------
    t_load0 = time.perf_counter()
    ms_step = wb.time_steps(head_mode, args.steps, max(args.warmup, 3), stream, use_graph, barrier)
    sb = step_bytes(layers)
    value = sb * world / (ms_step * 1e-3) / 1e9

    # ---- N > 1: is the summed gradient right?  (outside the timed region) -----------------
    dw_check = None
    variants = None
    if world > 1:
        with torch.cuda.stream(stream):
            wb.run_step(0, head_mode, stream.cuda_stream)
            stream.synchronize()
            worst, same = 0.0, True
            for b in wb.sets[0]:
                got = b["dw"].clone()
                mine = torch.empty_like(b["dw"])
                wb.backward_filter(b, stream.cuda_stream, dw=mine)
                stream.synchronize()
                want = mine.double()
                dist.all_reduce(want, op=dist.ReduceOp.SUM)
                scale = float(want.abs().max().item())
                worst = max(worst, float((got.double() - want).abs().max().item()) / max(scale, 1e-30))
                everyone = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(everyone, got)
                same = same and all(torch.equal(everyone[0], t) for t in everyone[1:])
            status = int(L.dwconv_b200_device_status())
        tol = 1e-2 if layers[0][6] == "f16" else 1e-4
        dw_check = {"ok": bool(worst <= tol and same and status == 0), "max_rel_err": worst,
                    "ranks_identical": bool(same), "device_status": status, "tolerance": tol,
                    "against": "NCCL all_reduce(SUM) of every rank's local dwconv_b200_backward_filter"}
        # the other ways to run the step, for the record
        variants = {}
        for mode in ("local", "sync", "sync_kernel", "sync_split", "pipelined"):
            variants[mode + "_ms"] = round(wb.time_steps(mode, 200, 10, stream, False, barrier), 5)
        variants["note"] = ("eager launches, 200 steps, max over ranks.  local: no exchange at all; "
                            "sync: fused backward + in-kernel exchange + finish per step (dW of the "
                            "step complete at its end); sync_kernel: fused backward whose second pass "
                            "also waits for the other ranks' sums (the whole all-reduce in that "
                            "kernel); sync_split: filter gradient + exchange first, "
                            "backward-input hides the stores' flight, then finish; pipelined: dW "
                            "completed by the next step's exchange (one step late)")

    with torch.cuda.stream(stream):
        # ---- spread of single steps, and the same step with L2 warm -----------------------
        n_single = 60
        graphs = wb.make_graphs(head_mode, stream) if use_graph else None

        def one(i):
            if graphs is not None:
                graphs[i % n_sets].replay()
            else:
                wb.run_step(i, head_mode, stream.cuda_stream)

        barrier()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_single + 1)]
        for i in range(n_single):
            marks[i].record(stream)
            one(i)
        marks[n_single].record(stream)
        stream.synchronize()
        barrier()
        singles = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(n_single))
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(5):
            wb.step_local(wb.sets[0], stream.cuda_stream)
        w0.record(stream)
        for _ in range(n_single):
            wb.step_local(wb.sets[0], stream.cuda_stream)
        w1.record(stream)
        stream.synchronize()
        spread = {"single_step_median_ms": round(statistics.median(singles), 5),
                  "single_step_best_ms": round(singles[0], 5),
                  "l2_warm_ms_per_step": round(w0.elapsed_time(w1) / n_single, 5),
                  "l2_warm_note": "same buffer set every step, launched eagerly, no exchange; "
                                  f"one set is {per_set / 1e6:.0f} MB against 126 MB of L2"}
        # ---- every operator alone, same rotation, same stream, CUDA events ----------------
        OPS = (("forward", wb.forward), ("backward_input", wb.backward_input),
               ("backward_filter", wb.backward_filter), ("backward_fused", wb.backward))
        op_ms = {}
        reps = max(20, min(args.steps, 200))
        for name, fn in OPS:
            for i in range(3):
                for b in wb.sets[i % n_sets]:
                    fn(b, stream.cuda_stream)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for i in range(reps):
                for b in wb.sets[i % n_sets]:
                    fn(b, stream.cuda_stream)
            z.record(stream)
            stream.synchronize()
            op_ms[name] = a.elapsed_time(z) / reps
        # context for the roofline: what a plain device copy of one operator's traffic (read |x|,
        # write |y| of the first layer) achieves at THIS size, same stream and timing
        b0 = wb.sets[0][0]
        cp_a, cp_z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        scratch = [torch.empty_like(wb.sets[i % n_sets][0]["x"]) for i in range(n_sets)]
        for i in range(3):
            scratch[i % n_sets].copy_(wb.sets[i % n_sets][0]["x"])
        cp_a.record(stream)
        for i in range(reps):
            scratch[i % n_sets].copy_(wb.sets[i % n_sets][0]["x"])
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
                wb.step_local(wb.sets[i % n_sets], stream.cuda_stream)
                i += 1
                if i % 64 == 0:
                    stream.synchronize()
            stream.synchronize()
        t_load1 = time.perf_counter()
    clocks = sampler.stop(t_load0, t_load1) if sampler is not None else None
    barrier()
    head_launches = wb.launches_per_step(head_mode)
    wb.close()
    del wb
    torch.cuda.empty_cache()

    # ---- the other half of the metric: the EfficientNet-B0 depthwise stack ------------------
    stack_entry, strong = None, None
    if not args.no_extras:
        def timed_workload(name, batch, steps):
            lay = [[batch] + list(l[1:]) for l in WORKLOADS[name]]
            w2 = Bench(lay, dev, rank, world, exchange=True, min_sets=2, max_sets=4)
            if world == 1:
                ms = w2.time_steps("local", steps, 5, stream, True, barrier)
            else:  # the faster of the two synchronous forms
                ms = min(w2.time_steps(m, steps, 5, stream, True, barrier) for m in ("sync", "sync_kernel"))
            out = {"per_gpu_batch": batch, "ms_per_step": round(ms, 5),
                   "images_per_s": round(batch * world / (ms * 1e-3), 1),
                   "algorithmic_gbps": round(step_bytes(lay) * world / (ms * 1e-3) / 1e9, 1),
                   "buffer_sets": w2.n_sets, "set_mb": round(w2.per_set / 1e6, 1)}
            barrier()
            w2.close()
            del w2
            torch.cuda.empty_cache()
            return out

        stack_entry = dict(workload="c3: " + DESCR["c3"], **timed_workload("c3", 128, 40))
        stack_entry["scaling"] = "weak (128 images per GPU)"
        strong = {}
        for name, gb in STRONG.items():
            if gb % world == 0 and gb // world >= 1:
                strong[name] = dict(global_batch=gb, **timed_workload(name, gb // world, 200))
        strong["note"] = ("fixed global batch divided over the ranks; dW summed over the ranks "
                          "inside the step (synchronous); one CUDA graph per step; small shards "
                          "fit the 126 MB L2 (see set_mb x buffer_sets)")

    # ---- e2e: public Python API, pinned host buffers, copies inside the timed region ----
    host = []
    depth = 1 if args.no_e2e else max(1, args.e2e_depth)
    more_hosts = [[] for _ in range(depth - 1)]
    for (N, C, H, k, s, p, dt) in layers:
        g = torch.Generator().manual_seed(77)
        ho = out_hw(H, k, s, p)
        hx = torch.randn((N, C, H, H), generator=g).to(tdt[dt]).pin_memory()
        hw_ = (torch.randn((C, 1, k, k), generator=g) / k).to(tdt[dt]).pin_memory()
        hdy = torch.randn((N, C, ho, ho), generator=g).to(tdt[dt]).pin_memory()
        outs = [torch.empty_like(hdy).pin_memory(), torch.empty_like(hx).pin_memory(),
                torch.empty_like(hw_).pin_memory()]
        host.append((hx, hw_, hdy, outs, s, p))
        # further sets of host buffers: the steps in flight at a time each have their own
        for extra in more_hosts:
            extra.append((hx.clone().pin_memory(), hw_, hdy.clone().pin_memory(),
                          [torch.empty_like(o).pin_memory() for o in outs], s, p))
    h2d = sum(t.numel() * t.element_size() for h in host for t in h[:3])
    d2h = sum(t.numel() * t.element_size() for h in host for t in h[3])

    # Every step reads its inputs from pinned host memory and leaves its results there.  `depth`
    # steps (default 2) are in flight at a time (HostMapsPipeline: the uploads of step i+1 run
    # under the downloads of step i, each step on host buffers of its own); `serial_ms_per_step`
    # is the same with one step at a time.
    pipes = [] if args.no_e2e else [
        dwconv_b200.HostMapsPipeline(hx.shape, hw_.shape[2], s, p, depth=depth, dtype=hx.dtype, device=dev,
                                     all_reduce=world > 1, chunk_images=args.e2e_chunk)
        for hx, hw_, hdy, outs, s, p in host]
    serial_pipes = [] if args.no_e2e else [
        dwconv_b200.HostMapsStep(hx.shape, hw_.shape[2], s, p, dtype=hx.dtype, device=dev,
                                 all_reduce=world > 1)
        for hx, hw_, hdy, outs, s, p in host]
    e2e_count = [0]

    def e2e_step():
        bufs = ([host] + more_hosts)[e2e_count[0] % depth]
        e2e_count[0] += 1
        for pipe, (hx, hw_, hdy, outs, s, p) in zip(pipes, bufs):
            pipe.run(hx, hw_, hdy, outs[0], outs[1], outs[2])

    def e2e_step_serial():
        for pipe, (hx, hw_, hdy, outs, s, p) in zip(serial_pipes, host):
            pipe.run(hx, hw_, hdy, outs[0], outs[1], outs[2])

    def max_over_ranks(v):
        if world > 1 and v is not None:
            t = torch.tensor([v], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    e2e_steps = 0 if args.no_e2e else max(4, min(args.steps, 20))
    serial_s = None
    if e2e_steps:
        for _ in range(3):
            e2e_step_serial()
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step_serial()
        torch.cuda.synchronize()
        serial_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
    for _ in range(3 * depth if e2e_steps else 0):  # each step object: eager, record, replay
        e2e_step()
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps if e2e_steps else None)
    e2e_val = sb * world / e2e_s / 1e9 if e2e_s else None
    # the bare ceiling of that leg: the same bytes up and down at once, no kernel at all
    ceiling_s = None
    if e2e_steps:
        s_up, s_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        dbuf = [(torch.empty_like(hx, device=dev), torch.empty_like(hdy, device=dev))
                for hx, hw_, hdy, outs, s, p in host]

        def copies():
            for (hx, hw_, hdy, outs, s, p), (dx_, dy_) in zip(host, dbuf):
                for dst, src, st in ((dx_, hx, s_up), (dy_, hdy, s_up), (outs[1], dx_, s_down),
                                     (outs[0], dy_, s_down)):
                    _lib.check(L.dwconv_b200_copy_async(dst.data_ptr(), src.data_ptr(),
                                                        src.numel() * src.element_size(),
                                                        st.cuda_stream), "copy_async")
        for _ in range(2):
            copies()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            copies()
        torch.cuda.synchronize()
        ceiling_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        del dbuf

    if rank == 0:
        peak, peak_src = load_peaks()
        # the dominant kernel of the headline step and its own algorithmic bytes per launch:
        # forward |x|+|y|+|w|; fused backward |x|+|dy|+|dx|+|w|+|dw| (dy is read once)
        bx, by, bw = (sum(v) for v in zip(*map(layer_bytes, layers)))
        kernel_bytes = {"forward": bx + by + bw, "backward_input": bx + by + bw,
                        "backward_filter": bx + by + bw, "backward_fused": 2 * bx + by + 2 * bw}
        in_step = (("forward", "backward_fused") if head_mode in ("local", "sync", "sync_kernel") else
                   ("forward", "backward_input", "backward_filter"))
        dom = max(in_step, key=lambda k: op_ms[k])
        achieved = kernel_bytes[dom] / (op_ms[dom] * 1e-3) / 1e9
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
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": layers[0][6], "data": "synthetic (seeded N(0,1); w ~ N(0,1/k^2))",
            "config": config_of(args, layers),
            "details": {
                "l2": f"rotating {n_sets} buffer sets ({n_sets * per_set / 1e6:.0f} MB touched "
                      f"between reuses; L2 is 126 MB)",
                "step": {"local": "forward, fused backward (dx + dW from one read of dy)",
                         "local_unfused": "forward, backward-input, backward-filter",
                         "sync": "forward, fused backward whose second pass sends dW to all ranks, "
                                 "exchange_finish (dW of this step complete at its end)",
                         "sync_kernel": "forward, fused backward whose second pass sends dW to all ranks "
                                        "and adds the ranks' sums (all-reduce inside the kernel; dW of "
                                        "this step complete at its end)",
                         "sync_split": "forward, backward-filter whose second pass sends dW to all "
                                       "ranks, backward-input, exchange_finish (dW of this step "
                                       "complete at its end)"}[head_mode],
                "cuda_graph": use_graph,
                "launch_calibration": calibration,
                "algorithmic_bytes_per_step": sb,
                "parallelism": "single GPU" if world == 1 else (
                    f"dp{world} (batch-sharded; dW summed over the GPUs inside the filter-gradient "
                    "kernel by peer stores over NVLink, synchronous)"),
            },
            "frac_of_8TBs": round(value / world / 8000.0, 4),
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 2),
                         "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4),
                         "peak_source": peak_src, "traffic": traffic,
                         "algorithmic_bytes_per_launch": kernel_bytes[dom],
                         "torch_copy_of_first_layer_x_gbps": round(copy_gbps, 1)},
            "timing_spread": spread,
            "ops_ms": {k: round(v, 5) for k, v in op_ms.items()},
            "ops_gbps": {k: round(kernel_bytes[k] / (v * 1e-3) / 1e9, 1) for k, v in op_ms.items()},
            "e2e": None if e2e_val is None else {
                "value": round(e2e_val, 3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3, 4),
                "copy_ceiling_ms": round(ceiling_s * 1e3, 4),
                "steps_in_flight": depth, "serial_ms_per_step": round(serial_s * 1e3, 4),
                "api": "dwconv_b200.HostMapsPipeline.run: pinned host x, w, dy -> pinned host y, dx, dw, "
                       "every step; a step's batch is cut into chunks of "
                       f"{pipes[0].steps[0].chunk} images (upload / kernels / download on three streams) and "
                       f"{depth} consecutive steps overlap, each on host buffers of its own; "
                       f"serial_ms_per_step: one step at a time (HostMapsStep.run, chunks of "
                       f"{serial_pipes[0].chunk} images)",
                "gpu_launches_per_step": sum(p.launches_per_run for p in pipes)},
            "stack": stack_entry,
            "strong": strong,
            "dw_check": dw_check,
            "step_variants_ms": variants,
            "numa_binding": numa,
            "gpu_launches": head_launches * args.steps,
            "clocks": clocks,
            "cpu_baseline": cpu_entry,
            "kernel_family": {1: "direct", 2: "rows"}.get(L.dwconv_b200_last_path(), "auto"),
        }
        print(json.dumps(line))
    ok = dw_check is None or dw_check["ok"]
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("bench.py: the exchanged filter gradient failed its check: "
                         + json.dumps(dw_check))


def time_api(layers, reps):
    """CUDA-event timing of the public Python API (``depthwise_conv2d`` forward, and forward +
    ``backward``) on arbitrary layers, the way ``oracle/ref_cuda.py --time`` times the reference's
    CUDA route: rotating buffer sets larger than L2, 3 warm-up calls; and of the three operators
    through the C entry points (``ops_ms``).  A layer is [N, C, H, (W,) k, stride, padding, dtype]
    with an optional last element "nhwc" for channels-last tensors.  Prints one JSON object."""
    import torch
    import dwconv_b200
    from dwconv_b200 import _lib
    dts = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
    res = []
    for layer in layers:
        layer = list(layer)
        nhwc = layer[-1] == "nhwc"  # optional last element: channels-last tensors
        spec = layer[:-1] if nhwc else layer
        if len(spec) == 8:
            N, C, H, W, k, s, p, dt = spec
        else:
            N, C, H, k, s, p, dt = spec
            W = H
        fmt = torch.channels_last if nhwc else torch.contiguous_format
        ho, wo = out_hw(H, k, s, p), out_hw(W, k, s, p)
        per_set = 2 * N * C * (H * W + ho * wo) * ESIZE[dt]
        n_sets = max(2, min(8, int(2 * L2_BYTES // per_set) + 2))
        sets = []
        for si in range(n_sets):
            g = torch.Generator(device="cuda").manual_seed(si)
            x = torch.randn((N, C, H, W), generator=g, device="cuda").to(dts[dt]).contiguous(
                memory_format=fmt).requires_grad_(True)
            w = (torch.randn((C, 1, k, k), generator=g, device="cuda") / k).to(dts[dt]).requires_grad_(True)
            dy = torch.randn((N, C, ho, wo), generator=g, device="cuda").to(dts[dt]).contiguous(
                memory_format=fmt)
            sets.append((x, w, dy))

        # the three operators through the C entry points (no Python layer, no allocation)
        shape = _lib.Shape(N, C, H, W, k, k, s, s, p, p, ho, wo)
        code = {"f32": _lib.F32, "f16": _lib.F16, "bf16": _lib.BF16}[dt]
        L = _lib.lib
        ys = [torch.empty_like(t[2]) for t in sets]
        dxs = [torch.empty_like(t[0]) for t in sets]
        ws_bytes = int(L.dwconv_b200_backward_filter_workspace_bytes(code, shape))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        dw = torch.empty((C, 1, k, k), dtype=dts[dt], device="cuda")
        st = torch.cuda.current_stream().cuda_stream

        def op_forward(i):
            x, w, dy = sets[i % n_sets]
            if nhwc:
                return L.dwconv_b200_forward_nhwc(x.data_ptr(), w.data_ptr(), ys[i % n_sets].data_ptr(), code,
                                                  shape, None, st)
            return L.dwconv_b200_forward(x.data_ptr(), w.data_ptr(), ys[i % n_sets].data_ptr(), code, shape, st)

        def op_backward_input(i):
            x, w, dy = sets[i % n_sets]
            f = L.dwconv_b200_backward_input_nhwc if nhwc else L.dwconv_b200_backward_input
            return f(dy.data_ptr(), w.data_ptr(), dxs[i % n_sets].data_ptr(), code, shape, st)

        def op_backward_filter(i):
            x, w, dy = sets[i % n_sets]
            f = L.dwconv_b200_backward_filter_nhwc if nhwc else L.dwconv_b200_backward_filter
            return f(x.data_ptr(), dy.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws_bytes, code, shape, st)

        ops = {}
        for name, fn in (("forward", op_forward), ("backward_input", op_backward_input),
                         ("backward_filter", op_backward_filter)):
            for i in range(3):
                _lib.check(fn(i), name)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for i in range(reps):
                fn(i)
            z.record()
            torch.cuda.synchronize()
            ops[name] = round(a.elapsed_time(z) / reps, 5)
        del ys, dxs

        def fwd(i):
            x, w, dy = sets[i % n_sets]
            with torch.no_grad():
                dwconv_b200.depthwise_conv2d(x, w, None, s, p)

        def fwd_bwd(i):
            x, w, dy = sets[i % n_sets]
            x.grad = None
            w.grad = None
            dwconv_b200.depthwise_conv2d(x, w, None, s, p).backward(dy)

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
        res.append({"layer": list(layer), "forward_ms": round(times["forward"], 5),
                    "forward_backward_ms": round(times["forward_backward"], 5),
                    "ops_ms": ops, "layout": "nhwc" if nhwc else "nchw",
                    "kernel_family": "nhwc" if nhwc else {1: "direct", 2: "rows", 3: "tiles"}.get(
                        _lib.lib.dwconv_b200_last_path()),
                    "buffer_sets": n_sets})
        del sets
        torch.cuda.empty_cache()
    print(json.dumps({"impl": "dwconv_b200 public API (depthwise_conv2d + autograd)", "layers": res}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--launch", default="auto", choices=["auto", "graph", "eager"],
                    help="replay one CUDA graph per step, launch eagerly, or time both and keep "
                         "the faster (default)")
    ap.add_argument("--unfused", action="store_true",
                    help="backward-input and backward-filter as separate operators")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    ap.add_argument("--e2e-chunk", type=int, default=None,
                    help="images per chunk in the host-buffer leg (default: HostMapsStep's choice)")
    ap.add_argument("--e2e-depth", type=int, default=2,
                    help="steps in flight at a time in the host-buffer leg (HostMapsPipeline depth)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the stack and strong-scaling legs (profiling)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--calibration-steps", type=int, default=120,
                    help="steps timed per launch mode before the headline (a profiler run wants few)")
    ap.add_argument("--time-api", metavar="JSON",
                    help="instead of the benchmark: time the public Python API on a JSON list of "
                         "[N, C, H, k, stride, pad, dtype] or [N, C, H, W, k, stride, pad, dtype]")
    ap.add_argument("--reps", type=int, default=50)
    args = ap.parse_args()
    if args.time_api:
        time_api(json.loads(args.time_api), args.reps)
        return
    layers = [list(l) for l in WORKLOADS[args.workload]]
    if args.impl == "reference":
        reference_arm(args, layers)
    else:
        gpu_arm(args, layers)


if __name__ == "__main__":
    main()
