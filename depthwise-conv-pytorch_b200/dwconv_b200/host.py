"""One layer's forward and both gradients for maps that live in pinned HOST memory.

The reference's functions take device tensors (torch_dwconv/dwconv.py:32-45); a caller whose
maps sit in host memory pays the PCIe copies either side of them.  ``HostMapsStep`` cuts the
batch into chunks of whole images and runs three streams side by side: chunk ``i+1`` goes up
to the device while the kernels work on chunk ``i`` and the results of chunk ``i-1`` come
back, so that a step costs about max(upload, download) instead of their sum plus the kernels.

``y`` and ``dx`` are what the one-call path gives, bit for bit (images are independent).
``dw`` is the fp32 sum (fp64 for float64 maps) of the per-chunk filter gradients in chunk
order: deterministic, but not the same rounding as one call over the whole batch.  Each
chunk's two gradients come from the fused backward call (one read of dy), whose second pass
adds straight into the running fp32 gradient: no kernel other than the library's own runs
between the copies.
"""
import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.float64: _lib.F64,
           torch.bfloat16: _lib.BF16}


def _pair(v):
    return (int(v[0]), int(v[1])) if isinstance(v, (tuple, list)) else (int(v), int(v))


def chunk_bounds(n_images, image_bytes, chunk_images=None, target_chunks=8, min_bytes=2 << 20):
    """Cuts a batch into runs of whole images.  By default about ``target_chunks`` equal
    chunks, but none smaller than ``min_bytes``: every chunk adds about 30 us of launch work
    (a dozen stream operations) to the step, measured on PCIe 5 x16, so many small chunks
    cost more than the shorter un-overlapped first upload and last download save; schedules
    with small first and last chunks measured the same as equal chunks."""
    if isinstance(chunk_images, (list, tuple)):  # explicit chunk sizes, in order
        if sum(chunk_images) != n_images or min(chunk_images) < 1:
            raise ValueError(f"chunk sizes {list(chunk_images)} do not add up to {n_images} images")
        bounds, a = [], 0
        for n in chunk_images:
            bounds.append((a, a + int(n)))
            a += int(n)
        return bounds
    if chunk_images is None:
        chunk_images = max(-(-n_images // target_chunks), -(-min_bytes // max(1, image_bytes)))
    step = max(1, min(int(chunk_images), n_images))
    return [(a, min(a + step, n_images)) for a in range(0, n_images, step)]


class HostMapsStep:
    """Pipelined ``y = conv(x, w)``, ``dx``, ``dw`` for host-resident ``x`` and ``dy``.

    Device staging buffers are allocated once here; ``run`` allocates nothing.  With
    ``use_graph`` (the default) the whole three-stream schedule for one set of host buffers is
    recorded into a CUDA graph on its second use and replayed from then on, which removes the
    per-chunk host work (a few dozen stream operations per chunk) from the step.
    """

    SLOTS = 3  # staging buffers per map: one filling, one in the kernels, one draining

    def __init__(self, x_shape, kernel_size, stride=1, padding=0, dtype=torch.float32,
                 device="cuda", chunk_images=None, all_reduce=False, group=None,
                 use_graph=True):
        N, C, H, W = (int(v) for v in x_shape)
        kh, kw = _pair(kernel_size)
        sh, sw = _pair(stride)
        ph, pw = _pair(padding)
        if dtype not in _DTYPES:
            raise RuntimeError(f"dwconv_b200: unsupported dtype {dtype} (float32, float16, bfloat16, float64)")
        L = _lib.lib
        Ho = L.dwconv_b200_out_size(H, 1, ph, ph, kh, sh)
        Wo = L.dwconv_b200_out_size(W, 1, pw, pw, kw, sw)
        if min(N, C, Ho, Wo) <= 0:
            raise RuntimeError(f"dwconv_b200.HostMapsStep: empty problem {tuple(x_shape)} -> {Ho} x {Wo}")
        self.device = torch.device(device)
        self.dtype, self.code = dtype, _DTYPES[dtype]
        self.acc_dtype = torch.float64 if dtype == torch.float64 else torch.float32
        self.x_shape, self.y_shape, self.w_shape = (N, C, H, W), (N, C, Ho, Wo), (C, 1, kh, kw)
        esize = torch.empty((), dtype=dtype).element_size()
        self.bounds = chunk_bounds(N, C * H * W * esize, chunk_images)
        self.chunk = max(b - a for a, b in self.bounds)   # staging buffers hold the largest chunk
        self.all_reduce, self.group = bool(all_reduce), group  # sum dw over the ranks of group
        self.use_graph = bool(use_graph)
        self._graphs = {}   # host buffer addresses -> recorded schedule (None after the first use)
        nc = self.chunk
        self._geo = (C, H, W, kh, kw, sh, sw, ph, pw, Ho, Wo)
        with torch.cuda.device(self.device):
            mk = lambda *s: torch.empty(s, dtype=dtype, device=self.device)  # noqa: E731
            self.dx_ = [mk(nc, C, H, W) for _ in range(self.SLOTS)]
            self.x_ = [mk(nc, C, H, W) for _ in range(self.SLOTS)]
            self.dy_ = [mk(nc, C, Ho, Wo) for _ in range(self.SLOTS)]
            self.y_ = [mk(nc, C, Ho, Wo) for _ in range(self.SLOTS)]
            self.w_ = mk(C, 1, kh, kw)
            self.dw_acc = torch.zeros((C, 1, kh, kw), dtype=self.acc_dtype, device=self.device)
            self.dw_out = mk(C, 1, kh, kw)
            self.ws_bytes = max(int(L.dwconv_b200_backward_filter_workspace_bytes(
                self.code, _lib.Shape(n, C, H, W, kh, kw, sh, sw, ph, pw, Ho, Wo)))
                for n in sorted({b - a for a, b in self.bounds}))
            self.ws = torch.empty(max(self.ws_bytes, 16), dtype=torch.uint8, device=self.device)
            self.s_up = torch.cuda.Stream(self.device)
            self.s_run = torch.cuda.Stream(self.device)
            self.s_down = torch.cuda.Stream(self.device)
            self.s_cap = torch.cuda.Stream(self.device)   # records the schedule into a graph
        self.h2d_bytes = (N * C * (H * W + Ho * Wo) + C * kh * kw) * esize
        self.d2h_bytes = (N * C * (H * W + Ho * Wo) + C * kh * kw) * esize
        self.launches_per_run = 3 * len(self.bounds)  # forward, fused backward first + second pass

    def _copy(self, dev_buf, host, a, b, up, stream):
        """Images a..b of a host map to / from the start of a staging buffer: one bare
        asynchronous copy (torch's ``copy_`` records an event per pinned copy, which costs tens of
        microseconds per chunk while the other direction is busy)."""
        per_image = host.stride(0) * host.element_size()
        hp, dp, nbytes = host.data_ptr() + a * per_image, dev_buf.data_ptr(), (b - a) * per_image
        dst, src = (dp, hp) if up else (hp, dp)
        _lib.check(_lib.lib.dwconv_b200_copy_async(dst, src, nbytes, stream.cuda_stream), "copy_async")

    def _shape(self, n):
        C, H, W, kh, kw, sh, sw, ph, pw, Ho, Wo = self._geo
        return _lib.Shape(n, C, H, W, kh, kw, sh, sw, ph, pw, Ho, Wo)

    def _check_host(self, t, shape, name):
        if t.is_cuda or tuple(t.shape) != tuple(shape) or t.dtype != self.dtype or not t.is_contiguous():
            raise RuntimeError(f"dwconv_b200.HostMapsStep: {name} must be a contiguous host tensor "
                               f"of shape {tuple(shape)} and dtype {self.dtype}")
        if not t.is_pinned():
            raise RuntimeError(f"dwconv_b200.HostMapsStep: {name} must be in pinned memory "
                               "(tensor.pin_memory()) so that its copies can overlap the kernels")

    MAX_GRAPHS = 8

    def run(self, x, w, dy, y, dx, dw):
        """Reads pinned host ``x, w, dy``; fills pinned host ``y, dx, dw``.  Returns after
        everything has been queued on the current stream; ``synchronize()`` waits for it."""
        for t, s, n in ((x, self.x_shape, "x"), (dy, self.y_shape, "dy"), (y, self.y_shape, "y"),
                        (dx, self.x_shape, "dx"), (w, self.w_shape, "w"), (dw, self.w_shape, "dw")):
            self._check_host(t, s, n)
        bufs = (x, w, dy, y, dx, dw)
        with torch.cuda.device(self.device):
            if not self.use_graph:
                self._enqueue(*bufs)
            else:
                key = tuple(t.data_ptr() for t in bufs)
                if key not in self._graphs:
                    # first use: eager (this is also where each kernel does its one-time set-up)
                    if len(self._graphs) >= self.MAX_GRAPHS:
                        self._graphs.pop(next(iter(self._graphs)))
                    self._graphs[key] = None
                    self._enqueue(*bufs)
                else:
                    if self._graphs[key] is None:
                        torch.cuda.synchronize(self.device)
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=self.s_cap):
                            self._enqueue(*bufs)
                        self._graphs[key] = g
                    self._graphs[key].replay()
            self._finish(dw)

    def _enqueue(self, x, w, dy, y, dx, dw):
        """Queues the chunk pipeline: forks the three streams off the current one and joins
        them back into it.  Leaves the batch's filter gradient in ``dw_acc``."""
        L, code = _lib.lib, self.code
        ev = torch.cuda.Event
        cur = torch.cuda.current_stream(self.device)
        start = ev()
        start.record(cur)
        for s in (self.s_up, self.s_run, self.s_down):
            s.wait_event(start)
        _lib.check(L.dwconv_b200_copy_async(self.w_.data_ptr(), w.data_ptr(),
                                            w.numel() * w.element_size(), self.s_up.cuda_stream),
                   "copy_async")
        ran, drained = {}, {}
        for i, (a, b) in enumerate(self.bounds):
            k, n = i % self.SLOTS, b - a
            with torch.cuda.stream(self.s_up):
                if i - self.SLOTS in ran:  # the kernels that read this slot have finished
                    self.s_up.wait_event(ran[i - self.SLOTS])
                self._copy(self.x_[k], x, a, b, True, self.s_up)
                self._copy(self.dy_[k], dy, a, b, True, self.s_up)
                up = ev()
                up.record(self.s_up)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(up)
                if i - self.SLOTS in drained:  # this slot's earlier results have left
                    self.s_run.wait_event(drained[i - self.SLOTS])
                st, shp = self.s_run.cuda_stream, self._shape(n)
                xk, dyk, yk, dxk = self.x_[k], self.dy_[k], self.y_[k], self.dx_[k]
                _lib.check(L.dwconv_b200_forward(xk.data_ptr(), self.w_.data_ptr(), yk.data_ptr(),
                                                 code, shp, st), "forward")
                # dx of the chunk, and dw_acc (+)= the chunk's filter gradient (first chunk: =)
                _lib.check(L.dwconv_b200_backward_accumulate(
                    xk.data_ptr(), dyk.data_ptr(), self.w_.data_ptr(), dxk.data_ptr(),
                    self.dw_acc.data_ptr(), 1 if i > 0 else 0, self.ws.data_ptr(), self.ws_bytes,
                    code, shp, st), "backward_accumulate")
                ran[i] = ev()
                ran[i].record(self.s_run)
            with torch.cuda.stream(self.s_down):
                self.s_down.wait_event(ran[i])
                self._copy(yk, y, a, b, False, self.s_down)
                self._copy(dxk, dx, a, b, False, self.s_down)
                drained[i] = ev()
                drained[i].record(self.s_down)
        for s in (self.s_up, self.s_run, self.s_down):
            done = ev()
            done.record(s)
            cur.wait_event(done)

    def _finish(self, dw):
        """The batch's filter gradient: summed over the ranks if asked, cast, sent to the host."""
        if self.all_reduce:
            torch.distributed.all_reduce(self.dw_acc, group=self.group)
        if self.dw_acc.dtype == self.dtype:   # fp32 / fp64 maps: the accumulator is the result
            dw.copy_(self.dw_acc, non_blocking=True)
        else:
            self.dw_out.copy_(self.dw_acc)    # one cast per step for 16-bit maps
            dw.copy_(self.dw_out, non_blocking=True)

    def synchronize(self):
        torch.cuda.current_stream(self.device).synchronize()


class HostMapsPipeline:
    """Consecutive steps overlapped in time.

    One ``HostMapsStep`` moves a step's inputs up, computes and moves the results down; the
    first upload of a step has no download to run beside and its last download no upload, so a
    step alone leaves each copy engine idle for about one chunk.  This class keeps ``depth``
    ``HostMapsStep`` objects (each with its own staging buffers) and gives them the steps in
    turn, each on a stream of its own: step ``i+1``'s uploads run under step ``i``'s downloads.
    Every step still reads all its inputs from, and writes all its results to, host memory.

    ``run`` returns an event that completes when that step's results are in the host buffers;
    the buffers of a step must not be reused before (``wait``).  Steps in flight at the same time
    need different host buffers.
    """

    def __init__(self, x_shape, kernel_size, stride=1, padding=0, depth=2, **kwargs):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        if depth > 1 and kwargs.get("chunk_images") is None:
            # the neighbouring steps hide a step's first upload and last download, so what is left
            # to save is the cost per copy: two chunks per step measured best on PCIe 5 x16
            # (c2, 128 images: 2.68 ms per step with 8 chunks, 2.50 ms with 2, 2.56 ms with 1)
            kwargs["chunk_images"] = max(1, -(-int(x_shape[0]) // 2))
        self.steps = [HostMapsStep(x_shape, kernel_size, stride, padding, **kwargs)
                      for _ in range(depth)]
        self.device = self.steps[0].device
        with torch.cuda.device(self.device):
            self.streams = [torch.cuda.Stream(self.device) for _ in range(depth)]
        self.depth, self.count = depth, 0
        self.x_shape, self.y_shape, self.w_shape = (self.steps[0].x_shape, self.steps[0].y_shape,
                                                    self.steps[0].w_shape)
        self.h2d_bytes, self.d2h_bytes = self.steps[0].h2d_bytes, self.steps[0].d2h_bytes
        self.launches_per_run = self.steps[0].launches_per_run

    def run(self, x, w, dy, y, dx, dw):
        """Queues one step (arguments as ``HostMapsStep.run``) behind the step that used the same
        slot ``depth`` steps ago, and beside the others; returns the event of its completion.
        Work queued earlier on the caller's current stream is waited for, as a single step would."""
        k = self.count % self.depth
        self.count += 1
        stream = self.streams[k]
        with torch.cuda.device(self.device):
            stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(stream):
                self.steps[k].run(x, w, dy, y, dx, dw)
                done = torch.cuda.Event()
                done.record(stream)
        return done

    @staticmethod
    def wait(event):
        event.synchronize()

    def synchronize(self):
        for s in self.streams:
            s.synchronize()
