"""Batch sharding across GPUs: the only multi-GPU structure this path has.

Images are independent, so forward and backward-input need no communication: each rank
(one process per GPU) runs them on its contiguous slice of the batch.  The filter gradient
is a sum over the batch, so the local dW of every layer is packed into one flat fp32
buffer and summed with a single ``all_reduce`` (NCCL over NVLink on GPUs, gloo in the CPU
tests), on a side stream so it can overlap the next step's forward -- or, on the GPUs of one
node, summed inside the kernel that finishes the gradient (``PeerFilterExchange``).

The reference has no distributed code; this module is new surface, outside its API.
"""
import torch
import torch.distributed as dist

import os

__all__ = ["shard_bounds", "shard_batch", "FilterGradReducer", "PeerFilterExchange",
           "bind_to_gpu_numa_node"]


def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(device_index, sysfs="/sys"):
    """Restricts the calling thread (and the threads it starts later) to the CPUs of the NUMA
    node the GPU is attached to, so that pinned host buffers allocated afterwards live in that
    node's memory and host<->device copies do not cross sockets.  With one process per GPU on a
    two-socket machine, unbound ranks otherwise allocate wherever they happen to run.
    Returns what was done; never raises (a container may hide sysfs)."""
    info = {"bound": False}
    try:
        props = torch.cuda.get_device_properties(device_index)
        addr = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        info["pci"] = addr
        with open(f"{sysfs}/bus/pci/devices/{addr}/numa_node") as f:
            node = int(f.read().strip())
        info["node"] = node
        if node < 0:
            return info
        with open(f"{sysfs}/devices/system/node/node{node}/cpulist") as f:
            cpus = _parse_cpulist(f.read()) & os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info.update(bound=True, cpus=len(cpus))
    except (OSError, ValueError, AttributeError, RuntimeError) as e:
        info["why"] = f"{type(e).__name__}: {e}"
    return info


def shard_bounds(n, world_size, rank):
    """[lo, hi) of rank's contiguous slice of n images: lo = rank*n // world_size."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return (rank * n) // world_size, ((rank + 1) * n) // world_size


def shard_batch(t, world_size, rank):
    """Rank's slice of a batch-major tensor (a view; images are contiguous)."""
    lo, hi = shard_bounds(t.shape[0], world_size, rank)
    return t[lo:hi]


class FilterGradReducer:
    """Sums the filter gradients of a fixed list of layers over all ranks with one collective.

    ``shapes``: one ``(C, 1, kh, kw)`` per layer.  ``reduce(grads)`` takes the local
    gradients (any float dtype), returns the global sums in the same dtypes.  Summation is in
    fp32 whatever the storage dtype, and for a fixed world size and algorithm the reduction
    order inside the collective is fixed, so results repeat run to run.
    """

    def __init__(self, shapes, device, group=None, side_stream=True):
        self.shapes = [tuple(s) for s in shapes]
        self.sizes = [int(torch.Size(s).numel()) for s in self.shapes]
        self.offsets = [0]
        for n in self.sizes:
            self.offsets.append(self.offsets[-1] + n)
        self.device = torch.device(device)
        self.group = group
        self.flat = torch.zeros(self.offsets[-1], dtype=torch.float32, device=self.device)
        self.stream = (torch.cuda.Stream(device=self.device)
                       if (side_stream and self.device.type == "cuda") else None)
        self._work = None

    @property
    def nbytes(self):
        return self.flat.numel() * 4

    def pack(self, grads):
        if len(grads) != len(self.shapes):
            raise ValueError(f"expected {len(self.shapes)} gradients, got {len(grads)}")
        for g, shape, lo, hi in zip(grads, self.shapes, self.offsets, self.offsets[1:]):
            if tuple(g.shape) != shape:
                raise ValueError(f"gradient shape {tuple(g.shape)} != {shape}")
            self.flat[lo:hi].copy_(g.reshape(-1))

    def start(self, grads):
        """Pack and launch the all-reduce; returns immediately on CUDA."""
        if self.stream is None:
            self.pack(grads)
            self._work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group,
                                         async_op=True)
            return
        cur = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            self.pack(grads)
            self._work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group,
                                         async_op=True)

    def finish(self, like):
        """Wait for the all-reduce; returns the summed gradients cast like ``like``."""
        if self._work is not None:
            self._work.wait()
            self._work = None
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        return [self.flat[lo:hi].view(shape).to(g.dtype)
                for g, shape, lo, hi in zip(like, self.shapes, self.offsets, self.offsets[1:])]

    def reduce(self, grads):
        self.start(grads)
        return self.finish(grads)


class PeerFilterExchange:
    """Filter gradient of ONE layer summed over the GPUs of a node inside the kernel that
    finishes it (``dwconv_b200_backward_filter_exchange``): no separate collective launch.

    Construction is collective over ``group`` (every rank creates the object for the same
    layers in the same order): each rank allocates its exchange buffer, the 64-byte
    inter-process handles are all-gathered on the host, and every rank maps its peers'
    buffers.  ``torch.distributed`` is used for that hand-shake only.

    The exchange is pipelined (a store to a peer needs several microseconds to become visible
    there): ``start(x, dy, ..., dw_prev)`` computes this call's local gradient, sends it to every
    rank and writes the PREVIOUS call's world sum into ``dw_prev``; ``finish(dw)`` completes the
    latest call.  ``backward_filter(x, dy)`` is ``start`` + ``finish``.  The world sum has
    identical bits on every rank.  All ranks must make the same calls.  Needs all ranks on one
    node with peer access between their GPUs; raises ``RuntimeError`` otherwise (use
    ``FilterGradReducer`` then).

    Tear-down is collective too: a peer's kernel stores into this rank's buffer, so no rank may
    free its buffer while any rank still has a call in flight.  ``close()`` therefore
    synchronises the device and meets the other ranks at a barrier before it unmaps and frees;
    every rank must call it (after its last ``finish``).  An object that is dropped without
    ``close()`` in a multi-rank run keeps its buffer until the process exits rather than risk
    freeing memory a peer is still writing.
    """

    def __init__(self, channels, kernel_size, dtype, device, group=None):
        from . import _lib
        import ctypes
        self._lib = _lib
        kh, kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        self.C, self.kh, self.kw = int(channels), int(kh), int(kw)
        self.dtype = dtype
        self.code = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.float64: _lib.F64,
           torch.bfloat16: _lib.BF16}[dtype]
        self.device = torch.device(device)
        self.group = group
        multi = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        self._ex = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib.dwconv_b200_exchange_create(
                self.code, self.C, self.kh, self.kw, self.world, self.rank,
                ctypes.byref(self._ex), handle), "exchange_create")
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
                _lib.check(_lib.lib.dwconv_b200_exchange_connect(self._ex, b"".join(handles)),
                           "exchange_connect")
                dist.barrier(group=group)  # nobody sends before every rank has mapped its peers
        self._ws = None

    def _prepare(self, x, dy, stride, padding):
        _lib = self._lib
        if (x.dim() != 4 or dy.dim() != 4 or tuple(dy.shape[:2]) != tuple(x.shape[:2])
                or x.shape[1] != self.C or x.dtype != self.dtype or dy.dtype != self.dtype
                or not x.is_contiguous() or not dy.is_contiguous()):
            raise RuntimeError(f"dwconv_b200.PeerFilterExchange: x {tuple(x.shape)} / dy "
                               f"{tuple(dy.shape)} must be contiguous {self.dtype} maps with the "
                               f"same batch and {self.C} channels")
        N, C, H, W = x.shape
        sh, sw = (stride, stride) if isinstance(stride, int) else stride
        ph, pw = (padding, padding) if isinstance(padding, int) else padding
        shape = _lib.Shape(N, C, H, W, self.kh, self.kw, sh, sw, ph, pw, dy.shape[2], dy.shape[3])
        nws = int(_lib.lib.dwconv_b200_backward_filter_workspace_bytes(self.code, shape))
        if self._ws is None or self._ws.numel() < nws:
            self._ws = torch.empty(nws, dtype=torch.uint8, device=self.device)
        return shape, nws

    def start(self, x, dy, stride=1, padding=0, dw_prev=None):
        """Local gradient of (x, dy), sent to all ranks; ``dw_prev`` (optional) receives the
        previous call's world sum."""
        shape, nws = self._prepare(x, dy, stride, padding)
        with torch.cuda.device(self.device):
            self.launch(x.data_ptr(), dy.data_ptr(), dw_prev.data_ptr() if dw_prev is not None else None,
                        self._ws.data_ptr(), nws, shape,
                        torch.cuda.current_stream(self.device).cuda_stream)

    def finish(self, dw=None, stream=None):
        """World sum of the latest ``start`` (waits for the peers' words if still in flight)."""
        if dw is None:
            dw = torch.empty((self.C, 1, self.kh, self.kw), dtype=self.dtype, device=self.device)
        with torch.cuda.device(self.device):
            st = stream if stream is not None else torch.cuda.current_stream(self.device).cuda_stream
            self._lib.check(self._lib.lib.dwconv_b200_exchange_finish(dw.data_ptr(), self._ex, st),
                            "exchange_finish")
        return dw

    def backward_filter(self, x, dy, stride=1, padding=0, dw=None):
        self.start(x, dy, stride, padding)
        return self.finish(dw)

    def launch(self, x_ptr, dy_ptr, dw_prev_ptr, ws_ptr, ws_bytes, shape, stream):
        """Raw-pointer form of ``start`` (what a CUDA-graph capture of a training step calls)."""
        self._lib.check(self._lib.lib.dwconv_b200_backward_filter_exchange(
            x_ptr, dy_ptr, dw_prev_ptr, ws_ptr, ws_bytes, self.code, shape, self._ex, stream),
            "backward_filter_exchange")

    def launch_backward(self, x_ptr, dy_ptr, w_ptr, dx_ptr, dw_prev_ptr, ws_ptr, ws_bytes, shape,
                        stream):
        """As ``launch``, with the fused backward's first pass: ``dx`` is written as well
        (``dwconv_b200_backward_exchange``)."""
        self._lib.check(self._lib.lib.dwconv_b200_backward_exchange(
            x_ptr, dy_ptr, w_ptr, dx_ptr, dw_prev_ptr, ws_ptr, ws_bytes, self.code, shape, self._ex,
            stream), "backward_exchange")

    def launch_allreduce(self, x_ptr, dy_ptr, w_ptr, dx_ptr, dw_ptr, ws_ptr, ws_bytes, shape, stream):
        """The whole sum inside the kernel that finishes the gradient: ``dw`` receives THIS
        call's world sum (the kernel waits for the other ranks' values after sending its own).
        With ``w_ptr`` / ``dx_ptr`` the first pass is the fused backward's and ``dx`` is written
        too; with both ``None`` only the filter gradient is computed."""
        L = self._lib.lib
        if dx_ptr is None:
            st = L.dwconv_b200_backward_filter_allreduce(x_ptr, dy_ptr, dw_ptr, ws_ptr, ws_bytes,
                                                         self.code, shape, self._ex, stream)
        else:
            st = L.dwconv_b200_backward_allreduce(x_ptr, dy_ptr, w_ptr, dx_ptr, dw_ptr, ws_ptr,
                                                  ws_bytes, self.code, shape, self._ex, stream)
        self._lib.check(st, "backward_allreduce")

    def allreduce_backward_filter(self, x, dy, stride=1, padding=0, dw=None):
        """Tensor form of ``launch_allreduce`` for the filter gradient alone."""
        shape, nws = self._prepare(x, dy, stride, padding)
        if dw is None:
            dw = torch.empty((self.C, 1, self.kh, self.kw), dtype=self.dtype, device=self.device)
        with torch.cuda.device(self.device):
            self.launch_allreduce(x.data_ptr(), dy.data_ptr(), None, None, dw.data_ptr(),
                                  self._ws.data_ptr(), nws, shape,
                                  torch.cuda.current_stream(self.device).cuda_stream)
        return dw

    def close(self):
        """Collective: every rank calls it, after its last ``finish``."""
        if not self._ex:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)   # this rank's calls have left the GPU
            if self.world > 1:
                dist.barrier(group=self.group)    # ... and so have everybody else's
            self._lib.lib.dwconv_b200_exchange_destroy(self._ex)
        self._ex = None

    def __del__(self):
        # Without the other ranks at a barrier it is not safe to free a buffer they may be
        # storing into: a single-rank object is destroyed, a multi-rank one is left to the
        # process exit.
        try:
            if getattr(self, "world", 2) == 1:
                self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass
