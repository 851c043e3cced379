"""Batch sharding across GPUs: the only multi-GPU structure this path has.

Images are independent, so forward and backward-input need no communication: each rank
(one process per GPU) runs them on its contiguous slice of the batch.  The filter gradient
is a sum over the batch, so the local dW of every layer is packed into one flat fp32
buffer and summed with a single ``all_reduce`` (NCCL over NVLink on GPUs, gloo in the CPU
tests), on a side stream so it can overlap the next step's forward.

The reference has no distributed code; this module is new surface, outside its API.
"""
import torch
import torch.distributed as dist

__all__ = ["shard_bounds", "shard_batch", "FilterGradReducer"]


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
