"""The depthwise layers of a network as one unit: module form, interchange with
``nn.Conv2d(groups=C)``, and a graph-replayed training step that reports images per second.

The reference's README claims its speed-up on "EfficientNet forward time" (README.md:10); the
layers it accelerates there are the network's depthwise convolutions, each fed by the pointwise
convolutions between them (which are not part of this library).  ``DepthwiseStack`` holds those
depthwise layers as ``DepthwiseConv2d`` modules (torch_dwconv/dwconv.py:133-175); ``StackStep``
runs forward, backward-input and backward-filter of every layer over static buffers, the way the
stack is benchmarked: each layer has its own input map and output gradient.
"""
import torch
from torch import nn

from . import _lib
from .dwconv import DepthwiseConv2d

# (channels, map height = width, filter, stride) of the depthwise layers of EfficientNet-B0 at
# 224 x 224 input; padding is filter // 2
EFFICIENTNET_B0_DEPTHWISE = (
    (32, 112, 3, 1), (96, 112, 3, 2), (144, 56, 5, 2), (240, 28, 3, 2),
    (480, 14, 5, 1), (672, 14, 5, 2), (1152, 7, 3, 1),
)

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.float64: _lib.F64,
           torch.bfloat16: _lib.BF16}


def from_conv2d(conv):
    """``DepthwiseConv2d`` sharing the weight VALUES of a depthwise ``nn.Conv2d``."""
    if not isinstance(conv, nn.Conv2d):
        raise TypeError(f"expected nn.Conv2d, got {type(conv).__name__}")
    kh, kw = conv.kernel_size
    if kh != kw:
        raise ValueError("DepthwiseConv2d takes one kernel_size (square filters)")
    if isinstance(conv.padding, str):
        raise ValueError("string padding is not supported")
    m = DepthwiseConv2d(conv.in_channels, conv.out_channels, kh, stride=conv.stride,
                        padding=conv.padding, dilation=conv.dilation, groups=conv.groups,
                        bias=conv.bias is not None, padding_mode=conv.padding_mode)
    m.load_state_dict({"weight": conv.weight.detach()})  # same key, same [C,1,k,k] shape
    return m.to(device=conv.weight.device, dtype=conv.weight.dtype)


def to_conv2d(module):
    """Depthwise ``nn.Conv2d`` (no bias) carrying a ``DepthwiseConv2d``'s weight values."""
    C = module.weight.shape[0]
    conv = nn.Conv2d(C, C, module.kernel_size, stride=module.stride, padding=module.padding,
                     groups=C, bias=False)
    conv.load_state_dict(module.state_dict())
    return conv.to(device=module.weight.device, dtype=module.weight.dtype)


class DepthwiseStack(nn.Module):
    """The depthwise layers of a network; ``forward`` takes one input map per layer."""

    def __init__(self, layers=EFFICIENTNET_B0_DEPTHWISE):
        super().__init__()
        self.spec = tuple(tuple(int(v) for v in l) for l in layers)
        self.layers = nn.ModuleList(
            DepthwiseConv2d(C, C, k, stride=s, padding=k // 2) for (C, H, k, s) in self.spec)

    def forward(self, inputs):
        if len(inputs) != len(self.layers):
            raise ValueError(f"expected {len(self.layers)} input maps, got {len(inputs)}")
        return [layer(x) for layer, x in zip(self.layers, inputs)]

    def input_shapes(self, batch):
        return [(batch, C, H, H) for (C, H, k, s) in self.spec]


class StackStep:
    """One training step of a ``DepthwiseStack`` over static device buffers: every layer's
    forward, then every layer's backward-input and backward-filter in reverse order, launched
    through the C entry points and replayed as one CUDA graph.

    ``x[i]``, ``dy[i]`` are the buffers to fill; ``y[i]``, ``dx[i]``, ``dw[i]`` hold the results
    after ``run()``.  Both gradients of a layer come from the fused backward call (one read of
    ``dy``).  ``exchanges`` (one ``PeerFilterExchange`` per layer, optional) makes ``dw`` the
    sum over all ranks: each layer's gradient is sent to the other GPUs inside the kernel that
    finishes it, the remaining layers' kernels hide the flight of those stores, and the step
    ends with one small kernel per layer that adds the ranks' values, so ``dw`` is the world sum
    of THIS step when ``run()`` has completed (as the reference returns the complete gradient
    from ``backward``, torch_dwconv/dwconv.py:66-70).
    """

    def __init__(self, stack, batch, device="cuda", use_graph=True, exchanges=None):
        self.stack, self.batch = stack, int(batch)
        self.device = torch.device(device)
        self.exchanges = exchanges
        L = _lib.lib
        self.x, self.dy, self.y, self.dx, self.dw, self._geo = [], [], [], [], [], []
        with torch.cuda.device(self.device):
            for layer, (C, H, k, s) in zip(stack.layers, stack.spec):
                w = layer.weight
                if w.device != self.device or w.dtype not in _DTYPES:
                    raise RuntimeError(f"dwconv_b200.StackStep: weights must be on {self.device} in "
                                       f"float32, float16 or float64 (got {w.device}, {w.dtype})")
                p = k // 2
                Ho = L.dwconv_b200_out_size(H, 1, p, p, k, s)
                mk = lambda *shape: torch.zeros(shape, dtype=w.dtype, device=self.device)  # noqa: E731
                self.x.append(mk(batch, C, H, H))
                self.dx.append(mk(batch, C, H, H))
                self.y.append(mk(batch, C, Ho, Ho))
                self.dy.append(mk(batch, C, Ho, Ho))
                self.dw.append(mk(C, 1, k, k))
                shape = _lib.Shape(batch, C, H, H, k, k, s, s, p, p, Ho, Ho)
                nws = int(L.dwconv_b200_backward_filter_workspace_bytes(_DTYPES[w.dtype], shape))
                self._geo.append((shape, _DTYPES[w.dtype], nws,
                                  torch.empty(max(nws, 16), dtype=torch.uint8, device=self.device)))
            self._stream = torch.cuda.Stream(self.device)
        self._graph = None
        self._use_graph = bool(use_graph)
        self._ran = 0

    def _enqueue(self, st):
        L = _lib.lib
        n = len(self._geo)
        for i in range(n):
            shape, code, nws, ws = self._geo[i]
            _lib.check(L.dwconv_b200_forward(self.x[i].data_ptr(), self.stack.layers[i].weight.data_ptr(),
                                             self.y[i].data_ptr(), code, shape, st), "forward")
        for i in reversed(range(n)):
            shape, code, nws, ws = self._geo[i]
            w = self.stack.layers[i].weight
            if self.exchanges is not None:
                self.exchanges[i].launch_backward(
                    self.x[i].data_ptr(), self.dy[i].data_ptr(), w.data_ptr(), self.dx[i].data_ptr(),
                    None, ws.data_ptr(), nws, shape, st)
            else:
                _lib.check(L.dwconv_b200_backward(
                    self.x[i].data_ptr(), self.dy[i].data_ptr(), w.data_ptr(), self.dx[i].data_ptr(),
                    self.dw[i].data_ptr(), ws.data_ptr(), nws, code, shape, st), "backward")
        if self.exchanges is not None:
            for i in reversed(range(n)):
                self.exchanges[i].finish(self.dw[i], stream=st)

    def run(self):
        """Queues one step on the current stream (the first call runs eagerly: kernel set-up;
        the second records the graph; later calls replay it)."""
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream(self.device)
            if not self._use_graph or self._ran == 0:
                self._enqueue(cur.cuda_stream)
            else:
                if self._graph is None:
                    torch.cuda.synchronize(self.device)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self._stream):
                        self._enqueue(torch.cuda.current_stream(self.device).cuda_stream)
                    self._graph = g
                self._graph.replay()
            self._ran += 1

    def finish(self):
        """Kept for callers of the earlier, pipelined form: ``run()`` now completes the sum
        over the ranks itself, so there is nothing left to do."""

    def images_per_second(self, steps=50, warmup=5):
        """Device-timed throughput of ``run()`` (CUDA events on the current stream)."""
        for _ in range(max(warmup, 2)):
            self.run()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream(self.device)
        a.record(cur)
        for _ in range(steps):
            self.run()
        z.record(cur)
        z.synchronize()
        return self.batch * steps / (a.elapsed_time(z) * 1e-3)

