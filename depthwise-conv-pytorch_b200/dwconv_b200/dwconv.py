"""Public API with the names and behaviour of ``torch_dwconv``
(torch_dwconv/dwconv.py): ``depthwise_conv2d``, ``DepthwiseConv2d``,
``DepthwiseConv2dFunction``, ``make_tuple``, ``check_options``.

Differences from the reference, all deliberate:

* no tensor ever goes to ``torch.nn.functional.conv2d`` from ``depthwise_conv2d``:
  the shapes the reference hands to it (small maps with stride 2 or a large
  filter, dwconv.py:125-128) are served by this library's own kernels, so a CPU
  tensor always raises ``RuntimeError('input must be a CUDA tensor')``;
* backward only computes the gradients autograd asks for, and returns one value
  per forward input (the reference always computes both and returns six);
* fp16 accumulates in fp32.
"""
import torch
from torch import nn
from torch.autograd import Function
from torch.nn import functional as F

from . import _C, _lib

_native = _lib.native


def use_dwconv2d_small(input, weight, up, stride, padding):
    """torch_dwconv/dwconv.py:9-12."""
    return _C.use_dwconv2d_small(input, weight, up[0], up[1], stride[0], stride[1],
                                 padding[0], padding[1])


def _is_channels_last(t):
    """A 4-d tensor laid out [n][h][w][c] (and not at the same time plain contiguous, which
    happens when C or H*W is 1)."""
    return (t.dim() == 4 and not t.is_contiguous()
            and t.is_contiguous(memory_format=torch.channels_last))


def _nhwc_served(code, kernel, stride):
    """What the channels-last kernels cover: square 3x3 / 5x5 / 7x7, equal strides 1 or 2,
    fp32 / fp16 / bf16 (other geometries are made contiguous NCHW, as the reference does)."""
    kh, kw = kernel.shape[2], kernel.shape[3]
    return (kh == kw and kh in (3, 5, 7) and stride[0] == stride[1] and stride[0] in (1, 2)
            and code in (_lib.F32, _lib.F16, _lib.BF16))


def _forward_shape(input, kernel, stride, pad):
    N, C, H, W = input.shape
    kh, kw = kernel.shape[2], kernel.shape[3]
    oh = _C.out_size(H, 1, pad[0], pad[0], kh, stride[0])
    ow = _C.out_size(W, 1, pad[1], pad[1], kw, stride[1])
    if oh <= 0 or ow <= 0:
        raise RuntimeError(
            f"depthwise_conv2d: filter {kh}x{kw} does not fit the padded input "
            f"{H + 2 * pad[0]}x{W + 2 * pad[1]}")
    return _lib.Shape(N, C, H, W, kh, kw, stride[0], stride[1], pad[0], pad[1], oh, ow)


_WS_BYTES = {}


def _workspace_bytes(code, s):
    """``dwconv_b200_backward_filter_workspace_bytes``, remembered per geometry."""
    key = (code, s.N, s.C, s.H, s.W, s.kh, s.kw, s.sh, s.sw, s.ph, s.pw, s.Ho, s.Wo)
    n = _WS_BYTES.get(key)
    if n is None:
        if len(_WS_BYTES) > 4096:
            _WS_BYTES.clear()
        n = _WS_BYTES[key] = int(_lib.lib.dwconv_b200_backward_filter_workspace_bytes(code, s))
    return n


class DepthwiseConv2dFunction(Function):
    """Autograd function; argument list of torch_dwconv/dwconv.py:15-46.

    ``small`` is accepted for call compatibility; kernel selection happens inside
    the library per shape, so the flag does not change the result.
    """

    @staticmethod
    def forward(ctx, input, kernel, stride, pad, small=False):
        stride = tuple(int(v) for v in stride)
        pad = tuple(int(v) for v in pad)
        ctx.stride, ctx.pad, ctx.use_small = stride, pad, small
        if _native is not None:
            # checks, layout decisions, allocation and the library call in one compiled call
            out, input, kernel, ctx.nhwc = _native.forward(input, kernel, stride[0], stride[1],
                                                           pad[0], pad[1])
            ctx.save_for_backward(input, kernel)
            return out
        _C._check_cuda(input, "input")
        _C._check_cuda(kernel, "kernel")
        code = _C._dtype_code(input, kernel)
        _C._check_filter(input, kernel)
        # channels-last maps are read and written in place (no NCHW copy); the result follows
        # the input's layout, as PyTorch's own convolution does
        nhwc = _is_channels_last(input) and _nhwc_served(code, kernel, stride)
        if not nhwc:
            input = input.contiguous()
        kernel = kernel.contiguous()
        shape = _forward_shape(input, kernel, stride, pad)
        out = torch.empty((shape.N, shape.C, shape.Ho, shape.Wo), dtype=input.dtype,
                          device=input.device,
                          memory_format=torch.channels_last if nhwc else torch.contiguous_format)
        with _C._on_device(input):
            if nhwc:
                st = _lib.lib.dwconv_b200_forward_nhwc(input.data_ptr(), kernel.data_ptr(),
                                                       out.data_ptr(), code, shape, None,
                                                       _C._stream(input))
            else:
                st = _lib.lib.dwconv_b200_forward(input.data_ptr(), kernel.data_ptr(), out.data_ptr(),
                                                  code, shape, _C._stream(input))
        _lib.check(st, "forward")
        ctx.nhwc = nhwc
        ctx.save_for_backward(input, kernel)
        ctx.shape = shape
        ctx.code = code
        return out

    @staticmethod
    def backward(ctx, grad_output):
        input, kernel = ctx.saved_tensors
        if _native is not None:
            stride, pad = ctx.stride, ctx.pad
            grad_input, grad_kernel = _native.backward(
                input, grad_output, kernel, stride[0], stride[1], pad[0], pad[1], ctx.nhwc,
                ctx.needs_input_grad[0], ctx.needs_input_grad[1])
            if _lib.CHECK_STATUS:
                _lib.check_device_status("backward")
            return grad_input, grad_kernel, None, None, None
        shape, code = ctx.shape, ctx.code
        if tuple(grad_output.shape) != (shape.N, shape.C, shape.Ho, shape.Wo):
            raise RuntimeError(f"depthwise_conv2d backward: grad_output has shape "
                               f"{tuple(grad_output.shape)}, expected "
                               f"{(shape.N, shape.C, shape.Ho, shape.Wo)}")
        if ctx.nhwc:
            return DepthwiseConv2dFunction._backward_nhwc(ctx, grad_output, input, kernel)
        grad_output = grad_output.contiguous()
        grad_input = grad_kernel = None
        with _C._on_device(input):
            stream = _C._stream(input)
            want_dx, want_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
            if want_dw:
                nbytes = _workspace_bytes(code, shape)
                ws = torch.empty(nbytes, dtype=torch.uint8, device=input.device)
                grad_kernel = torch.empty_like(kernel)
            if want_dx:
                grad_input = torch.empty_like(input)
            if want_dx and want_dw:
                # both gradients from one pass over grad_output
                st = _lib.lib.dwconv_b200_backward(
                    input.data_ptr(), grad_output.data_ptr(), kernel.data_ptr(),
                    grad_input.data_ptr(), grad_kernel.data_ptr(), ws.data_ptr(), nbytes, code,
                    shape, stream)
                _lib.check(st, "backward")
            elif want_dx:
                st = _lib.lib.dwconv_b200_backward_input(
                    grad_output.data_ptr(), kernel.data_ptr(), grad_input.data_ptr(), code, shape,
                    stream)
                _lib.check(st, "backward_input")
            elif want_dw:
                st = _lib.lib.dwconv_b200_backward_filter(
                    input.data_ptr(), grad_output.data_ptr(), grad_kernel.data_ptr(),
                    ws.data_ptr(), nbytes, code, shape, stream)
                _lib.check(st, "backward_filter")
            if _lib.CHECK_STATUS:
                _lib.check_device_status("backward")
        return grad_input, grad_kernel, None, None, None


    @staticmethod
    def _backward_nhwc(ctx, grad_output, input, kernel):
        """Both gradients for a channels-last forward: dy is taken channels-last (a copy only
        if autograd hands it over in another layout), dx is channels-last like the input."""
        shape, code = ctx.shape, ctx.code
        grad_output = grad_output.contiguous(memory_format=torch.channels_last)
        grad_input = grad_kernel = None
        with _C._on_device(input):
            stream = _C._stream(input)
            if ctx.needs_input_grad[0] and ctx.needs_input_grad[1]:
                nbytes = _workspace_bytes(code, shape)
                ws = torch.empty(nbytes, dtype=torch.uint8, device=input.device)
                grad_input = torch.empty_like(input, memory_format=torch.channels_last)
                grad_kernel = torch.empty_like(kernel)
                st = _lib.lib.dwconv_b200_backward_nhwc(
                    input.data_ptr(), grad_output.data_ptr(), kernel.data_ptr(), grad_input.data_ptr(),
                    grad_kernel.data_ptr(), ws.data_ptr(), nbytes, code, shape, stream)
                _lib.check(st, "backward_nhwc")
                if _lib.CHECK_STATUS:
                    _lib.check_device_status("backward")
                return grad_input, grad_kernel, None, None, None
            if ctx.needs_input_grad[0]:
                grad_input = torch.empty_like(input, memory_format=torch.channels_last)
                st = _lib.lib.dwconv_b200_backward_input_nhwc(
                    grad_output.data_ptr(), kernel.data_ptr(), grad_input.data_ptr(), code, shape,
                    stream)
                _lib.check(st, "backward_input_nhwc")
            if ctx.needs_input_grad[1]:
                nbytes = _workspace_bytes(code, shape)
                ws = torch.empty(nbytes, dtype=torch.uint8, device=input.device)
                grad_kernel = torch.empty_like(kernel)
                st = _lib.lib.dwconv_b200_backward_filter_nhwc(
                    input.data_ptr(), grad_output.data_ptr(), grad_kernel.data_ptr(), ws.data_ptr(),
                    nbytes, code, shape, stream)
                _lib.check(st, "backward_filter_nhwc")
            if _lib.CHECK_STATUS:
                _lib.check_device_status("backward")
        return grad_input, grad_kernel, None, None, None


depthwise_conv2d_fn = DepthwiseConv2dFunction.apply

_ACTIVATIONS = {None: _lib.ACT_NONE, "none": _lib.ACT_NONE, "relu": _lib.ACT_RELU,
                "relu6": _lib.ACT_RELU6, "silu": _lib.ACT_SILU, "swish": _lib.ACT_SILU,
                "hardswish": _lib.ACT_HARDSWISH}


class DepthwiseConv2dEpilogueFunction(Function):
    """``act(conv(input, kernel) * scale[c] + bias[c])`` in one kernel (new surface: the
    reference rejects a bias, torch_dwconv/dwconv.py:108-109).

    Gradients flow to ``input`` and ``kernel`` for the activations whose derivative can be read
    off the output (none, ReLU, ReLU6): ``grad_output`` is masked and scaled with elementwise
    torch operations and handed to the fused backward.  ``scale`` and ``bias`` are constants
    (a folded batch-norm): they get no gradient.  SiLU and hard-swish are forward-only.
    """

    @staticmethod
    def forward(ctx, input, kernel, scale, bias, act, stride, pad):
        _C._check_cuda(input, "input")
        _C._check_cuda(kernel, "kernel")
        code = _C._dtype_code(input, kernel)
        _C._check_filter(input, kernel)
        C = input.shape[1]
        for t, name in ((scale, "scale"), (bias, "bias")):
            if t is not None:
                _C._dtype_code(input, t)
                if t.numel() != C:
                    raise RuntimeError(f"depthwise_conv2d_epilogue: {name} must have {C} elements, "
                                       f"got {tuple(t.shape)}")
        input = input.contiguous()
        kernel = kernel.contiguous()
        scale_c = scale.contiguous() if scale is not None else None
        bias_c = bias.contiguous() if bias is not None else None
        shape = _forward_shape(input, kernel, stride, pad)
        out = torch.empty((shape.N, shape.C, shape.Ho, shape.Wo), dtype=input.dtype,
                          device=input.device)
        ep = _lib.Epilogue(scale_c.data_ptr() if scale_c is not None else None,
                           bias_c.data_ptr() if bias_c is not None else None, act)
        with _C._on_device(input):
            st = _lib.lib.dwconv_b200_forward_epilogue(input.data_ptr(), kernel.data_ptr(),
                                                       out.data_ptr(), code, shape, ep,
                                                       _C._stream(input))
        _lib.check(st, "forward_epilogue")
        ctx.save_for_backward(input, kernel, scale_c, out)
        ctx.shape, ctx.code, ctx.act = shape, code, act
        return out

    @staticmethod
    def backward(ctx, grad_output):
        input, kernel, scale, out = ctx.saved_tensors
        if ctx.act not in (_lib.ACT_NONE, _lib.ACT_RELU, _lib.ACT_RELU6):
            raise RuntimeError("depthwise_conv2d_epilogue: this activation is forward-only "
                               "(its derivative is not a function of the output)")
        g = grad_output
        if scale is not None:
            g = g * scale.view(1, -1, 1, 1)
        if ctx.act == _lib.ACT_RELU:
            g = torch.where(out > 0, g, torch.zeros((), dtype=g.dtype, device=g.device))
        elif ctx.act == _lib.ACT_RELU6:
            g = torch.where((out > 0) & (out < 6), g, torch.zeros((), dtype=g.dtype, device=g.device))
        g = g.contiguous()
        shape, code = ctx.shape, ctx.code
        grad_input = grad_kernel = None
        with _C._on_device(input):
            stream = _C._stream(input)
            nbytes = _workspace_bytes(code, shape)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=input.device)
            grad_input = torch.empty_like(input)
            grad_kernel = torch.empty_like(kernel)
            st = _lib.lib.dwconv_b200_backward(
                input.data_ptr(), g.data_ptr(), kernel.data_ptr(), grad_input.data_ptr(),
                grad_kernel.data_ptr(), ws.data_ptr(), nbytes, code, shape, stream)
            _lib.check(st, "backward")
        return grad_input, grad_kernel, None, None, None, None, None


def depthwise_conv2d_epilogue(input, weight, scale=None, bias=None, activation=None, stride=1,
                              padding=0):
    """Depthwise convolution followed, inside the same kernel, by a per-channel scale and
    shift and an activation: ``act(conv(input, weight) * scale[c] + bias[c])``.

    ``scale`` / ``bias``: 1-d tensors of C elements (or ``None``), same dtype and device as the
    input.  ``activation``: ``None``, ``'relu'``, ``'relu6'``, ``'silu'`` (= ``'swish'``) or
    ``'hardswish'``.  Opt-in: ``depthwise_conv2d`` keeps the reference's behaviour of rejecting
    a bias.
    """
    stride = make_tuple(stride, 2)
    padding = make_tuple(padding, 2)
    check_options(input.shape[1], weight.shape[0], 1, None, None)
    if activation not in _ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}; expected one of "
                         f"{sorted(k for k in _ACTIVATIONS if k)}")
    for t, name in ((scale, "scale"), (bias, "bias")):
        if t is not None and t.requires_grad:
            raise RuntimeError(f"depthwise_conv2d_epilogue: {name} is a constant of the fused "
                               "epilogue and gets no gradient; detach it")
    return DepthwiseConv2dEpilogueFunction.apply(
        input, weight, scale, bias, _ACTIVATIONS[activation],
        tuple(int(v) for v in stride), tuple(int(v) for v in padding))


def make_tuple(value, n_value):
    """int -> n-tuple, 1-sequence -> repeated, n-sequence -> itself (dwconv.py:76-91)."""
    if not isinstance(value, (list, tuple)):
        return (value,) * n_value
    n_item = len(value)
    if n_item > n_value:
        raise ValueError(
            f'Number items does not match with requirements: {n_item}, expected: {n_value}'
        )
    if n_item == n_value:
        return value
    return value * n_value


def check_options(in_channels, out_channels, dilation, groups, bias, padding_mode='zeros'):
    """Restrictions of the depthwise operator, with the reference's messages (dwconv.py:94-112)."""
    dilation = make_tuple(dilation, 2)
    if dilation[0] > 1 or dilation[1] > 1:
        raise ValueError('DepthwiseConv2d does not support dilations > 1')
    if groups is not None and groups != in_channels:
        raise ValueError('DepthwiseConv2d does not support groups != in_channels')
    if in_channels != out_channels:
        raise ValueError('DepthwiseConv2d does not support in_channels != out_channels')
    if bias:
        raise ValueError('DepthwiseConv2d does not support bias')
    if padding_mode != 'zeros':
        raise ValueError('DepthwiseConv2d does not non-zero paddings')


def depthwise_conv2d(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=None):
    """Depthwise cross-correlation, multiplier 1 (dwconv.py:115-130)."""
    stride = make_tuple(stride, 2)
    padding = make_tuple(padding, 2)
    check_options(input.shape[1], weight.shape[0], dilation, groups, bias)
    small = use_dwconv2d_small(input, weight, (1, 1), stride, padding)
    return depthwise_conv2d_fn(input, weight, stride, padding, small)


class DepthwiseConv2d(nn.Module):
    """Module form (dwconv.py:133-175); ``state_dict`` is ``{'weight': [C,1,k,k]}``."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1,
                 groups=None, bias=False, padding_mode='zeros', custom=True):
        super().__init__()
        check_options(in_channels, out_channels, dilation, groups, bias, padding_mode)
        self.stride = stride
        self.padding = padding
        self.in_channel = in_channels
        self.kernel_size = kernel_size
        self.weight = nn.Parameter(torch.randn(out_channels, 1, kernel_size, kernel_size))
        self.custom = custom

    def forward(self, input):
        if self.custom:
            return depthwise_conv2d(input, self.weight, None, self.stride, self.padding)
        # custom=False is the caller asking for PyTorch's own operator (dwconv.py:166-173)
        return F.conv2d(input, self.weight, stride=self.stride, padding=self.padding,
                        groups=input.shape[1])
