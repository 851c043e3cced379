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


def use_dwconv2d_small(input, weight, up, stride, padding):
    """torch_dwconv/dwconv.py:9-12."""
    return _C.use_dwconv2d_small(input, weight, up[0], up[1], stride[0], stride[1],
                                 padding[0], padding[1])


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
        _C._check_cuda(input, "input")
        _C._check_cuda(kernel, "kernel")
        code = _C._dtype_code(input, kernel)
        stride = tuple(int(v) for v in stride)
        pad = tuple(int(v) for v in pad)
        _C._check_filter(input, kernel)
        input = input.contiguous()
        kernel = kernel.contiguous()
        shape = _forward_shape(input, kernel, stride, pad)
        out = torch.empty((shape.N, shape.C, shape.Ho, shape.Wo), dtype=input.dtype,
                          device=input.device)
        with _C._on_device(input):
            st = _lib.lib.dwconv_b200_forward(input.data_ptr(), kernel.data_ptr(), out.data_ptr(),
                                              code, shape, _C._stream(input))
        _lib.check(st, "forward")
        ctx.save_for_backward(input, kernel)
        ctx.shape = shape
        ctx.code = code
        ctx.stride = stride
        ctx.pad = pad
        ctx.use_small = small
        # what the reference's backward passes to its operator (dwconv.py:39-44);
        # kept for introspection, the C entry point takes the forward geometry
        ctx.g_pad = (shape.kh - pad[0] - 1, shape.H - shape.Ho * stride[0] + pad[0],
                     shape.kw - pad[1] - 1, shape.W - shape.Wo * stride[1] + pad[1])
        return out

    @staticmethod
    def backward(ctx, grad_output):
        input, kernel = ctx.saved_tensors
        shape, code = ctx.shape, ctx.code
        if tuple(grad_output.shape) != (shape.N, shape.C, shape.Ho, shape.Wo):
            raise RuntimeError(f"depthwise_conv2d backward: grad_output has shape "
                               f"{tuple(grad_output.shape)}, expected "
                               f"{(shape.N, shape.C, shape.Ho, shape.Wo)}")
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


depthwise_conv2d_fn = DepthwiseConv2dFunction.apply


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
