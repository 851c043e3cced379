"""dwconv_b200: depthwise conv2d for B200, a drop-in for ``torch_dwconv``."""
from .dwconv import (DepthwiseConv2d, DepthwiseConv2dFunction, check_options,  # noqa: F401
                     depthwise_conv2d, depthwise_conv2d_epilogue, depthwise_conv2d_fn, make_tuple,
                     use_dwconv2d_small)
from . import _C  # noqa: F401
from .host import HostMapsPipeline, HostMapsStep  # noqa: F401
from .stack import (EFFICIENTNET_B0_DEPTHWISE, DepthwiseStack, StackStep,  # noqa: F401
                    from_conv2d, to_conv2d)

__all__ = ["depthwise_conv2d", "depthwise_conv2d_epilogue", "DepthwiseConv2d", "HostMapsStep", "HostMapsPipeline", "DepthwiseStack", "StackStep",
           "from_conv2d", "to_conv2d"]
