"""Import-name shim: ``import torch_dwconv`` resolves to dwconv_b200.

Put ``depthwise-conv-pytorch_b200/compat`` (and ``depthwise-conv-pytorch_b200``) on
``sys.path`` and code written against rosinality/depthwise-conv-pytorch --
including its test files -- runs unchanged (torch_dwconv/__init__.py:1).
"""
from dwconv_b200 import DepthwiseConv2d, depthwise_conv2d  # noqa: F401
from dwconv_b200 import _C, dwconv  # noqa: F401
