"""``flow.nn.functional``: torch.nn.functional plus the fused ops of ``flow._C``."""
from torch.nn.functional import *  # noqa: F401,F403
import torch.nn.functional as _F

from .._C import (fused_bias_add_dropout, fused_bias_add_gelu, fused_scale_mask_softmax,  # noqa: F401
                  fused_scale_mask_softmax_dropout, fused_scale_tril_softmax_mask_scale)


def __getattr__(name):
    return getattr(_F, name)


def conv2d(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """torch's conv2d, or the implicit-GEMM tcgen05 kernels for bf16 channels-last stride-1 "same" convolutions."""
    from .modules.conv import conv2d as _conv2d
    return _conv2d(input, weight, bias, stride, padding, dilation, groups)
