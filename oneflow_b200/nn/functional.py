"""``flow.nn.functional``: torch.nn.functional plus the fused ops of ``flow._C``."""
from torch.nn.functional import *  # noqa: F401,F403
import torch.nn.functional as _F

from .._C import (fused_bias_add_dropout, fused_bias_add_gelu, fused_scale_mask_softmax,  # noqa: F401
                  fused_scale_mask_softmax_dropout, fused_scale_tril_softmax_mask_scale)


def __getattr__(name):
    return getattr(_F, name)
