"""``flow.backends.cudnn`` (reference: python/oneflow/backends/cudnn/__init__.py:16-27)."""
import torch

from ...framework.config_util import api_enable_cudnn_conv_heuristic_search_algo as enable_conv_heuristic_search_algo  # noqa: F401
from ...framework.config_util import api_enable_cudnn_fused_normalization_add_relu as enable_fused_normalization_add_relu  # noqa: F401
from ...framework.config_util import api_reserved_device_mem_mbyte as set_reserved_mem_mbytes  # noqa: F401

benchmark = False


def __getattr__(name):
    return getattr(torch.backends.cudnn, name)
