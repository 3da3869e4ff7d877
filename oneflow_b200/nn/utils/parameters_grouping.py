"""``oneflow.nn.utils.parameters_grouping`` import path (reference: python/oneflow/nn/utils/parameters_grouping.py)."""
from . import ContiguousParamsGroup, numel_in_bucket  # noqa: F401
