"""``flow.utils.global_view``: apply to_global / to_local over pytrees (state dicts, nested containers) and
the ``global_mode`` context (reference: python/oneflow/utils/global_view/*.py)."""
import contextlib

import torch
from torch.utils import _pytree as pytree

from ...framework import global_tensor as GT

_MODE = []


def to_global(obj, placement=None, sbp=None, **kwargs):
    return pytree.tree_map(lambda x: GT.to_global(x, placement, sbp, **kwargs) if isinstance(x, torch.Tensor) else x, obj)


def to_local(obj, copy=False):
    return pytree.tree_map(lambda x: GT.to_local(x, copy=copy) if isinstance(x, torch.Tensor) else x, obj)


@contextlib.contextmanager
def global_mode(enabled, placement=None, sbp=None):
    """Within the context, current_global_mode() reports the placement/sbp new tensors should take."""
    _MODE.append((enabled, placement, sbp))
    try:
        yield
    finally:
        _MODE.pop()


class current_global_mode:
    def __init__(self):
        self.is_enabled, self.placement, self.sbp = _MODE[-1] if _MODE else (False, None, None)
