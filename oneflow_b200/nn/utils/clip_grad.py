"""``oneflow.nn.utils.clip_grad`` import path (reference: python/oneflow/nn/utils/clip_grad.py)."""
from . import clip_grad_norm_, clip_grad_value_  # noqa: F401
