"""Eager activation checkpointing (reference: python/oneflow/utils/checkpoint.py, saved-tensor hooks)."""
from torch.utils.checkpoint import checkpoint as _ckpt


def checkpoint(function, *args, use_reentrant=False, **kwargs):
    return _ckpt(function, *args, use_reentrant=use_reentrant, **kwargs)
