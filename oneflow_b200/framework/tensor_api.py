"""Tensor construction and the methods the flow API adds to tensors.

Local tensors ARE ``torch.Tensor`` objects (``flow.Tensor`` answers ``isinstance`` for them and builds them);
global tensors are ``GlobalTensor`` wrappers. ``to_global`` / ``to_local`` / ``is_global`` / ``placement`` /
``sbp`` are attached to ``torch.Tensor`` so that both kinds share one surface
(reference: python/oneflow/framework/tensor.py, nn/modules/global_cast.py:40-95)."""
from __future__ import annotations

import numpy as np
import torch

from .. import sbp as S
from . import global_tensor as GT
from .placement import placement as Placement


class _TensorMeta(type):
    def __instancecheck__(cls, obj):
        return isinstance(obj, torch.Tensor)

    def __call__(cls, *args, **kwargs):
        return torch.Tensor(*args, **kwargs)


class Tensor(metaclass=_TensorMeta):
    """``flow.Tensor``: ``isinstance(x, flow.Tensor)`` holds for every local and global tensor and
    ``flow.Tensor(2, 3)`` builds a local tensor. Instances of this class itself only exist inside
    checkpoints being written, where they carry the tensor state under the class path ``oneflow.Tensor``."""
    _pickle_state = None

    def __getstate__(self):
        return self._pickle_state


Tensor.__module__ = "oneflow"


def _globalize(t, placement, sbp, requires_grad=False):
    if placement is None:
        return t.requires_grad_(requires_grad) if requires_grad else t
    nd = S.normalize(sbp if sbp is not None else S.broadcast, placement.ndim)
    allb = (S.broadcast,) * placement.ndim
    g = GT.to_global(t, placement, allb)
    g = GT.to_global(g, placement, nd)
    if requires_grad:
        g.requires_grad_(True)
    return g


def tensor(data, dtype=None, device=None, placement=None, sbp=None, requires_grad=False, pin_memory=False):
    if isinstance(data, GT.GlobalTensor):
        out = data.detach().clone()
        if dtype is not None:
            out = out.to(dtype)
        return out.requires_grad_(requires_grad) if requires_grad else out
    if isinstance(data, torch.Tensor):
        t = data.detach().clone()
        if dtype is not None:
            t = t.to(dtype)
    else:
        if isinstance(data, np.ndarray) and data.dtype == np.float64 and dtype is None:
            dtype = torch.float32 if False else None
        t = torch.tensor(data, dtype=dtype)
    if placement is not None:
        return _globalize(t, placement, sbp, requires_grad)
    if device is not None:
        t = t.to(device)
    if pin_memory:
        t = t.pin_memory()
    return t.requires_grad_(requires_grad) if requires_grad else t


def _factory(torch_fn):
    def fn(*args, placement=None, sbp=None, device=None, requires_grad=False, **kwargs):
        if placement is None:
            if device is not None:
                kwargs["device"] = device
            t = torch_fn(*args, **kwargs)
            return t.requires_grad_(requires_grad) if requires_grad else t
        # global: every rank draws the logical tensor (first rank's values win along broadcast axes)
        kwargs["device"] = placement.device() if placement.contains(GT._rank()) else "cpu"
        t = torch_fn(*args, **kwargs)
        return _globalize(t, placement, sbp, requires_grad)
    fn.__name__ = torch_fn.__name__
    fn.__doc__ = f"flow.{torch_fn.__name__}: torch.{torch_fn.__name__} plus ``placement=`` / ``sbp=`` for global tensors."
    return fn


zeros, ones, empty, full = (_factory(f) for f in (torch.zeros, torch.ones, torch.empty, torch.full))
randn, rand, randint, randperm = (_factory(f) for f in (torch.randn, torch.rand, torch.randint, torch.randperm))
arange, eye, linspace = (_factory(f) for f in (torch.arange, torch.eye, torch.linspace))


def from_numpy(a):
    return torch.from_numpy(a)


def install_tensor_methods():
    T = torch.Tensor
    if getattr(T, "_ofb_patched", False):
        return
    T.to_global = lambda self, placement=None, sbp=None, **kw: GT.to_global(self, placement, sbp, **kw)
    T.to_local = lambda self, copy=False: GT.to_local(self, copy=copy)
    T.is_global = property(lambda self: isinstance(self, GT.GlobalTensor))
    T.is_local = property(lambda self: not isinstance(self, GT.GlobalTensor))

    def _placement(self):
        raise RuntimeError("local tensor has no placement; call to_global first")

    def _sbp(self):
        raise RuntimeError("local tensor has no sbp; call to_global first")
    T.placement = property(_placement)
    T.sbp = property(_sbp)
    T.global_id = lambda self: id(self)
    T._ofb_patched = True
