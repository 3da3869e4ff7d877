"""Additions to ``nn.Module``: ``to_global(placement, sbp)`` / ``to_local()`` convert every parameter and
buffer (reference: python/oneflow/nn/modules/module.py:1586-1597), ``make_contiguous_params_group``
places all parameters (and their gradients) in flat buffers (``:1804``)."""
from __future__ import annotations

import torch

from .. import sbp as S
from ..framework import global_tensor as GT


def module_to_global(self, placement=None, sbp=None):
    if placement is None:
        raise ValueError("to_global needs a placement")
    for m in self.modules():
        for name, p in list(m._parameters.items()):
            if p is None:
                continue
            g = GT.to_global(p.detach(), placement, sbp if sbp is not None else S.broadcast)
            newp = torch.nn.Parameter(g, requires_grad=p.requires_grad)
            m._parameters[name] = newp
        for name, b in list(m._buffers.items()):
            if b is None:
                continue
            m._buffers[name] = GT.to_global(b, placement, sbp if sbp is not None else S.broadcast)
    return self


def module_to_local(self):
    for m in self.modules():
        for name, p in list(m._parameters.items()):
            if p is not None and isinstance(p, GT.GlobalTensor):
                m._parameters[name] = torch.nn.Parameter(p._local.detach(), requires_grad=p.requires_grad)
        for name, b in list(m._buffers.items()):
            if b is not None and isinstance(b, GT.GlobalTensor):
                m._buffers[name] = b._local
    return self


def make_contiguous_params_group(self):
    """Moves all (local) parameters into one flat buffer per dtype; returns {dtype: flat tensor}."""
    by_dtype = {}
    for p in self.parameters():
        if isinstance(p, GT.GlobalTensor):
            continue
        by_dtype.setdefault((p.dtype, p.device), []).append(p)
    flats = {}
    for (dt, dev), ps in by_dtype.items():
        sizes = [(p.numel() + 63) // 64 * 64 for p in ps]
        flat = torch.zeros(sum(sizes), dtype=dt, device=dev)
        off = 0
        for p, n in zip(ps, sizes):
            view = flat[off:off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            off += n
        flats[dt] = flat
    self._contiguous_params = flats
    return flats


def install():
    M = torch.nn.Module
    if getattr(M, "_ofb_patched", False):
        return
    M.to_global = module_to_global
    M.to_local = module_to_local
    M.make_contiguous_params_group = make_contiguous_params_group
    M._ofb_patched = True
