"""``flow.nn.utils``: clip_grad_norm_/clip_grad_value_ that understand global tensors (the norm of a
partial-sum or split gradient is taken over the whole logical tensor), plus torch's helpers.
Reference: python/oneflow/nn/utils/clip_grad.py, fused_clip_grad.cu."""
from __future__ import annotations

import math

import torch
from torch.nn.utils import (parameters_to_vector, vector_to_parameters, weight_norm, remove_weight_norm,  # noqa: F401
                            rnn, prune, spectral_norm, clip_grad_value_ as _torch_clip_value)

from ...framework import global_tensor as GT


def clip_grad_norm_(parameters, max_norm, norm_type=2.0, error_if_nonfinite=False, fused=False):
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return torch.tensor(0.0)
    norm_type = float(norm_type)
    locals_ = [p for p in params if not isinstance(p, GT.GlobalTensor)]
    if fused and locals_ and all(p.is_cuda for p in locals_) and norm_type == 2.0 and len(locals_) == len(params):
        from ..ops import kernels as K
        sq = K.multi_tensor_sqsum([p.grad.contiguous() for p in params])
        factor, found, total = K.clip_factor(sq, float(max_norm))
        for p in params:
            p.grad.mul_(factor)
        return total[0]
    norms = []
    for p in params:
        g = p.grad
        if isinstance(g, GT.GlobalTensor):
            # a P gradient must be summed before its norm means anything: box to B once and keep it
            if any(s.kind == "P" for s in g.sbp):
                g = GT.rebox(g, tuple(GT.B if s.kind == "P" else s for s in g.sbp))
                p.grad = g
            n = torch.linalg.vector_norm(g.detach(), norm_type)
            n = GT.rebox(n, (GT.B,) * n.placement.ndim)._local if isinstance(n, GT.GlobalTensor) else n
            norms.append(n.float().cpu() if n.numel() else torch.zeros(()))
        else:
            norms.append(torch.linalg.vector_norm(g.detach(), norm_type).float().cpu())
    if math.isinf(norm_type):
        total = torch.stack(norms).max() if norm_type > 0 else torch.stack(norms).min()
    else:
        total = torch.linalg.vector_norm(torch.stack(norms), norm_type)
    if error_if_nonfinite and not torch.isfinite(total):
        raise RuntimeError("The total norm of gradients is non-finite")
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0).item()
    if coef < 1.0:
        for p in params:
            p.grad.mul_(coef)
    return total


def clip_grad_value_(parameters, clip_value):
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    for p in parameters:
        if p.grad is not None:
            p.grad.clamp_(-clip_value, clip_value)


from torch.nn.utils import skip_init  # noqa: E402,F401


def numel_in_bucket(tensor):
    """Elements a tensor occupies in a grouped buffer: its size rounded up to 512 bytes, so every member starts on
    an address vector loads and TMA accept (reference: python/oneflow/nn/utils/parameters_grouping.py:27-39)."""
    if not tensor.is_floating_point():
        raise TypeError("parameter grouping takes floating-point tensors only")
    unit = 512 // tensor.element_size()
    return -(-tensor.numel() // unit) * unit


class ContiguousParamsGroup:
    """Moves groups of parameters (a list of lists; a flat list is one group) and their gradients into contiguous flat
    buffers, one per (group, dtype, device): every parameter becomes a view into its buffer and its ``.grad`` a view
    into the buffer's gradient, so an optimizer or a gradient all-reduce can run once over ``grouped_parameters`` /
    ``grouped_parameters_grad`` instead of once per tensor
    (reference: python/oneflow/nn/utils/parameters_grouping.py:42-302).  Parameters without ``requires_grad`` are left
    alone.  Parameters that already live in a buffer made by an earlier group are regrouped on that buffer when
    ``group_on_current_buffer``: runs of neighbours of one group inside it become one slice."""

    def __init__(self, params_group_list, group_on_current_buffer=True):
        groups = list(params_group_list)
        if groups and isinstance(groups[0], torch.Tensor):
            groups = [groups]
        self.params_group_list = [[p for p in g if p.requires_grad] for g in groups]
        self.group_on_current_buffer = group_on_current_buffer
        self.grouped_tensors, self.grouped_grads = [], []
        have_buffer = any(hasattr(p, "_ref_tensor") for g in self.params_group_list for p in g)
        if group_on_current_buffer and have_buffer:
            self._group_on_current_buffer()
        else:
            self._group_on_new_buffer()

    def _group_globals(self):
        """Global parameters: one flat buffer of this rank's shards per (group, dtype, placement, sbp); each parameter's
        local shard and local gradient become views into it, and the buffer is presented as a global tensor of the
        same placement and sbp (its logical extent is the local extent times the number of shards when split)."""
        from ...framework import global_tensor as GT
        todo = {}
        for idx, params in enumerate(self.params_group_list):
            for p in params:
                if isinstance(p, GT.GlobalTensor):
                    todo.setdefault((p.dtype, p.placement, tuple(p.sbp), idx), []).append(p)
        for (dt, pl, nd, idx), ps in todo.items():
            total = sum(numel_in_bucket(p._local) for p in ps)
            flat = torch.zeros(total, dtype=dt, device=ps[0]._local.device)
            gflat = torch.zeros(total, dtype=dt, device=ps[0]._local.device)
            at = 0
            for p in ps:
                n = p._local.numel()
                flat[at:at + n] = p._local.detach().reshape(-1)
                p._local.data = flat[at:at + n].view(p._local.shape)
                p._ofb_grad_view = gflat[at:at + n].view(p._local.shape)
                at += numel_in_bucket(p._local)
            shards = 1
            for axis, s in enumerate(nd):
                if s.kind == "S":
                    shards *= pl.hierarchy[axis]
            flat_nd = tuple(GT.S.split(0) if s.kind == "S" else s for s in nd)
            self.grouped_tensors.append(GT.wrap(flat, (total * shards,), pl, flat_nd))
            self.grouped_grads.append(GT.wrap(gflat, (total * shards,), pl, flat_nd))
        self.params_group_list = [[p for p in params if not isinstance(p, GT.GlobalTensor)] for params in self.params_group_list]

    def _group_on_new_buffer(self):
        self._group_globals()
        sizes = {}
        for idx, params in enumerate(self.params_group_list):
            for p in params:
                key = (p.dtype, p.device, idx)
                sizes[key] = sizes.get(key, 0) + numel_in_bucket(p)
        buffers, cursor = {}, {}
        for key, size in sizes.items():
            buf = torch.zeros(size, dtype=key[0], device=key[1])
            buf.grad = torch.zeros(size, dtype=key[0], device=key[1])
            buffers[key], cursor[key] = buf, 0
            self.grouped_tensors.append(buf)
            self.grouped_grads.append(buf.grad)
        for idx, params in enumerate(self.params_group_list):
            for p in params:
                key = (p.dtype, p.device, idx)
                buf, at, n = buffers[key], cursor[key], p.numel()
                buf[at:at + n] = p.data.reshape(-1)
                old_grad = p.grad
                p.data = buf[at:at + n].view(p.shape)
                p.grad = buf.grad[at:at + n].view(p.shape)
                if old_grad is not None:
                    p.grad.copy_(old_grad)
                p._ref_tensor, p._ref_index = buf, at
                cursor[key] = at + numel_in_bucket(p)

    def _group_on_current_buffer(self):
        for params in self.params_group_list:
            by_buf, alone = {}, []
            for p in params:
                if not hasattr(p, "_ref_tensor"):
                    alone.append(p)                       # never grouped before: stays on its own, after the buffers
                    continue
                by_buf.setdefault(id(p._ref_tensor), []).append(p)
            for members in by_buf.values():
                members.sort(key=lambda q: q._ref_index)
                buf = members[0]._ref_tensor
                lo = members[0]._ref_index
                hi = lo + numel_in_bucket(members[0])
                for q in members[1:]:
                    if q._ref_index == hi:                # direct neighbour: extend the run
                        hi += numel_in_bucket(q)
                        continue
                    self.grouped_tensors.append(buf[lo:hi])
                    self.grouped_grads.append(buf.grad[lo:hi])
                    lo, hi = q._ref_index, q._ref_index + numel_in_bucket(q)
                self.grouped_tensors.append(buf[lo:hi])
                self.grouped_grads.append(buf.grad[lo:hi])
            for p in alone:
                self.grouped_tensors.append(p)
                self.grouped_grads.append(p.grad)

    @property
    def grouped_grads(self):
        return self._grouped_grads

    @grouped_grads.setter
    def grouped_grads(self, v):
        self._grouped_grads = v

    @property
    def grouped_parameters(self):
        return self.grouped_tensors

    @property
    def grouped_parameters_grad(self):
        return self.grouped_grads
