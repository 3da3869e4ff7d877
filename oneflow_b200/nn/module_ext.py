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
    """Moves all local parameters (and their gradients) into flat buffers, one per dtype and device, and keeps the
    grouping as ``self.cpg`` (a ``nn.utils.ContiguousParamsGroup``): optimizers and gradient collectives can then work
    on ``self.cpg.grouped_parameters`` / ``grouped_grads`` (reference: python/oneflow/nn/modules/module.py,
    ``make_contiguous_params_group``)."""
    from .utils import ContiguousParamsGroup
    params = [p for p in self.parameters() if not isinstance(p, GT.GlobalTensor)]
    self.cpg = ContiguousParamsGroup([params], group_on_current_buffer=False)
    return self.cpg


def install():
    M = torch.nn.Module
    if getattr(M, "_ofb_patched", False):
        return
    M.to_global = module_to_global
    M.to_local = module_to_local
    M.make_contiguous_params_group = make_contiguous_params_group
    _load = M.load_state_dict

    def load_state_dict(self, state_dict, strict=True, assign=False):
        """``load_state_dict`` that also takes numpy arrays as values (the reference converts them)."""
        import numpy as np
        if any(isinstance(v, np.ndarray) for v in state_dict.values()):
            state_dict = type(state_dict)((k, torch.from_numpy(np.ascontiguousarray(v)) if isinstance(v, np.ndarray) else v)
                                          for k, v in state_dict.items())
        return _load(self, state_dict, strict=strict, assign=assign)
    M.load_state_dict = load_state_dict

    _state = M.state_dict

    def state_dict(self, *args, destination=None, prefix="", keep_vars=True):
        """``state_dict`` whose values are the parameters and buffers themselves (the reference never detaches
        them: python/oneflow/nn/modules/module.py, ``_save_to_state_dict``); ``keep_vars=False`` detaches."""
        return _state(self, *args, destination=destination, prefix=prefix, keep_vars=keep_vars)
    M.state_dict = state_dict

    def _tuple_hook(hook):
        # backward hooks see ``TensorTuple`` arguments; a returned gradient is cast to the dtype it replaces
        from oneflow._oneflow_internal import TensorTuple

        def wrapped(module, grad_input, grad_output):
            res = hook(module, TensorTuple(grad_input), TensorTuple(grad_output))
            if res is None:
                return None
            res = tuple(res) if isinstance(res, (tuple, list)) else (res,)
            return tuple(r.to(dtype=g.dtype, device=g.device) if isinstance(r, torch.Tensor) and g is not None else r
                         for r, g in zip(res, grad_input))
        wrapped.__wrapped__ = hook
        return wrapped

    _full, _legacy = M.register_full_backward_hook, M.register_backward_hook

    def register_full_backward_hook(self, hook, prepend=False):
        return _full(self, _tuple_hook(hook), prepend=prepend)

    def register_backward_hook(self, hook):
        return _legacy(self, _tuple_hook(hook))
    register_full_backward_hook.__doc__, register_backward_hook.__doc__ = _full.__doc__, _legacy.__doc__
    M.register_full_backward_hook = register_full_backward_hook
    M.register_backward_hook = register_backward_hook

    def _global_batch_first(cls):
        # The library's RNN kernels turn a batch-first result around with an in-place ``transpose_``; a global
        # tensor's logical shape is fixed at construction, so for global inputs the two transposes are done here,
        # out of place, and the kernel runs sequence-first.
        fwd = cls.forward

        def forward(self, input, hx=None):
            if isinstance(input, GT.GlobalTensor) and self.batch_first and input.dim() == 3:
                self.batch_first = False
                try:
                    out, h = fwd(self, input.transpose(0, 1).contiguous(), hx)
                finally:
                    self.batch_first = True
                return out.transpose(0, 1), h
            return fwd(self, input, hx)
        forward.__doc__ = fwd.__doc__
        cls.forward = forward
    for _cls in (torch.nn.RNN, torch.nn.LSTM, torch.nn.GRU):
        _global_batch_first(_cls)
    M._ofb_patched = True
