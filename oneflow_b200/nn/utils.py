"""``flow.nn.utils``: clip_grad_norm_/clip_grad_value_ that understand global tensors (the norm of a
partial-sum or split gradient is taken over the whole logical tensor), plus torch's helpers.
Reference: python/oneflow/nn/utils/clip_grad.py, fused_clip_grad.cu."""
from __future__ import annotations

import math

import torch
from torch.nn.utils import (parameters_to_vector, vector_to_parameters, weight_norm, remove_weight_norm,  # noqa: F401
                            rnn, prune, spectral_norm, clip_grad_value_ as _torch_clip_value)

from ..framework import global_tensor as GT


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
        total = torch.stack(norms).max()
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
