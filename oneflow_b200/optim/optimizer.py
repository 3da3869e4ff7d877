"""Optimizers with the reference's constructor surface (python/oneflow/nn/optimizer/*.py): SGD, Adam,
AdamW, Adagrad, Adadelta, RMSprop, LAMB, LBFGS. Param-group options ``clip_grad_max_norm`` /
``clip_grad_norm_type`` (applied by ``clip_grad()``, which nn.Graph calls before every step) and
``fused=True`` (local CUDA parameters are updated by the multi-tensor kernels of csrc/kernels/optim.cu in
one launch per 48 tensors). Global-tensor parameters go through the SBP dispatch: partial-sum gradients
are boxed to the parameter's layout by the update ops themselves.

Update maths follow oneflow/user/kernels/model_update_kernel_util.h:25-140 (see csrc/kernels/optim.cu)."""
from __future__ import annotations

import math

import torch

from ..framework import global_tensor as GT


def _local(t):
    return t._local if isinstance(t, GT.GlobalTensor) else t


class _ClipMixin:
    def clip_grad(self, error_if_nonfinite=False):
        """Global-norm clipping per param group carrying ``clip_grad_max_norm``."""
        for g in self.param_groups:
            mx = g.get("clip_grad_max_norm")
            if mx is None:
                continue
            nt = float(g.get("clip_grad_norm_type", 2.0))
            from ..nn.utils import clip_grad_norm_
            clip_grad_norm_(g["params"], mx, nt, error_if_nonfinite)

    def _fusable(self):
        ps = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        return bool(ps) and all((not isinstance(p, GT.GlobalTensor)) and p.is_cuda and p.dtype == torch.float32
                                and p.is_contiguous() and p.grad.is_contiguous() and p.data_ptr() % 16 == 0
                                and p.grad.data_ptr() % 16 == 0 for p in ps)


class SGD(_ClipMixin, torch.optim.SGD):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, maximize=False,
                 contiguous_params=False, fused=False):
        self._fused = fused
        super().__init__(params, lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                         nesterov=nesterov, maximize=maximize)

    @torch.no_grad()
    def step(self, closure=None):
        if not (self._fused and self._fusable()):
            return super().step(closure)
        from ..ops import kernels as K
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.grad is not None]
            ms = None
            if g["momentum"] != 0:
                ms = []
                for p in ps:
                    st = self.state[p]
                    if "momentum_buffer" not in st or st["momentum_buffer"] is None:
                        st["momentum_buffer"] = torch.zeros_like(p)
                        first = True
                    ms.append(st["momentum_buffer"])
            # torch semantics: coupled weight decay (l2), first momentum step copies the gradient
            K.multi_tensor_sgd([p.grad for p in ps], [p.data for p in ps], None, ms, lr=g["lr"], momentum=g["momentum"],
                               dampening=g["dampening"], nesterov=g["nesterov"], maximize=g["maximize"],
                               l2=g["weight_decay"])
        return loss


class _AdamBase(_ClipMixin):
    def _fused_step(self, decoupled):
        from ..ops import kernels as K
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.grad is not None]
            if not ps:
                continue
            ms, vs = [], []
            for p in ps:
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"] = torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
            step = int(self.state[ps[0]]["step"].item())
            b1, b2 = g["betas"]
            K.multi_tensor_adamw([p.grad for p in ps], [p.data for p in ps], None, ms, vs, lr=g["lr"], beta1=b1, beta2=b2,
                                 eps=g["eps"], weight_decay=g["weight_decay"] if decoupled else 0.0,
                                 l2=0.0 if decoupled else g["weight_decay"], step=step,
                                 bias_correction=getattr(self, "_bias_correction", True))


class Adam(_AdamBase, torch.optim.Adam):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False,
                 do_bias_correction=True, contiguous_params=False, fused=False):
        self._fused, self._bias_correction = fused, do_bias_correction
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)

    @torch.no_grad()
    def step(self, closure=None):
        if self._fused and self._fusable() and not any(g["amsgrad"] for g in self.param_groups):
            loss = closure() if closure is not None else None
            self._fused_step(decoupled=False)
            return loss
        return super().step(closure)


class AdamW(_AdamBase, torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False,
                 do_bias_correction=True, contiguous_params=False, fused=False):
        self._fused, self._bias_correction = fused, do_bias_correction
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)

    @torch.no_grad()
    def step(self, closure=None):
        if self._fused and self._fusable() and not any(g["amsgrad"] for g in self.param_groups):
            loss = closure() if closure is not None else None
            self._fused_step(decoupled=True)
            return loss
        return super().step(closure)


class Adagrad(_ClipMixin, torch.optim.Adagrad):
    def __init__(self, params, lr=1e-3, lr_decay=0.0, weight_decay=0.0, initial_accumulator_value=0.0, eps=1e-10,
                 contiguous_params=False):
        super().__init__(params, lr=lr, lr_decay=lr_decay, weight_decay=weight_decay,
                         initial_accumulator_value=initial_accumulator_value, eps=eps)


class Adadelta(_ClipMixin, torch.optim.Adadelta):
    def __init__(self, params, lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0, maximize=False, contiguous_params=False):
        super().__init__(params, lr=lr, rho=rho, eps=eps, weight_decay=weight_decay, maximize=maximize)


class RMSprop(_ClipMixin, torch.optim.RMSprop):
    def __init__(self, params, lr=1e-3, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False,
                 contiguous_params=False):
        super().__init__(params, lr=lr, alpha=alpha, eps=eps, weight_decay=weight_decay, momentum=momentum, centered=centered)


class LBFGS(_ClipMixin, torch.optim.LBFGS):
    pass


class LAMB(_ClipMixin, torch.optim.Optimizer):
    """Layer-wise adaptive moments (reference: python/oneflow/nn/optimizer/lamb.py; kernel lamb_update)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.0, adam_w_mode=True,
                 do_bias_correction=True, amsgrad=False, contiguous_params=False):
        if amsgrad:
            raise RuntimeError("LAMB does not support AMSGrad")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adam_w_mode=adam_w_mode,
                                      do_bias_correction=do_bias_correction))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                grad = p.grad
                if not g["adam_w_mode"] and g["weight_decay"]:
                    grad = grad + g["weight_decay"] * p
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
                bc1 = 1 - b1 ** st["step"] if g["do_bias_correction"] else 1.0
                bc2 = 1 - b2 ** st["step"] if g["do_bias_correction"] else 1.0
                upd = (m / bc1) / ((v / bc2).sqrt() + g["eps"])
                if g["adam_w_mode"] and g["weight_decay"]:
                    upd = upd + g["weight_decay"] * p
                wn, un = float(torch.linalg.vector_norm(p)), float(torch.linalg.vector_norm(upd))
                trust = wn / un if wn > 0 and un > 0 else 1.0
                p.add_(upd, alpha=-g["lr"] * trust)
        return loss
