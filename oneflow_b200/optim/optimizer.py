"""Optimizers with the reference's constructor surface and update rules (python/oneflow/nn/optimizer/*.py;
oneflow/user/kernels/model_update_kernel_util.h:25-140): SGD, Adam, AdamW, Adagrad, Adadelta, RMSprop, LAMB, Ftrl,
LBFGS.  Every hyper-parameter — ``do_bias_correction``, ``amsgrad``, ``clip_grad_max_norm`` / ``clip_grad_norm_type``
included — lives in the param group, so ``state_dict()`` / ``load_state_dict()`` carry it and a freshly built optimizer
continues exactly where the saved one stopped.  ``clip_grad()`` applies the per-group norm clipping (``nn.Graph``
calls it before every step).  ``fused=True`` updates local CUDA fp32 parameters with the multi-tensor kernels of
csrc/kernels/optim.cu, one launch per 48 tensors.  Global-tensor parameters go through the SBP dispatch: the update
ops box partial-sum gradients to the parameter's layout.

Where the rules differ from PyTorch's optimizers of the same name (and why these are not subclasses of them):
SGD damps the first momentum step too and allows Nesterov with dampening; RMSprop puts epsilon under the square root
and folds the learning rate into its momentum buffer; Adam / AdamW / LAMB can run without bias correction.
"""
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

    def support_sparse(self):
        return False

    def _fusable(self):
        ps = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        return bool(ps) and all((not isinstance(p, GT.GlobalTensor)) and p.is_cuda and p.dtype == torch.float32
                                and p.is_contiguous() and p.grad.is_contiguous() and p.data_ptr() % 16 == 0
                                and p.grad.data_ptr() % 16 == 0 for p in ps)


def _lr(g):
    """Learning rate of a group.  (The group option ``lr_scale`` is a graph-mode feature: ``nn.Graph`` multiplies the
    rate by it around its optimizer step; eager steps ignore it, as the reference does.)"""
    return g["lr"]


class _Base(_ClipMixin, torch.optim.Optimizer):
    """Shared step loop: ``_update(p, grad, state, group)`` per parameter with a gradient; ``state["step"]`` counts from 1."""

    def __init__(self, params, defaults, contiguous_params=False, fused=False):
        self._fused = bool(fused)
        self._contiguous = bool(contiguous_params)
        super().__init__(params, defaults)

    def _init_state(self, p, state, group):
        pass

    def _fused_step(self):
        return False

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._fused and self._fusable() and self._fused_step():
            return loss
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if "step" not in state:
                    state["step"] = 0
                    self._init_state(p, state, group)
                state["step"] = int(state["step"]) + 1
                self._update(p, p.grad, state, group)
        return loss


class SGD(_Base):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, maximize=False,
                 contiguous_params=False, fused=False):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if momentum < 0.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay: {weight_decay}")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov, maximize=maximize), contiguous_params, fused)

    def _update(self, p, grad, state, g):
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        if g["momentum"] > 0:
            buf = state.get("momentum_buf")
            if buf is None:
                buf = state["momentum_buf"] = torch.zeros_like(p)
            buf.mul_(g["momentum"]).add_(grad, alpha=1 - g["dampening"])
            grad = grad + g["momentum"] * buf if g["nesterov"] else buf
            p.add_(grad, alpha=_lr(g) if g["maximize"] else -_lr(g))
        else:
            p.add_(grad, alpha=-_lr(g))

    def _fused_step(self):
        from ..ops import kernels as K
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.grad is not None]
            if not ps:
                continue
            ms = None
            if g["momentum"] > 0:
                ms = []
                for p in ps:
                    st = self.state[p]
                    if st.get("momentum_buf") is None:
                        st["momentum_buf"] = torch.zeros_like(p)
                    ms.append(st["momentum_buf"])
            for p in ps:
                self.state[p]["step"] = int(self.state[p].get("step", 0)) + 1
            K.multi_tensor_sgd([p.grad for p in ps], [p.data for p in ps], None, ms, lr=_lr(g), momentum=g["momentum"],
                               dampening=g["dampening"], nesterov=g["nesterov"],
                               maximize=g["maximize"] and g["momentum"] > 0, l2=g["weight_decay"])
        return True


class _AdamFamily(_Base):
    decoupled = False

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False, do_bias_correction=True,
                 contiguous_params=False, fused=False):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if eps < 0.0:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid beta parameters: {betas}")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                                      do_bias_correction=do_bias_correction), contiguous_params, fused)

    def _init_state(self, p, state, g):
        state["exp_avg"] = torch.zeros_like(p)
        state["exp_avg_sq"] = torch.zeros_like(p)
        if g["amsgrad"]:
            state["max_exp_avg_sq"] = torch.zeros_like(p)

    def _update(self, p, grad, state, g):
        b1, b2 = g["betas"]
        if not self.decoupled and g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        m, v = state["exp_avg"], state["exp_avg_sq"]
        m.mul_(b1).add_(grad, alpha=1 - b1)
        v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
        bc1 = 1 - b1 ** state["step"] if g["do_bias_correction"] else 1.0
        bc2 = 1 - b2 ** state["step"] if g["do_bias_correction"] else 1.0
        if g["amsgrad"]:
            mx = state.get("max_exp_avg_sq")
            if mx is None:
                mx = state["max_exp_avg_sq"] = torch.zeros_like(p)
            torch.maximum(mx, v, out=mx)
            denom = mx.sqrt() / math.sqrt(bc2) + g["eps"]
        else:
            denom = v.sqrt() / math.sqrt(bc2) + g["eps"]
        if self.decoupled and g["weight_decay"]:
            p.mul_(1 - _lr(g) * g["weight_decay"])
        p.addcdiv_(m, denom, value=-_lr(g) / bc1)

    def _fused_step(self):
        if any(g["amsgrad"] for g in self.param_groups):
            return False
        from ..ops import kernels as K
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.grad is not None]
            if not ps:
                continue
            ms, vs = [], []
            for p in ps:
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"] = 0
                    self._init_state(p, st, g)
                st["step"] = int(st["step"]) + 1
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
            b1, b2 = g["betas"]
            K.multi_tensor_adamw([p.grad for p in ps], [p.data for p in ps], None, ms, vs, lr=_lr(g), beta1=b1, beta2=b2,
                                 eps=g["eps"], weight_decay=g["weight_decay"] if self.decoupled else 0.0,
                                 l2=0.0 if self.decoupled else g["weight_decay"], step=int(self.state[ps[0]]["step"]),
                                 bias_correction=g["do_bias_correction"])
        return True


class Adam(_AdamFamily):
    """Adam with the weight decay added to the gradient (L2)."""


class AdamW(_AdamFamily):
    """Adam with decoupled weight decay."""
    decoupled = True


class Adagrad(_Base):
    def __init__(self, params, lr=1e-3, lr_decay=0.0, weight_decay=0.0, initial_accumulator_value=0.0, eps=1e-10,
                 contiguous_params=False):
        super().__init__(params, dict(lr=lr, lr_decay=lr_decay, weight_decay=weight_decay,
                                      initial_accumulator_value=initial_accumulator_value, eps=eps), contiguous_params)

    def _init_state(self, p, state, g):
        state["sum"] = torch.full_like(p, g["initial_accumulator_value"])

    def _update(self, p, grad, state, g):
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        s = state["sum"]
        s.addcmul_(grad, grad)
        lr = _lr(g) / (1 + (state["step"] - 1) * g["lr_decay"])
        p.addcdiv_(grad, s.sqrt() + g["eps"], value=-lr)


class Adadelta(_Base):
    def __init__(self, params, lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0, maximize=False, contiguous_params=False):
        super().__init__(params, dict(lr=lr, rho=rho, eps=eps, weight_decay=weight_decay, maximize=maximize), contiguous_params)

    def _init_state(self, p, state, g):
        state["square_avg"] = torch.zeros_like(p)
        state["acc_delta"] = torch.zeros_like(p)

    def _update(self, p, grad, state, g):
        if g["maximize"]:
            grad = -grad
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        sq, acc, rho, eps = state["square_avg"], state["acc_delta"], g["rho"], g["eps"]
        sq.mul_(rho).addcmul_(grad, grad, value=1 - rho)
        delta = (acc + eps).sqrt_().div_((sq + eps).sqrt_()).mul_(grad)
        acc.mul_(rho).addcmul_(delta, delta, value=1 - rho)
        p.add_(delta, alpha=-_lr(g))


class RMSprop(_Base):
    """``r = alpha r + (1 - alpha) g^2``; centered also tracks ``ḡ = alpha ḡ + (1 - alpha) g`` and uses ``r - ḡ^2``;
    ``v = momentum v + lr g / sqrt(r + eps)``; ``p -= v``."""

    def __init__(self, params, lr=1e-3, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False,
                 contiguous_params=False):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if alpha < 0.0:
            raise ValueError(f"Invalid alpha value: {alpha}")
        if eps < 0.0:
            raise ValueError(f"Invalid epsilon value: {eps}")
        super().__init__(params, dict(lr=lr, alpha=alpha, eps=eps, weight_decay=weight_decay, momentum=momentum,
                                      centered=centered), contiguous_params)

    def _init_state(self, p, state, g):
        state["square_avg"] = torch.zeros_like(p)
        state["momentum_buffer"] = torch.zeros_like(p)
        if g["centered"]:
            state["grad_avg"] = torch.zeros_like(p)

    def _update(self, p, grad, state, g):
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        a = g["alpha"]
        r = state["square_avg"]
        r.mul_(a).addcmul_(grad, grad, value=1 - a)
        if g["centered"]:
            gm = state.get("grad_avg")
            if gm is None:
                gm = state["grad_avg"] = torch.zeros_like(p)
            gm.mul_(a).add_(grad, alpha=1 - a)
            denom = (r - gm * gm + g["eps"]).sqrt_()
        else:
            denom = (r + g["eps"]).sqrt_()
        v = state["momentum_buffer"]
        v.mul_(g["momentum"]).addcdiv_(grad, denom, value=_lr(g))
        p.sub_(v)


class LAMB(_Base):
    """Layer-wise adaptive moments: an Adam direction per tensor, scaled by ``||w|| / ||direction||``
    (reference: python/oneflow/nn/optimizer/lamb.py; kernel lamb_update)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.0, adam_w_mode=True,
                 do_bias_correction=True, amsgrad=False, contiguous_params=False):
        if amsgrad:
            raise RuntimeError("LAMB does not support AMSGrad")
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adam_w_mode=adam_w_mode,
                                      do_bias_correction=do_bias_correction, amsgrad=False), contiguous_params)

    def _init_state(self, p, state, g):
        state["exp_avg"] = torch.zeros_like(p)
        state["exp_avg_sq"] = torch.zeros_like(p)

    def _update(self, p, grad, state, g):
        b1, b2 = g["betas"]
        if not g["adam_w_mode"] and g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        m, v = state["exp_avg"], state["exp_avg_sq"]
        m.mul_(b1).add_(grad, alpha=1 - b1)
        v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
        bc1 = 1 - b1 ** state["step"] if g["do_bias_correction"] else 1.0
        bc2 = 1 - b2 ** state["step"] if g["do_bias_correction"] else 1.0
        direction = (m / bc1) / (v.sqrt() / math.sqrt(bc2) + g["eps"])
        wn, dn = float(torch.linalg.vector_norm(p)), float(torch.linalg.vector_norm(direction))
        trust = wn / dn if wn > 0 and dn > 0 else 1.0
        if g["adam_w_mode"] and g["weight_decay"]:
            direction = direction + g["weight_decay"] * p
        p.add_(direction, alpha=-_lr(g) * trust)


class Ftrl(_Base):
    """FTRL-proximal (reference: python/oneflow/nn/optimizer/ftrl.py): ``n' = n + g^2``;
    ``z += g - (n'^p - n^p) / lr * w`` with ``p = lr_power``; ``w = 0`` where ``|z| < lambda1``, else
    ``(sign(z) lambda1 - z) / ((beta + n'^p) / lr + lambda2)``."""

    def __init__(self, params, lr=1e-3, weight_decay=0.0, lr_power=-0.5, initial_accumulator_value=0.1, lambda1=0.0,
                 lambda2=0.0, beta=0.0, contiguous_params=False):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, lr_power=lr_power,
                                      initial_accumulator_value=initial_accumulator_value, lambda1=lambda1, lambda2=lambda2,
                                      beta=beta), contiguous_params)

    def _init_state(self, p, state, g):
        state["accumulate"] = torch.full_like(p, g["initial_accumulator_value"])
        state["z"] = torch.zeros_like(p)

    def _update(self, p, grad, state, g):
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        n, z, lp, lr = state["accumulate"], state["z"], g["lr_power"], _lr(g)
        new_n = n + grad * grad
        z.add_(grad - (new_n.pow(lp) - n.pow(lp)) / lr * p)
        n.copy_(new_n)
        upd = (torch.sign(z) * g["lambda1"] - z) / ((g["beta"] + new_n.pow(lp)) / lr + g["lambda2"])
        p.copy_(torch.where(z.abs() < g["lambda1"], torch.zeros_like(upd), upd))


class LBFGS(_ClipMixin, torch.optim.LBFGS):
    def __init__(self, params, lr=1.0, max_iter=20, max_eval=None, tolerance_grad=1e-7, tolerance_change=1e-9,
                 history_size=100, line_search_fn=None, contiguous_params=False):
        super().__init__(params, lr=lr, max_iter=max_iter, max_eval=max_eval, tolerance_grad=tolerance_grad,
                         tolerance_change=tolerance_change, history_size=history_size, line_search_fn=line_search_fn)


class ParamGroup(dict):
    """One optimizer param group: ``{"params": [...], option: value, ...}`` completed with the optimizer's defaults
    (reference: python/oneflow/optim/optimizer.py, ``ParamGroup``)."""

    def __init__(self, parameters, default_options):
        if isinstance(parameters, dict):
            if "params" not in parameters:
                raise ValueError("a param group needs a 'params' entry")
            super().__init__(parameters)
            self["params"] = list(parameters["params"])
        else:
            super().__init__(params=list(parameters))
        for k, v in default_options.items():
            self.setdefault(k, v)
        self._enable_clip_grad = self.get("clip_grad_max_norm") is not None

    @property
    def options(self):
        return {k: v for k, v in self.items() if k != "params"}

    @property
    def parameters(self):
        return self["params"]
