"""LR schedulers with the reference's names (python/oneflow/nn/optimizer/{step_lr,multistep_lr,cosine_*,
polynomial_lr,linear_lr,constant_lr,lambda_lr,warmup_lr,sequential_lr,chained_scheduler,
reduce_lr_on_plateau,...}.py). torch's schedulers provide the mechanics; the ones torch lacks
(CosineDecayLR, PolynomialLR with cycle, WarmupLR wrapping another scheduler) are implemented here."""
from __future__ import annotations

import math

from torch.optim import lr_scheduler as _t
from torch.optim.lr_scheduler import (ChainedScheduler, ConstantLR, CosineAnnealingLR, CosineAnnealingWarmRestarts,  # noqa: F401
                                      ExponentialLR, LambdaLR, LinearLR, MultiplicativeLR, MultiStepLR, ReduceLROnPlateau,
                                      SequentialLR, StepLR)

LRScheduler = _t.LRScheduler


class CosineDecayLR(_t.LRScheduler):
    """lr = base * ((1 - alpha) * 0.5 * (1 + cos(pi * min(step, decay_steps) / decay_steps)) + alpha)."""

    def __init__(self, optimizer, decay_steps, alpha=0.0, last_step=-1, verbose=False):
        self.decay_steps, self.alpha = decay_steps, alpha
        super().__init__(optimizer, last_epoch=last_step)

    def get_lr(self):
        s = min(self.last_epoch, self.decay_steps)
        c = 0.5 * (1 + math.cos(math.pi * s / self.decay_steps))
        return [b * ((1 - self.alpha) * c + self.alpha) for b in self.base_lrs]


class PolynomialLR(_t.LRScheduler):
    def __init__(self, optimizer, decay_batch=None, end_learning_rate=1e-4, power=1.0, cycle=False, last_step=-1,
                 verbose=False, total_iters=None):
        self.decay_batch = decay_batch if decay_batch is not None else total_iters
        self.end_lr, self.power, self.cycle = end_learning_rate, power, cycle
        super().__init__(optimizer, last_epoch=last_step)

    def get_lr(self):
        step, decay = self.last_epoch, self.decay_batch
        if self.cycle:
            decay = decay * max(1, math.ceil(step / decay))
        else:
            step = min(step, decay)
        f = (1 - step / decay) ** self.power
        return [(b - self.end_lr) * f + self.end_lr for b in self.base_lrs]


class WarmupLR(_t.LRScheduler):
    """Constant or linear warm-up for ``warmup_iters`` steps, then the wrapped scheduler (or the base lr).
    Without ``warmup_prefix`` the wrapped scheduler counts steps from 0 underneath the warm-up and a linear warm-up ends
    on the value that scheduler has at step ``warmup_iters``; with it the wrapped scheduler starts after the warm-up and
    the warm-up ends on the base lr (reference: python/oneflow/nn/optimizer/warmup_lr.py:96-200)."""

    def __init__(self, scheduler_or_optimizer, warmup_factor=1.0 / 3, warmup_iters=5, warmup_method="linear",
                 warmup_prefix=False, last_step=-1, verbose=False):
        if isinstance(scheduler_or_optimizer, _t.LRScheduler):
            self.inner = scheduler_or_optimizer
            optimizer = self.inner.optimizer
        else:
            self.inner, optimizer = None, scheduler_or_optimizer
        if warmup_method not in ("linear", "constant"):
            raise ValueError(f"'warmup_method' must be 'linear' or 'constant', but got {warmup_method}")
        if self.inner is None and warmup_iters == 0:
            raise ValueError("When 'scheduler_or_optimizer' is an optimizer warmup_iters can't be equal to 0")
        self.factor, self.iters, self.method, self.prefix = warmup_factor, warmup_iters, warmup_method, warmup_prefix
        self.end_factors = None
        if self.inner is not None and not warmup_prefix and warmup_method == "linear" and warmup_iters > 0:
            self.end_factors = self._inner_factors_at(warmup_iters)
        self._started = False              # the base class takes one step while constructing; the wrapped one already did
        super().__init__(optimizer, last_epoch=last_step)
        self._started = True

    def _inner_factors_at(self, steps):
        """lr / base lr of the wrapped scheduler ``steps`` steps from now, found by stepping it and rolling back."""
        import copy
        import warnings
        opt = self.inner.optimizer
        state, lrs = copy.deepcopy(self.inner.state_dict()), [g["lr"] for g in opt.param_groups]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            for _ in range(steps):
                self.inner.step()
        out = [g["lr"] / b if b else 1.0 for g, b in zip(opt.param_groups, self.inner.base_lrs)]
        self.inner.load_state_dict(state)
        for g, lr in zip(opt.param_groups, lrs):
            g["lr"] = lr
        return out

    def get_lr(self):
        s = self.last_epoch
        if s < self.iters:
            if self.method == "constant":
                return [b * self.factor for b in self.base_lrs]
            ends = self.end_factors or [1.0] * len(self.base_lrs)
            return [b * (self.factor + (e - self.factor) * s / max(self.iters, 1)) for b, e in zip(self.base_lrs, ends)]
        if self.inner is None:
            return list(self.base_lrs)
        return list(self.inner.get_last_lr())

    def step(self, epoch=None):
        if self.inner is not None and self._started and self.last_epoch + 1 > (self.iters if self.prefix else 0):
            self.inner.step()
        super().step()


WarmUpLR = WarmupLR


class CosineAnnealingWarmRestartsLR(CosineAnnealingWarmRestarts):
    pass
