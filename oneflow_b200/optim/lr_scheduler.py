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
    """Constant or linear warm-up for ``warmup_iters`` steps, then the wrapped scheduler (or the base lr)."""

    def __init__(self, scheduler_or_optimizer, warmup_factor=1.0 / 3, warmup_iters=5, warmup_method="linear",
                 warmup_prefix=False, last_step=-1, verbose=False):
        if isinstance(scheduler_or_optimizer, _t.LRScheduler):
            self.inner = scheduler_or_optimizer
            optimizer = self.inner.optimizer
        else:
            self.inner, optimizer = None, scheduler_or_optimizer
        if warmup_method not in ("linear", "constant"):
            raise ValueError("warmup_method must be 'linear' or 'constant'")
        self.factor, self.iters, self.method, self.prefix = warmup_factor, warmup_iters, warmup_method, warmup_prefix
        super().__init__(optimizer, last_epoch=last_step)

    def get_lr(self):
        s = self.last_epoch
        if s < self.iters:
            if self.method == "constant":
                f = self.factor
            else:
                f = self.factor + (1 - self.factor) * s / max(self.iters, 1)
            return [b * f for b in self.base_lrs]
        if self.inner is None:
            return list(self.base_lrs)
        return list(self.inner.get_last_lr())

    def step(self, epoch=None):
        if self.inner is not None and self.last_epoch + 1 >= (self.iters if self.prefix else 0):
            self.inner.step()
        super().step()


class CosineAnnealingWarmRestartsLR(CosineAnnealingWarmRestarts):
    pass
