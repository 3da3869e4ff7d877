"""Learning-rate schedulers with the reference's semantics (python/oneflow/nn/optimizer/*.py): every schedule is a
closed form ``get_lr(base_lr, step)`` of the initial learning rate and the step count, so schedules compose exactly —
``WarmupLR`` / ``SequentialLR`` switch between closed forms at milestones, ``ChainedScheduler`` nests them — and a
schedule can be evaluated at any step without replaying the steps before it (what ``nn.Graph`` needs to rebuild the
rate after a resume).  ``step()`` writes the rate into ``optimizer.param_groups[i]["lr"]``; the constructor performs
step 0.  torch's recursive schedulers are not used here: their chained form reads the optimizer's current rate, which
breaks as soon as a warm-up has rewritten it.
"""
from __future__ import annotations

import bisect
import math
import types

from torch.optim import Optimizer
from torch.optim.lr_scheduler import ReduceLROnPlateau  # noqa: F401  (metric driven, no closed form)


class LRScheduler:
    def __init__(self, optimizer, last_step=-1, verbose=False):
        if not isinstance(optimizer, Optimizer):
            raise TypeError(f"{type(optimizer).__name__} is not an Optimizer object")
        self.optimizer, self.last_step, self.verbose = optimizer, last_step, verbose
        self._init_base_lrs()
        self.step()

    # -- state
    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, state_dict):
        self.__dict__.update(state_dict)

    def _init_base_lrs(self):
        groups = self.optimizer.param_groups
        if self.last_step == -1:
            for g in groups:
                g.setdefault("initial_lr", g["lr"])
        else:
            for i, g in enumerate(groups):
                if "initial_lr" not in g:
                    raise KeyError(f"param 'initial_lr' is not specified in param_groups[{i}] when resuming an optimizer")
        self.base_lrs = [g["initial_lr"] for g in groups]

    # -- schedule
    def get_lr(self, base_lr, step):
        raise NotImplementedError

    def get_last_lr(self):
        return self._last_lr

    def print_lr(self, group, lr):
        print(f"Last step {self.last_step} of {type(self)} adjusting learning rate of param_groups[{group}] to {lr:.5f}")

    def update_lrs(self, lrs):
        self._last_lr = []
        for i, (g, lr) in enumerate(zip(self.optimizer.param_groups, lrs)):
            g["lr"] = lr
            self._last_lr.append(lr)
            if self.verbose:
                self.print_lr(i, lr)

    def step(self):
        self.last_step += 1
        self.update_lrs([self.get_lr(b, self.last_step) for b in self.base_lrs])

    # torch spelling of the step counter
    @property
    def last_epoch(self):
        return self.last_step


_LRScheduler = LRScheduler


class CosineDecayLR(LRScheduler):
    """``base * ((1 - alpha) * (1 + cos(pi * step / decay_steps)) / 2 + alpha)`` until ``decay_steps``, then
    ``base * alpha``."""

    def __init__(self, optimizer, decay_steps, alpha=0.0, last_step=-1, verbose=False):
        if decay_steps <= 0:
            raise ValueError(f"decay_steps must be greater than zero, but got {decay_steps}")
        self.decay_steps, self.alpha = decay_steps, alpha
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        if step >= self.decay_steps:
            return base_lr * self.alpha
        return base_lr * ((1 - self.alpha) * 0.5 * (1 + math.cos(math.pi * step / self.decay_steps)) + self.alpha)


class CosineAnnealingLR(LRScheduler):
    """``eta_min + (base - eta_min) * (1 + cos(pi * step / T_max)) / 2`` (periodic beyond ``T_max``)."""

    def __init__(self, optimizer, T_max, eta_min=0.0, last_step=-1, verbose=False):
        self.T_max, self.eta_min = T_max, eta_min
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        return self.eta_min + (base_lr - self.eta_min) * 0.5 * (1 + math.cos(math.pi * step / self.T_max))


class CosineAnnealingWarmRestarts(LRScheduler):
    """Cosine cycles of length ``T_0 * T_mult**i``; the peak of cycle i is ``base * decay_rate**i``; after
    ``restart_limit`` cycles (0: no limit) the rate stays at ``eta_min``."""

    def __init__(self, optimizer, T_0, T_mult=1, eta_min=0.0, decay_rate=1.0, restart_limit=0, last_step=-1, verbose=False):
        if not isinstance(T_0, int) or T_0 <= 0:
            raise ValueError(f"Expected positive integer T_0, but got {T_0}")
        if not isinstance(T_mult, int) or T_mult < 1:
            raise ValueError(f"Expected integer T_mult >= 1, but got {T_mult}")
        self.T_0, self.T_mult, self.eta_min, self.decay_rate, self.restart_limit = T_0, T_mult, eta_min, decay_rate, restart_limit
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        if self.T_mult > 1:
            cycle = math.floor(math.log(1 - step / self.T_0 * (1 - self.T_mult), self.T_mult))
            length = self.T_mult ** cycle * self.T_0
            pos = step - (1 - self.T_mult ** cycle) / (1 - self.T_mult) * self.T_0
        else:
            cycle, length = step // self.T_0, self.T_0
            pos = step - cycle * self.T_0
        if self.restart_limit > 0 and cycle >= self.restart_limit:
            return self.eta_min
        peak = base_lr * self.decay_rate ** cycle
        return self.eta_min + (peak - self.eta_min) * 0.5 * (1 + math.cos(math.pi * pos / length))


class CosineAnnealingWarmRestartsLR(CosineAnnealingWarmRestarts):
    pass


class StepLR(LRScheduler):
    def __init__(self, optimizer, step_size, gamma=0.1, last_step=-1, verbose=False):
        if step_size <= 0:
            raise ValueError(f"step_size must greater than zero, but got {step_size}")
        if gamma <= 0:
            raise ValueError(f"gamma must greater than zero, but got {gamma}")
        self.step_size, self.gamma = step_size, gamma
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        return base_lr * self.gamma ** (step // self.step_size)


class MultiStepLR(LRScheduler):
    def __init__(self, optimizer, milestones, gamma=0.1, last_step=-1, verbose=False):
        milestones = list(milestones)
        if any(b <= a for a, b in zip(milestones, milestones[1:])):
            raise ValueError("milestones should be a list of increasing integers")
        if gamma <= 0:
            raise ValueError(f"gamma must greater than zero, but got {gamma}")
        self.milestones, self.gamma = milestones, gamma
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        return base_lr * self.gamma ** bisect.bisect_right(self.milestones, step)


class ExponentialLR(LRScheduler):
    def __init__(self, optimizer, gamma, last_step=-1, verbose=False):
        if gamma <= 0:
            raise ValueError(f"'gamma' must be greater than zero, but got {gamma}")
        self.gamma = gamma
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        return base_lr * self.gamma ** step


class PolynomialLR(LRScheduler):
    """``(base - end) * (1 - step / decay_batch) ** power + end``; with ``cycle`` the horizon grows to the next
    multiple of ``decay_batch`` instead of the rate staying at ``end``."""

    def __init__(self, optimizer, decay_batch=None, end_learning_rate=1e-4, power=1.0, cycle=False, last_step=-1, verbose=False,
                 total_iters=None):
        decay_batch = decay_batch if decay_batch is not None else total_iters
        if decay_batch is None or decay_batch <= 0:
            raise ValueError(f"decay_batch must be greater than zero, but got {decay_batch}")
        self.max_decay_steps, self.end_learning_rate, self.power, self.cycle = decay_batch, end_learning_rate, power, cycle
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        horizon = self.max_decay_steps
        if self.cycle:
            cur = max(step, 1)
            horizon *= math.ceil(cur / horizon)
        else:
            cur = min(step, horizon)
        return (base_lr - self.end_learning_rate) * (1 - cur / horizon) ** self.power + self.end_learning_rate


class ConstantLR(LRScheduler):
    def __init__(self, optimizer, factor=1.0 / 3, total_iters=5, last_step=-1, verbose=False):
        if factor > 1.0 or factor < 0:
            raise ValueError("Constant multiplicative factor expected to be between 0 and 1.")
        self.factor, self.total_iters = factor, total_iters
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        return base_lr * self.factor if step < self.total_iters else base_lr


class LinearLR(LRScheduler):
    def __init__(self, optimizer, start_factor=1.0 / 3, end_factor=1.0, total_iters=5, last_step=-1, verbose=False):
        if start_factor > 1.0 or start_factor < 0:
            raise ValueError("Starting multiplicative factor expected to be between 0 and 1.")
        if end_factor > 1.0 or end_factor < 0:
            raise ValueError("Ending multiplicative factor expected to be between 0 and 1.")
        self.start_factor, self.end_factor, self.total_iters = start_factor, end_factor, total_iters
        super().__init__(optimizer, last_step, verbose)

    def get_lr(self, base_lr, step):
        if step >= self.total_iters:
            return base_lr * self.end_factor
        return base_lr * (self.start_factor + (self.end_factor - self.start_factor) * step / self.total_iters)


def _per_group(optimizer, fns, what):
    if isinstance(fns, (list, tuple)):
        if len(fns) != len(optimizer.param_groups):
            raise ValueError(f"Expected {len(optimizer.param_groups)} {what}, but got {len(fns)}")
        return list(fns)
    return [fns] * len(optimizer.param_groups)


class LambdaLR(LRScheduler):
    """``base * lr_lambda(step)``, one function for all groups or one per group."""

    def __init__(self, optimizer, lr_lambda, last_step=-1, verbose=False):
        self.lr_lambdas = _per_group(optimizer, lr_lambda, "lr_lambdas")
        super().__init__(optimizer, last_step, verbose)

    def state_dict(self):
        sd = {k: v for k, v in self.__dict__.items() if k not in ("optimizer", "lr_lambdas")}
        sd["lr_lambdas"] = [None if isinstance(f, types.FunctionType) else f.__dict__.copy() for f in self.lr_lambdas]
        return sd

    def load_state_dict(self, state_dict):
        fns = state_dict.pop("lr_lambdas")
        self.__dict__.update(state_dict)
        state_dict["lr_lambdas"] = fns
        for fn, st in zip(self.lr_lambdas, fns):
            if st is not None:
                fn.__dict__.update(st)

    def step(self):
        self.last_step += 1
        self.update_lrs([b * f(self.last_step) for b, f in zip(self.base_lrs, self.lr_lambdas)])


class MultiplicativeLR(LambdaLR):
    """``lr <- lr * lr_lambda(step)`` from step 1 on (the one schedule defined by recurrence)."""

    def step(self):
        self.last_step += 1
        groups = self.optimizer.param_groups
        if self.last_step > 0:
            self.update_lrs([g["lr"] * f(self.last_step) for g, f in zip(groups, self.lr_lambdas)])
        else:
            self.update_lrs([g["lr"] for g in groups])


def _same_optimizer(optimizer, schedulers, who):
    for i, s in enumerate(schedulers):
        if s.optimizer is not optimizer:
            raise ValueError(f"{who} expects all schedulers to belong to the same optimizer, but the scheduler at index {i} "
                             "belongs to another one")


class _Composite(LRScheduler):
    def state_dict(self):
        sd = {k: v for k, v in self.__dict__.items() if k not in ("optimizer", "schedulers")}
        sd["schedulers"] = [s.state_dict() for s in self.schedulers]
        return sd

    def load_state_dict(self, state_dict):
        subs = state_dict.pop("schedulers")
        self.__dict__.update(state_dict)
        state_dict["schedulers"] = subs
        for s, sd in zip(self.schedulers, subs):
            s.load_state_dict(sd)


class SequentialLR(_Composite):
    """Scheduler i is in charge from milestone i-1 to milestone i.  With ``interval_rescaling`` it sees steps counted
    from its milestone, otherwise the global step count."""

    def __init__(self, optimizer, schedulers, milestones, interval_rescaling=False, last_step=-1, verbose=False):
        schedulers, milestones = list(schedulers), list(milestones)
        if not schedulers:
            raise ValueError("Sequential Schedulers expects at least one scheduler")
        _same_optimizer(optimizer, schedulers, "Sequential Schedulers")
        if len(milestones) != len(schedulers) - 1:
            raise ValueError(f"Sequential Schedulers expects one more scheduler than milestones, but got {len(schedulers)} "
                             f"schedulers and {len(milestones)} milestones")
        if isinstance(interval_rescaling, (list, tuple)):
            if len(interval_rescaling) != len(milestones):
                raise ValueError("'interval_rescaling' expects a bool or one bool per milestone")
            interval_rescaling = [bool(r) for r in interval_rescaling]
        else:
            interval_rescaling = [bool(interval_rescaling)] * len(milestones)
        self.schedulers, self.milestones, self.interval_rescaling = schedulers, milestones, interval_rescaling
        super().__init__(optimizer, last_step, verbose)

    def step(self):
        self.last_step += 1
        i = bisect.bisect_right(self.milestones, self.last_step)
        local = self.last_step - self.milestones[i - 1] if i > 0 and self.interval_rescaling[i - 1] else self.last_step
        s = self.schedulers[i]
        s.last_step = local
        self.update_lrs([s.get_lr(b, local) for b in self.base_lrs])


class ChainedScheduler(_Composite):
    """Applies the schedulers one inside the other: the rate scheduler k yields is the base of scheduler k+1."""

    def __init__(self, schedulers):
        schedulers = list(schedulers)
        if not schedulers:
            raise ValueError("ChainedScheduler expects at least one scheduler")
        opt = schedulers[0].optimizer
        _same_optimizer(opt, schedulers, "ChainedScheduler")
        self.schedulers = schedulers
        self.optimizer, self.last_step, self.verbose = opt, schedulers[0].last_step - 1, False
        self.base_lrs = list(schedulers[0].base_lrs)
        self.step()

    def step(self):
        self.last_step += 1
        lrs = list(self.schedulers[0].base_lrs)
        for s in self.schedulers:
            lrs = [s.get_lr(lr, self.last_step) for lr in lrs]
            s.last_step = self.last_step
        self.update_lrs(lrs)


class _UnboundLinear(LinearLR):
    """LinearLR whose end factor is not limited to [0, 1] (a warm-up may end above or below the base rate) and that
    does not write the optimizer when constructed (the enclosing schedule does)."""

    def __init__(self, optimizer, start_factor, end_factor, total_iters, last_step):
        self.start_factor, self.end_factor, self.total_iters = start_factor, end_factor, total_iters
        self.optimizer, self.last_step, self.verbose = optimizer, last_step, False
        self.base_lrs = [g["initial_lr"] for g in optimizer.param_groups]


class _UnboundConstant(ConstantLR):
    def __init__(self, optimizer, factor, total_iters, last_step):
        self.factor, self.total_iters = factor, total_iters
        self.optimizer, self.last_step, self.verbose = optimizer, last_step, False
        self.base_lrs = [g["initial_lr"] for g in optimizer.param_groups]


class WarmupLR(SequentialLR):
    """``warmup_iters`` steps of constant (``base * warmup_factor``) or linear warm-up, then the wrapped scheduler, or the
    base rate when an optimizer was passed.  Without ``warmup_prefix`` the wrapped scheduler keeps counting global
    steps and a linear warm-up ends on the value that scheduler has at step ``warmup_iters``; with it the wrapped
    scheduler starts from its step 0 after the warm-up and the warm-up ends on the base rate."""

    def __init__(self, scheduler_or_optimizer, warmup_factor=1.0 / 3, warmup_iters=5, warmup_method="linear",
                 warmup_prefix=False, last_step=-1, verbose=False):
        if not isinstance(scheduler_or_optimizer, (LRScheduler, Optimizer)):
            raise ValueError("'scheduler_or_optimizer' must be a LRScheduler or an Optimizer, but got "
                             f"{type(scheduler_or_optimizer)}")
        if warmup_method not in ("linear", "constant"):
            raise ValueError(f"'warmup_method' must be 'linear' or 'constant', but got {warmup_method}")
        if isinstance(scheduler_or_optimizer, LRScheduler):
            inner, opt = scheduler_or_optimizer, scheduler_or_optimizer.optimizer
        else:
            inner, opt = None, scheduler_or_optimizer
        if inner is None and warmup_iters == 0:
            raise ValueError("When 'scheduler_or_optimizer' is an optimizer warmup_iters can't be equal to 0")
        self.warmup_factor, self.warmup_iters = warmup_factor, warmup_iters
        self.warmup_method, self.warmup_prefix = warmup_method, warmup_prefix
        self.optimizer, self.last_step, self.verbose = opt, last_step, verbose
        self._init_base_lrs()
        warm = None
        if warmup_iters > 0:
            if warmup_method == "linear":
                end = 1.0
                if inner is not None and not warmup_prefix:
                    base = self.base_lrs[0]
                    if any(not math.isclose(b, base) for b in self.base_lrs):
                        raise ValueError("The param_groups in optimizer have different warmup configs, please use different "
                                         "optimizers.")
                    end = inner.get_lr(base, warmup_iters) / base
                warm = _UnboundLinear(opt, warmup_factor, end, warmup_iters, last_step)
            else:
                warm = _UnboundConstant(opt, warmup_factor, warmup_iters, last_step)
        schedulers = [s for s in (warm, inner) if s is not None]
        milestones = [warmup_iters] if warm is not None and inner is not None else []
        super().__init__(opt, schedulers, milestones, [bool(warmup_prefix)] * len(milestones), last_step, verbose)


WarmUpLR = WarmupLR
