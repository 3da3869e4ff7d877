"""Fused optimizer state of an ``nn.Graph``: what the reference's optimizer passes build at compile time.

When a graph is compiled, every optimizer it was given is turned into flat buffers on this rank
(reference: the model-update ops generated per variable, oneflow/core/job_rewriter/optimizer.cpp and
adam_optm.cpp, then fused by fuse_update_ops_pass.cpp / multi_tensor_model_update.cpp; gradient accumulation
buffers from the acc/unpack ops of lazy_op_interpreter.cpp:270-330):

* the local shards of its parameters move into ONE flat buffer in the parameters' dtype (the tensors the
  modules use become views of it), ordered [decayed | not decayed] per param group;
* one flat fp32 gradient buffer of the same layout: every parameter gets a ``_main_grad`` view, into which the
  fused ops accumulate weight gradients straight from the GEMM epilogue over all micro-batches of a step
  (framework/fused_ops.py); gradients that arrive through plain autograd (``p.grad``) are folded in at step time;
* fp32 master weights and Adam moments (or the momentum buffer) as flat buffers, updated by one multi-tensor
  kernel per segment, which also writes the parameters' low-precision copy.

Gradient layouts: a parameter gradient produced from activations whose rows were split along a mesh axis is a
partial sum (``P``) on that axis. At step time every axis on which ALL local gradients are partial is treated as a
data-parallel axis: one flat all-reduce, or with ``config.enable_zero`` a flat reduce-scatter into this rank's
slice, whose master weights / moments are the only ones kept (ZeRO stage 1:
oneflow/core/job_rewriter/optimizer_placement_optimization_pass.cpp:381-467), followed by an all-gather of the
updated parameters. Axes on which only some gradients are partial (LayerNorm parameters and row-parallel biases
under sequence parallelism) get one packed all-reduce of just those tensors. The global gradient norm counts
every logical element once: each rank contributes ||local gradient||^2 / (number of ranks holding a copy).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ...framework import global_tensor as GT
from ...ops import kernels as K


def _loc(t):
    return t._local if isinstance(t, GT.GlobalTensor) else t


def _align(n, a=64):
    return (n + a - 1) // a * a


class _Slot:
    __slots__ = ("param", "off", "n", "group", "decay")


class FlatOptimizer:
    """Flat-buffer execution of one ``flow.optim`` optimizer (AdamW / Adam / SGD) for the parameters that live on this
    rank. ``step()`` = gradient sync + clip + fused update; hyper-parameters are read from the optimizer's param groups
    at every step, so LR schedulers keep working on the original object."""

    def __init__(self, optim, zero_stage=0, grad_scaler=None):
        from ...optim import optimizer as O
        self.optim = optim
        self.kind = "adam" if isinstance(optim, O._AdamFamily) else ("sgd" if isinstance(optim, O.SGD) else None)
        if self.kind is None:
            raise TypeError("FlatOptimizer handles Adam, AdamW and SGD")
        self.zero_stage = zero_stage
        me = GT._rank()
        slots = []
        for gi, g in enumerate(optim.param_groups):
            for p in g["params"]:
                if not p.requires_grad:
                    continue
                if isinstance(p, GT.GlobalTensor) and not p._placement.contains(me):
                    continue
                if _loc(p).numel() == 0:
                    continue
                s = _Slot()
                s.param, s.group = p, gi
                s.decay = float(g.get("weight_decay", 0.0)) != 0.0
                s.n = _loc(p).numel()
                slots.append(s)
        if not slots:
            self.slots, self.total = [], 0
            return
        dev, dt = _loc(slots[0].param).device, _loc(slots[0].param).dtype
        if any(_loc(s.param).device != dev or _loc(s.param).dtype != dt for s in slots):
            raise TypeError("FlatOptimizer needs all parameters of an optimizer on one device in one dtype")
        # replicated-on-a-model-axis tensors (vectors, mostly) go last inside their group so that their packed
        # all-reduce touches neighbouring memory
        slots.sort(key=lambda s: (s.group, _loc(s.param).dim() < 2))
        off = 0
        for s in slots:
            s.off = off
            off += _align(s.n)
        self.slots, self.total, self.device, self.dtype = slots, off, dev, dt
        self.flat = torch.zeros(off, dtype=dt, device=dev)
        self.grad = torch.zeros(off, dtype=torch.float32, device=dev)
        for s in slots:
            p = s.param
            loc = _loc(p)
            view = self.flat[s.off:s.off + s.n].view(loc.shape)
            view.copy_(loc.detach())
            if isinstance(p, GT.GlobalTensor):
                p._local = view
            else:
                p.data = view
            p._main_grad = self.grad[s.off:s.off + s.n].view(loc.shape)
            p._grad_nd_sbp = None
        self.step_count = 0
        self._state_ready = False
        self._arena = None
        self._dp = None          # (placement, axis, group, ranks, collective helper) once the first step has seen the layouts
        self._lo, self._hi = 0, off
        self._sq = None
        self.last_norm = None

    # ------------------------------------------------------------------ layout discovery (first step)
    def _discover(self):
        """Reads the gradient layouts recorded by the first backward and decides the data-parallel axis."""
        pls = {}
        for s in self.slots:
            p = s.param
            if isinstance(p, GT.GlobalTensor):
                pls.setdefault(p._placement, []).append(s)
        self._dp = None
        self._partial_sets = []       # [(placement, axis, [slots])] needing a packed all-reduce
        if not dist.is_initialized():
            return
        for pl, ss in pls.items():
            for a, n in enumerate(pl.hierarchy):
                if n == 1:
                    continue
                part = [s for s in ss if s.param._grad_nd_sbp is not None and s.param._grad_nd_sbp[a].kind == "P"]
                if not part:
                    continue
                if len(part) == len(ss) and len(pls) == 1 and len(ss) == len(self.slots) and self._dp is None:
                    self._dp = (pl, a)
                else:
                    self._partial_sets.append((pl, a, part))

    def _dp_helper(self):
        pl, a = self._dp
        me = GT._rank()
        ranks = pl.axis_ranks(a, me)
        group = pl.axis_group(a)
        if self.zero_stage >= 1:
            from ...parallel.zero import ZeroShard
            return ZeroShard(group, ranks, self.device)
        from ...parallel.zero import GradAllReduce
        return GradAllReduce(group, ranks, self.device)

    def _move_into_arena(self):
        """ZeRO on CUDA: the gradient and parameter buffers move into a peer-mapped arena (parallel.zero.ArenaZero), the
        parameters' tensors and their ``_main_grad`` views are re-pointed, and from then on the gradient reduce-scatter
        and the parameter all-gather work in place on them."""
        from ...parallel.zero import ArenaZero
        pl, a = self._dp
        me = GT._rank()
        az = ArenaZero(pl.axis_group(a), pl.axis_ranks(a, me), self.device, self.total, self.dtype)
        az.flat[:self.total].copy_(self.flat)
        az.grad[:self.total].copy_(self.grad)
        self.flat, self.grad = az.flat, az.grad
        for s in self.slots:
            p = s.param
            shape = _loc(p).shape
            view = self.flat[s.off:s.off + s.n].view(shape)
            if isinstance(p, GT.GlobalTensor):
                p._local = view
            else:
                p.data = view
            p._main_grad = self.grad[s.off:s.off + s.n].view(shape)
        return az

    def _init_state(self):
        self._discover()
        self._arena = None
        if self._dp is not None and self.zero_stage >= 1 and self.device.type == "cuda" and \
                self.dtype in (torch.float32, torch.bfloat16) and self._dp[0].hierarchy[self._dp[1]] <= 8:
            self._arena = self._move_into_arena()
            self._helper = self._arena
        else:
            self._helper = self._dp_helper() if self._dp is not None else None
        if self._helper is not None and self.zero_stage >= 1:
            self._lo, self._hi = self._helper.range(self.total)
        n = self._hi - self._lo
        self.master = self.flat[self._lo:self._hi].float()
        self.m = torch.zeros(n, dtype=torch.float32, device=self.device) if (self.kind == "adam" or self._momentum()) else None
        self.v = torch.zeros(n, dtype=torch.float32, device=self.device) if self.kind == "adam" else None
        self._sq = torch.zeros(2, dtype=torch.float32, device=self.device)
        self._state_ready = True

    def _momentum(self):
        return any(float(g.get("momentum", 0.0)) != 0.0 for g in self.optim.param_groups)

    # ------------------------------------------------------------------ step
    def zero_grad(self):
        if self.total:
            self.grad.zero_()
        for s in self.slots:
            s.param.grad = None

    def _fold_autograd_grads(self):
        """Gradients that reached ``p.grad`` through plain autograd are added into the flat buffer in the layout the
        buffer already holds for that parameter (partial sums stay partial: the reduced value goes to one rank)."""
        from ... import sbp as S
        for s in self.slots:
            p = s.param
            g = p.grad
            if g is None:
                continue
            if isinstance(g, GT.GlobalTensor):
                have = p._grad_nd_sbp
                if have is None:
                    have = tuple(x if x.kind == "P" else px for x, px in zip(g._nd_sbp, p._nd_sbp))
                    p._grad_nd_sbp = have
                want = tuple(S.partial_sum if h.kind == "P" else px for h, px in zip(have, p._nd_sbp))
                g = GT.rebox(g.detach(), want)._local
            p._main_grad.add_(g.detach().to(torch.float32).view(p._main_grad.shape))
            p.grad = None

    def _replication(self, s):
        """Number of ranks that hold a copy of this slot's (synchronised) local gradient."""
        p = s.param
        if not isinstance(p, GT.GlobalTensor):
            return dist.get_world_size() if dist.is_initialized() and self._dp is None and False else 1
        r = 1
        for a, (n, sb) in enumerate(zip(p._placement.hierarchy, p._nd_sbp)):
            if sb.kind != "S" and not (self._dp is not None and self.zero_stage >= 1 and (p._placement, a) == self._dp):
                r *= n
        return r

    def step(self, loss_scale=1.0, found_inf_extra=None):
        if not self.total:
            return
        self._fold_autograd_grads()
        if not self._state_ready:
            self._init_state()
        self.step_count += 1
        inv = 1.0 / loss_scale
        # 1. partial sums over model-parallel axes that concern only some tensors: one packed all-reduce per axis
        for pl, a, part in self._partial_sets:
            views = [s.param._main_grad.reshape(-1) for s in part]
            packed = torch.cat(views)
            dist.all_reduce(packed, group=pl.axis_group(a))
            o = 0
            for v in views:
                v.copy_(packed[o:o + v.numel()])
                o += v.numel()
        # 2. the data-parallel axis: flat mean over the axis (all-reduce, or reduce-scatter into this rank's slice)
        if self._helper is not None:
            if self._arena is not None:
                grad_shard = self._arena.reduce_scatter_grads()[:self._hi - self._lo]
            else:
                grad_shard = self._helper.reduce_scatter_grads(self.grad, self._lo, self._hi)
            dp_n = self._helper.size
            if self.zero_stage < 1:
                grad_shard = self.grad[self._lo:self._hi]
            # the helpers average; the reference sums partial gradients of a mean loss computed per shard, which is the
            # same thing when the loss is a mean over the global batch (the local loss is already divided by the global
            # count only if the user wrote it so): keep the sum semantics of P -> B here
            if dp_n > 1:
                inv *= float(dp_n)
        else:
            grad_shard = self.grad
        # 3. global norm over all ranks, every logical element once
        clip = max((float(g.get("clip_grad_max_norm") or 0.0) for g in self.optim.param_groups), default=0.0)
        factor = found = None
        if clip > 0.0 or found_inf_extra is not None:
            by_rep = {}
            for s in self.slots:
                lo, hi = max(s.off, self._lo), min(s.off + s.n, self._hi)
                if hi > lo:
                    by_rep.setdefault(self._replication(s), []).append(grad_shard[lo - self._lo:hi - self._lo])
            sq = self._sq.zero_()
            for rep, views in by_rep.items():
                part = K.multi_tensor_sqsum(views)
                sq[0] += part[0] * (inv * inv / rep)
                sq[1] += part[1]
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(sq)
            factor, found, self.last_norm = K.clip_factor(sq, clip)
        # 4. fused update per (group, decay) segment of this rank's slice
        for lo, hi, g in self._segments():
            a, b = lo - self._lo, hi - self._lo
            self._update(grad_shard[a:b], a, b, lo, hi, g, inv, factor, found)
        # 5. ZeRO: the updated low-precision parameters of the other slices
        if self._arena is not None:
            self._arena.all_gather_params()
        elif self._helper is not None and self.zero_stage >= 1:
            self._helper.all_gather_params(self.flat, self._lo, self._hi)

    def _segments(self):
        segs = []
        cur = None
        for s in self.slots:
            key = s.group
            lo, hi = max(s.off, self._lo), min(s.off + _align(s.n), self._hi)
            if hi <= lo:
                continue
            if cur is not None and cur[2] == key and cur[1] == lo:
                cur[1] = hi
            else:
                cur = [lo, hi, key]
                segs.append(cur)
        return [(lo, hi, self.optim.param_groups[k]) for lo, hi, k in segs]

    def _update(self, grad, a, b, lo, hi, g, scale, factor, found):
        lr = g["lr"] * g.get("lr_scale", 1.0)
        if self.kind == "adam":
            b1, b2 = g["betas"]
            dec = getattr(self.optim, "decoupled", False)
            K.multi_tensor_adamw([grad], [self.master[a:b]], [self.flat[lo:hi]], [self.m[a:b]], [self.v[a:b]], lr=lr,
                                 beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"] if dec else 0.0,
                                 l2=0.0 if dec else g["weight_decay"], scale=scale, step=self.step_count,
                                 bias_correction=g.get("do_bias_correction", True), scale_tensor=factor, skip_if=found)
        else:
            mom = float(g.get("momentum", 0.0))
            K.multi_tensor_sgd([grad], [self.master[a:b]], [self.flat[lo:hi]], [self.m[a:b]] if self.m is not None else None,
                               lr=lr, momentum=mom, dampening=float(g.get("dampening", 0.0)), nesterov=bool(g.get("nesterov", False)),
                               maximize=bool(g.get("maximize", False)), l2=float(g.get("weight_decay", 0.0)), scale=scale,
                               scale_tensor=factor, skip_if=found)

    # ------------------------------------------------------------------ state
    def state_dict(self):
        sd = {"step": self.step_count, "lo": self._lo, "hi": self._hi}
        if self._state_ready:
            sd.update(master=self.master, m=self.m, v=self.v)
        return sd

    def load_state_dict(self, sd):
        self.step_count = int(sd.get("step", 0))
        if "master" in sd:
            if not self._state_ready:
                self._discover()
                self._helper = None
                self._lo, self._hi = int(sd["lo"]), int(sd["hi"])
                self.master = sd["master"].to(self.device).clone()
                self.m = sd["m"].to(self.device).clone() if sd.get("m") is not None else None
                self.v = sd["v"].to(self.device).clone() if sd.get("v") is not None else None
                self._sq = torch.zeros(2, dtype=torch.float32, device=self.device)
                self._state_ready = True
                self._helper = self._dp_helper() if self._dp is not None else None
            else:
                self.master.copy_(sd["master"])
                if self.m is not None and sd.get("m") is not None:
                    self.m.copy_(sd["m"])
                if self.v is not None and sd.get("v") is not None:
                    self.v.copy_(sd["v"])
            self.flat[self._lo:self._hi].copy_(self.master)
