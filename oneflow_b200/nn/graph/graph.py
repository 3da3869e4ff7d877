"""``flow.nn.Graph``: the static-graph training / inference front-end.

The reference traces ``build()`` into a Job, runs ~45 rewrite passes and executes a Plan on an actor
runtime (python/oneflow/nn/graph/graph.py:257-286, 846-877, 1359-1449, 1740-1795). Here the same contract
is met without a tracing compiler: ``build()`` runs on the eager engine (global tensors dispatch through
the SBP rules, kernels launch on CUDA streams), and nn.Graph supplies what the passes provided —

* one call = one mini-batch: with ``set_gradient_accumulation_steps(N)`` tensor inputs are unpacked on
  dim 0 into N micro-batches, gradients accumulate, outputs are packed again (lazy_op_interpreter.cpp:270-330);
* ``loss.backward()`` inside ``build`` feeds the optimizers added with ``add_optimizer``; after the last
  micro-batch gradients are clipped (``clip_grad_max_norm``), the (fused) optimizer steps, LR schedulers
  step and the train-step counter advances;
* ``config.enable_amp`` runs ``build`` under autocast; ``set_grad_scaler`` adds dynamic / static loss scaling;
* ``config.enable_zero`` turns broadcast parameters (and therefore their optimizer states) into ``S(0)``
  shards over the data-parallel axis (optimizer_placement_optimization_pass.cpp);
* ``GraphModule.set_stage(stage_id, placement)`` moves a block's inputs to its stage's placement
  (proxy.py:240-308), ``activation_checkpointing`` recomputes the block in backward;
* ``state_dict`` / ``load_state_dict`` cover module blocks, optimizer states and ``System-Train-TrainStep``;
* inputs must keep the same meta on every call (nn_graph.cpp:882-893).
"""
from __future__ import annotations

import contextlib
import os
from collections import OrderedDict
from typing import List

import torch
import torch.distributed as dist

from ...framework import global_tensor as GT
from ... import sbp as S
from .graph_config import GraphConfig


class GraphModule:
    """Per-block graph settings reached through ``block.to(GraphModule)`` (or the older ``block.config``)."""

    def __init__(self, proxy):
        self._proxy = proxy
        self.stage_id = None
        self.stage_placement = None
        self.activation_checkpointing = False

    def set_stage(self, stage_id=None, placement=None):
        self.stage_id, self.stage_placement = stage_id, placement
        return self

    # older attribute-style API
    @property
    def stage_id_(self):
        return self.stage_id


class Proxy:
    """Base of what a Graph holds in place of an ``nn.Module`` or tensor attribute: ``.to(GraphModule)`` gives the
    graph-side settings, ``.to(nn.Module)`` the original (reference: python/oneflow/nn/graph/proxy.py:60-79)."""


class ModuleProxy(Proxy):
    """What ``self.m = module`` becomes inside a Graph: calls go to the module, with stage placement and
    activation checkpointing applied; attribute access reaches sub-modules (as proxies) and parameters."""

    def __init__(self, module, name, graph):
        object.__setattr__(self, "_module", module)
        object.__setattr__(self, "_name", name)
        object.__setattr__(self, "_graph", graph)
        object.__setattr__(self, "_gm", GraphModule(self))
        object.__setattr__(self, "_children", {})

    def to(self, kind=None, *args, **kwargs):
        if kind is GraphModule or kind is None:
            return self._gm
        if kind is torch.nn.Module:
            return self._module
        self._module.to(kind, *args, **kwargs)
        return self

    @property
    def config(self):
        return self._gm

    @property
    def origin(self):
        return self._module

    def __getattr__(self, name):
        mod = object.__getattribute__(self, "_module")
        child = mod._modules.get(name) if hasattr(mod, "_modules") else None
        if child is not None:
            ch = self._children.get(name)
            if ch is None:
                ch = ModuleProxy(child, f"{self._name}.{name}", self._graph)
                self._children[name] = ch
            return ch
        return getattr(mod, name)

    def __setattr__(self, name, value):
        setattr(self._module, name, value)

    # containers (ModuleList / Sequential / ModuleDict): ``self.m.layers[i].to(GraphModule).set_stage(...)``
    def _child(self, key):
        mod = object.__getattribute__(self, "_module")
        name = str(key)
        if isinstance(key, int) and key < 0:
            name = str(len(mod) + key)
        child = mod._modules.get(name)
        if child is None:
            raise KeyError(key)
        ch = self._children.get(name)
        if ch is None:
            ch = ModuleProxy(child, f"{self._name}.{name}", self._graph)
            self._children[name] = ch
        return ch

    def __getitem__(self, key):
        if isinstance(key, slice):
            return [self._child(i) for i in range(*key.indices(len(self._module)))]
        return self._child(key)

    def __len__(self):
        return len(self._module)

    def __iter__(self):
        mod = self._module
        if isinstance(mod, torch.nn.ModuleDict):
            return iter(mod.keys())
        return (self._child(i) for i in range(len(mod)))

    def _walk(self):
        yield self
        for ch in self._children.values():
            yield from ch._walk()

    def __call__(self, *args, **kwargs):
        gm = self._gm
        if gm.stage_placement is not None:
            args = tuple(_to_stage(a, gm.stage_placement) for a in args)
            kwargs = {k: _to_stage(v, gm.stage_placement) for k, v in kwargs.items()}
            if not gm.stage_placement.contains(GT._rank()):
                # a stage of another rank: the recorded plan knows what it returns, nothing of it runs here
                meta = self.__dict__.get("_skip_meta")
                if meta is not None and not kwargs:
                    return _skipped_stage(meta, args)
                out = self._call_module(gm, args, kwargs)
                if not kwargs:
                    self.__dict__["_skip_meta"] = _record_outputs(out)
                return out
        return self._call_module(gm, args, kwargs)

    def _call_module(self, gm, args, kwargs):
        mod = self._module
        fn = mod
        if self._children:
            fn = _ChildPatched(self)
        if gm.activation_checkpointing and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint
            return checkpoint(fn, *args, use_reentrant=False, **kwargs)
        return fn(*args, **kwargs)


class _ChildPatched:
    """Calls the module while its children that have proxies are temporarily replaced by shims calling those proxies,
    so that stage / checkpoint settings of nested blocks take effect. Pure containers (ModuleList, ModuleDict) stay in
    place and their entries are replaced instead."""

    def __init__(self, proxy):
        self.proxy = proxy

    @staticmethod
    def _patch(proxy, saved):
        mod = proxy._module
        for name, ch in proxy._children.items():
            child = mod._modules.get(name)
            if child is None:
                continue
            if isinstance(child, (torch.nn.ModuleList, torch.nn.ModuleDict)):
                _ChildPatched._patch(ch, saved)
            else:
                saved.append((mod, name, child))
                mod._modules[name] = _CallShim(ch)

    def __call__(self, *args, **kwargs):
        saved = []
        self._patch(self.proxy, saved)
        try:
            return self.proxy._module(*args, **kwargs)
        finally:
            for mod, name, m in saved:
                mod._modules[name] = m


class _CallShim(torch.nn.Module):
    def __init__(self, proxy):
        super().__init__()
        object.__setattr__(self, "_p", proxy)

    def forward(self, *a, **k):
        return self._p(*a, **k)


def _to_stage(x, placement):
    if isinstance(x, GT.GlobalTensor) and x.placement != placement:
        nd = x.sbp if len(x.sbp) == placement.ndim else (S.broadcast,) * placement.ndim
        return GT.to_global(x, placement, nd)
    return x


def _record_outputs(out):
    """(tree spec, per-leaf description) of what a stage's module returned on a rank outside its placement."""
    from torch.utils import _pytree as pytree
    flat, spec = pytree.tree_flatten(out)
    leaves = []
    for t in flat:
        if isinstance(t, GT.GlobalTensor):
            leaves.append(("g", tuple(t.shape), t.dtype, t.placement, t.sbp, bool(t.requires_grad)))
        elif isinstance(t, torch.Tensor):
            return None                      # a local tensor result cannot be reproduced without running the module
        else:
            leaves.append(("o", t))
    return spec, leaves


class _SkippedStage(torch.autograd.Function):
    """Stands for a pipeline stage that runs on other ranks: placeholders of the recorded outputs go forward, placeholder
    gradients of the inputs go backward (the stage-boundary ``to_global`` around it moves the real data)."""

    @staticmethod
    def forward(ctx, leaves, anchor, *tensors):
        ctx.in_meta = [(tuple(t.shape), t.dtype, t.placement, t.sbp) if isinstance(t, GT.GlobalTensor) else None for t in tensors]
        gl = [l for l in leaves if l[0] == "g"]
        outs = tuple(GT._placeholder(torch.empty(l[1], dtype=l[2], device="meta"), l[3], l[4]) for l in gl)
        ctx.mark_non_differentiable(*[o for o, l in zip(outs, gl) if not (l[5] and o.dtype.is_floating_point)])
        return outs

    @staticmethod
    def backward(ctx, *grads):
        res = [None, None]
        for m in ctx.in_meta:
            res.append(None if m is None or not m[1].is_floating_point else
                       GT._placeholder(torch.empty(m[0], dtype=m[1], device="meta"), m[2], m[3]))
        return tuple(res)


def _skipped_stage(meta, args):
    from torch.utils import _pytree as pytree
    spec, leaves = meta
    tensors = [a for a in args if isinstance(a, torch.Tensor)]
    # the real stage's outputs depend on its parameters, so they take part in autograd even when no input does: the
    # anchor gives the stand-in the same property (the stage-boundary transfer after it must get its backward node)
    anchor = torch.zeros((), requires_grad=torch.is_grad_enabled())
    outs = list(_SkippedStage.apply(leaves, anchor, *tensors))
    flat = [outs.pop(0) if l[0] == "g" else l[1] for l in leaves]
    return pytree.tree_unflatten(flat, spec)


class Graph:
    _nesting = 0

    def __init__(self, enable_get_runtime_state_dict=False):
        object.__setattr__(self, "_blocks", OrderedDict())
        self.config = GraphConfig()
        self._opts = []            # dicts: optim, lr_sch, is_sparse
        self._grad_scaler = None
        self._compiled = False
        self._train_step = 0
        self._input_meta = None
        self._debug_level = -1
        self._debug_ranks = None
        self._name = f"{type(self).__name__}_{id(self) & 0xffff}"
        self._pending_state = None
        self._flat = []
        self._plan = None

    # ------------------------------------------------------------------ construction API
    def __setattr__(self, name, value):
        if isinstance(value, torch.nn.Module):
            self._blocks[name] = ModuleProxy(value, name, self)
            return
        object.__setattr__(self, name, value)

    def __getattr__(self, name):
        blocks = object.__getattribute__(self, "_blocks")
        if name in blocks:
            return blocks[name]
        raise AttributeError(name)

    def build(self, *args, **kwargs):
        raise NotImplementedError("nn.Graph subclasses must implement build()")

    def add_optimizer(self, optim, *, lr_sch=None, is_sparse=False):
        if lr_sch is not None and getattr(lr_sch, "optimizer", optim) is not optim:
            raise ValueError("lr_sch must wrap the optimizer it is added with")
        if lr_sch is not None:
            # The graph advances a schedule of its own, as the reference compiles the schedule into the job: the
            # caller's scheduler object is left where it is and can go on driving eager steps.
            import copy
            lr_sch = copy.deepcopy(lr_sch, {id(optim): optim})
        self._opts.append({"optim": optim, "lr_sch": lr_sch, "is_sparse": is_sparse})
        self.config.training = True

    def set_grad_scaler(self, grad_scaler):
        self._grad_scaler = grad_scaler

    @property
    def name(self):
        return self._name

    @property
    def training(self):
        return self.config.training

    @property
    def _is_compiled(self):
        return self._compiled

    @property
    def is_compiled(self):
        """True once the first call has fixed placement decisions and input meta."""
        return self._compiled

    # ------------------------------------------------------------------ sharing / runtime state / dynamic shapes
    def enable_shared(self, mode=True):
        """Lets other graphs of the same class reuse this graph's compile-time decisions (auto-parallel choices)
        through :meth:`share_from`; must be set before the first call
        (reference: python/oneflow/nn/graph/graph.py:879-899)."""
        if mode and self._compiled:
            raise RuntimeError("enable_shared must be set before graph compile")
        object.__setattr__(self, "_enable_shared_from_this", bool(mode))

    def share_from(self, shared_graph):
        if not isinstance(shared_graph, Graph):
            raise TypeError("shared_graph must be an instance of nn.Graph")
        if not getattr(shared_graph, "_enable_shared_from_this", False):
            raise RuntimeError("shared_graph must have been enabled to be shared")
        if not shared_graph._compiled:
            raise RuntimeError("shared_graph must have been compiled")
        object.__setattr__(self, "_shared_graph", shared_graph)

    def enable_save_runtime_state_dict(self, mode=True):
        if mode and self._compiled:
            raise RuntimeError("enable_save_runtime_state_dict must be set before graph compile")
        object.__setattr__(self, "_enable_save_runtime_state_dict", bool(mode))

    @staticmethod
    def with_dynamic_input_shape(*, size=10, enable_shared=True):
        """Decorator for ``__init__``: the graph then accepts inputs of changing shapes, remembering the
        ``size`` most recently used input signatures instead of insisting on the first one
        (reference: python/oneflow/nn/graph/graph.py:2125-2143, python/oneflow/nn/graph/cache.py)."""
        import functools

        def deco(init):
            @functools.wraps(init)
            def wrapped(self, *args, **kwargs):
                init(self, *args, **kwargs)
                object.__setattr__(self, "_dynamic_metas", OrderedDict())
                object.__setattr__(self, "_dynamic_cache_size", int(size))
            return wrapped
        return deco

    def _ops_repr(self):
        """One line per block and leaf module, in execution-independent (registration) order."""
        lines = []
        for name, proxy in self._blocks.items():
            for sub, mod in proxy._module.named_modules():
                if not list(mod.children()):
                    lines.append(f"(OPERATOR: {self._name}.{name}{'.' + sub if sub else ''}: {mod})")
        return lines

    @property
    def _graph_proto(self):
        """A plain-dict description of the graph: name, config, blocks with stage settings, optimizers, input meta."""
        cfg = {k: v for k, v in vars(self.config).items() if not k.startswith("_") and isinstance(v, (int, float, bool, str, type(None)))}
        blocks = {n: {"type": type(p._module).__name__, "stage_id": p._gm.stage_id,
                      "activation_checkpointing": p._gm.activation_checkpointing,
                      "parameters": sum(q.numel() for q in p._module.parameters())} for n, p in self._blocks.items()}
        return {"name": self._name, "training": self.config.training, "config": cfg, "blocks": blocks,
                "optimizers": [type(o["optim"]).__name__ for o in self._opts],
                "inputs": [str(m) for m in (self._input_meta or [])], "compiled": self._compiled}

    @property
    def _full_graph_proto(self):
        return self._graph_proto

    @property
    def _compiled_graph_proto(self):
        return self._graph_proto if self._compiled else None

    def debug(self, v_level=-1, *, ranks=None, max_py_stack_depth=2, only_user_py_stack=True, op_repr_with_py_stack=False):
        self._debug_level, self._debug_ranks = v_level, ranks
        from ...framework import boxing
        me = dist.get_rank() if dist.is_initialized() else 0
        boxing.debug_routes = v_level >= 1 and (ranks is None or me in (ranks if isinstance(ranks, (list, tuple)) else [ranks]))

    @classmethod
    def trace(cls, func):
        """Wraps a plain function as a graph (inference): ``g = Graph.trace(f); g(x)``."""
        class _Traced(Graph):
            def build(self, *a, **k):
                return func(*a, **k)
        return _Traced()

    # ------------------------------------------------------------------ state
    def state_dict(self, destination=None):
        sd = destination if destination is not None else OrderedDict()
        for name, proxy in self._blocks.items():
            sd[name] = proxy._module.state_dict()
        for i, o in enumerate(self._opts):
            opt = o["optim"]
            sd[f"System-Optimizer-{i}"] = opt.state_dict()
            if o.get("flat") is not None:
                sd[f"System-FlatOptimizer-{i}"] = o["flat"].state_dict()
            if o["lr_sch"] is not None:
                sd[f"System-LRScheduler-{i}"] = o["lr_sch"].state_dict()
        if self._grad_scaler is not None and hasattr(self._grad_scaler, "state_dict"):
            sd["System-GradScaler"] = self._grad_scaler.state_dict()
        sd["System-Train-TrainStep"] = torch.tensor([self._train_step], dtype=torch.int64)
        return sd

    def load_state_dict(self, state_dict, strict=True):
        for name, proxy in self._blocks.items():
            if name in state_dict:
                proxy._module.load_state_dict(state_dict[name], strict=strict)
            elif strict:
                raise KeyError(f"missing block {name} in state dict")
        for i, o in enumerate(self._opts):
            k = f"System-Optimizer-{i}"
            if k in state_dict:
                o["optim"].load_state_dict(state_dict[k])
            k = f"System-FlatOptimizer-{i}"
            if k in state_dict and o.get("flat") is not None:
                o["flat"].load_state_dict(state_dict[k])
            k = f"System-LRScheduler-{i}"
            if k in state_dict and o["lr_sch"] is not None:
                o["lr_sch"].load_state_dict(state_dict[k])
        if "System-GradScaler" in state_dict and self._grad_scaler is not None:
            self._grad_scaler.load_state_dict(state_dict["System-GradScaler"])
        ts = state_dict.get("System-Train-TrainStep")
        if ts is not None:
            self._train_step = int(torch.as_tensor(ts).reshape(-1)[0])

    def runtime_state_dict(self, destination=None):
        """State needed to run without re-compiling: there is no compiled plan to cache here, so this is
        the ordinary state dict plus the recorded input meta."""
        sd = self.state_dict(destination)
        sd["System-InputMeta"] = self._input_meta
        sd["System-Plan"] = self._plan
        return sd

    def load_runtime_state_dict(self, state_dict, *, warmup_with_run=True):
        self._input_meta = state_dict.get("System-InputMeta")
        self.load_state_dict({k: v for k, v in state_dict.items() if k not in ("System-InputMeta", "System-Plan")}, strict=False)

    # ------------------------------------------------------------------ compile
    def _all_params(self):
        seen, out = set(), []
        for o in self._opts:
            for g in o["optim"].param_groups:
                for p in g["params"]:
                    if id(p) not in seen:
                        seen.add(id(p))
                        out.append(p)
        return out

    def _apply_zero(self):
        """B parameters become S(0) shards on the first mesh axis whose size divides dim 0 (ZeRO): the
        optimizer states created from them are sharded alike, gradients arrive by reduce-scatter and the
        consumers all-gather on use."""
        if self.config.zero_stage <= 0:
            return
        flat_ids = {id(sl.param) for f in getattr(self, "_flat", []) for sl in f.slots}
        for p in self._all_params():
            if id(p) in flat_ids:
                continue          # sharded inside the flat optimizer state
            if not isinstance(p, GT.GlobalTensor):
                continue
            if p.numel() < self.config.zero_shard_min_size:
                continue
            nd = list(p.sbp)
            for axis, s in enumerate(nd):
                n = p.placement.hierarchy[axis]
                if s.kind == "B" and n > 1 and p.dim() > 0 and p.shape[0] % n == 0 and \
                        not any(o.kind == "S" and o.axis == 0 for o in nd):
                    nd[axis] = S.split(0)
                    break
            if tuple(nd) != p.sbp:
                new = GT.rebox(p.detach(), nd)
                p._local, p._nd_sbp = new._local, new._nd_sbp

    def _build_flat_optimizers(self):
        """Optimizer generation at compile time: Adam / AdamW / SGD whose parameters are bf16 CUDA tensors (or any
        parameters with ``config.enable_multi_tensor_update``) run as flat fused buffers (nn/graph/flat_optim.py); their
        ZeRO sharding happens inside that state, over the data-parallel axis found at the first step."""
        from ...optim import optimizer as O
        from .flat_optim import FlatOptimizer
        self._flat = []
        for o in self._opts:
            opt = o["optim"]
            o["flat"] = None
            if not isinstance(opt, (O._AdamFamily, O.SGD)) or o["is_sparse"]:
                continue
            if any(g.get("amsgrad") for g in opt.param_groups):
                continue
            ps = [p for g in opt.param_groups for p in g["params"] if p.requires_grad]
            locs = [p._local if isinstance(p, GT.GlobalTensor) else p for p in ps]
            locs = [t for t in locs if t is not None and t.numel()]
            if not locs:
                continue
            auto = all(t.is_cuda and t.dtype == torch.bfloat16 for t in locs)
            if not (auto or self.config.multi_tensor_update):
                continue
            if len({(t.device, t.dtype) for t in locs}) != 1 or not locs[0].dtype.is_floating_point:
                continue
            f = FlatOptimizer(opt, zero_stage=self.config.zero_stage)
            o["flat"] = f
            self._flat.append(f)

    def _apply_auto_parallel(self, args):
        """``config.enable_auto_parallel``: the Linear layers whose weights are still fully broadcast on a 1-D placement
        get the SBP signatures that the chain solver of framework/auto_parallel.py finds cheapest (data, column or row
        parallel); the dispatch rules insert the boxing between them."""
        if not self.config.auto_parallel:
            return
        from ...framework import auto_parallel as AP
        tokens = None
        for a in args:
            if isinstance(a, GT.GlobalTensor) and a.dim() >= 2:
                tokens = int(a.numel() // a.shape[-1])
                break
        if tokens is None:
            return
        specs, mods = [], {}
        for blk in self._blocks.values():
            root = blk.origin if hasattr(blk, "origin") else blk
            if not isinstance(root, torch.nn.Module):
                continue
            for name, m in root.named_modules():
                w = getattr(m, "weight", None)
                if isinstance(m, torch.nn.Linear) and isinstance(w, GT.GlobalTensor) and len(w.placement.hierarchy) == 1 and \
                        w.placement.hierarchy[0] > 1 and all(s_.kind == "B" for s_ in w.sbp):
                    key = f"{id(root)}.{name}"
                    specs.append(AP.LinearSpec(key, m.in_features, m.out_features, tokens, w.element_size()))
                    mods[key] = m
        if not specs:
            return
        world = next(iter(mods.values())).weight.placement.hierarchy[0]
        ratio = float(self.config.extra.get("auto_parallel_computation_cost_ratio", 1.0) or 1.0)
        choices = AP.solve_chain(specs, world, flops_per_s=1.4e15 / max(ratio, 1e-6))
        for c in choices:
            m = mods[c.name]
            if c.kind == "data":
                continue
            w = m.weight
            new = GT.rebox(w.detach(), [S.split(0) if c.kind == "column" else S.split(1)])
            w._local, w._nd_sbp = new._local, new._nd_sbp
            if m.bias is not None and c.kind == "column":
                nb = GT.rebox(m.bias.detach(), [S.split(0)])
                m.bias._local, m.bias._nd_sbp = nb._local, nb._nd_sbp
        self._auto_parallel_choices = [(c.name.split(".", 1)[1], c.kind) for c in choices]

    def _filter_states(self):
        """Names of the graph's state tensors (parameters and buffers of its blocks, each tensor once), in block
        order (reference: python/oneflow/nn/graph/graph.py:716-741)."""
        seen, names = set(), []
        for bname, proxy in self._blocks.items():
            mod = proxy._module
            for kind in (mod.named_parameters(), mod.named_buffers()):
                for n, t in kind:
                    if id(t) not in seen:
                        seen.add(id(t))
                        names.append(f"{bname}.{n}")
        self._eager_state_op_names = list(names)
        return names

    def _generate_config_proto(self):
        """Fills ``self.config.proto``: the job configuration with one entry per optimizer (its parameter groups,
        update rule and learning-rate schedule), as the reference hands to its compiler."""
        state = getattr(self, "_eager_state_op_names", None) or self._filter_states()
        by_id = {}
        for bname, proxy in self._blocks.items():
            for n, t in proxy._module.named_parameters():
                by_id.setdefault(id(t), f"{bname}.{n}")
        opts = []
        for o in self._opts:
            opt, sch = o["optim"], o["lr_sch"]
            groups = []
            for g in opt.param_groups:
                conf = {k: v for k, v in g.items() if k != "params" and isinstance(v, (int, float, bool, str, tuple, type(None)))}
                conf["variable_op_names"] = [by_id.get(id(p), "<unnamed>") for p in g["params"] if p.requires_grad]
                groups.append(conf)
            opts.append({"type": type(opt).__name__, "param_groups": groups, "is_sparse": o["is_sparse"],
                         "lr_scheduler": None if sch is None else type(sch).__name__})
        self.config._proto = dict(self.config._as_dict(), job_name=self._name, state_op_names=state, optimizer_conf=opts)
        return self.config._proto

    def _compile(self, *args):
        if len(args) == 1 and isinstance(args[0], tuple):
            args = args[0]
        self._generate_config_proto()
        if Graph._nesting > 0:
            raise RuntimeError("nn.Graph objects cannot be nested")
        shared = getattr(self, "_shared_graph", None)
        if shared is not None and getattr(shared, "_auto_parallel_choices", None) is not None and not self.config.auto_parallel:
            self._auto_parallel_choices = list(shared._auto_parallel_choices)
        self._apply_auto_parallel(args)
        self._build_flat_optimizers()
        self._apply_zero()
        self._compiled = True
        if self._pending_state is not None:
            self.load_state_dict(self._pending_state)
            self._pending_state = None

    @staticmethod
    def _meta(a):
        if isinstance(a, GT.GlobalTensor):
            return ("g", tuple(a.shape), a.dtype, a.placement, a.sbp)
        if isinstance(a, torch.Tensor):
            return ("l", tuple(a.shape), a.dtype, a.device.type)
        return ("o", type(a))

    # ------------------------------------------------------------------ run
    def __call__(self, *args, **kwargs):
        if not self._compiled:
            self._compile(args)
            self._input_meta = [self._meta(a) for a in args]
        elif getattr(self, "_dynamic_metas", None) is not None:
            key = tuple(self._meta(a) for a in args)
            self._dynamic_metas[key] = True
            self._dynamic_metas.move_to_end(key)
            while len(self._dynamic_metas) > self._dynamic_cache_size:
                self._dynamic_metas.popitem(last=False)
        else:
            meta = [self._meta(a) for a in args]
            # ONEFLOW_RUN_GRAPH_BY_VM=1: the graph is replayed op by op, so any input signature is accepted
            by_vm = os.getenv("ONEFLOW_RUN_GRAPH_BY_VM") == "1"
            if self._input_meta is not None and meta != self._input_meta and not by_vm:
                raise RuntimeError(f"nn.Graph {self._name}: inputs must keep the same shape/dtype/placement/sbp on every call "
                                   f"(first call {self._input_meta}, now {meta})")
        try:
            return self._run(self._shield_inputs(args), kwargs)
        finally:
            probe = self.__dict__.pop("_probe", None)
            if probe is not None:
                self._written_inputs = {i for i, t, v in probe if t._version != v}

    def _shield_inputs(self, args):
        """In-place operations inside ``build`` must not reach the caller's tensors (a graph works on its own
        copies of the inputs). The first call runs on clones of all local tensor inputs and notes which of them
        ``build`` wrote to; later calls clone only those."""
        local = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor) and not isinstance(a, GT.GlobalTensor)]
        known = getattr(self, "_written_inputs", None)
        if known is None:
            out = list(args)
            for i in local:
                out[i] = args[i].clone()
            self._probe = [(i, out[i], out[i]._version) for i in local]
            return tuple(out)
        if not known:
            return args
        out = list(args)
        for i in known:
            if i < len(out) and isinstance(out[i], torch.Tensor) and not isinstance(out[i], GT.GlobalTensor):
                out[i] = out[i].clone()
        return tuple(out)

    @contextlib.contextmanager
    def _backward_scaling(self, factor_fn):
        """Inside build(), ``loss.backward()`` applies the gradient-accumulation average and the loss scale. While a
        pipeline schedule runs, the call is recorded instead and executed when the schedule reaches that micro-batch's
        backward slot."""
        orig = torch.Tensor.backward
        graph = self

        def backward(t, gradient=None, *a, **k):
            f = factor_fn()
            if f != 1.0:
                if gradient is None:
                    if t.numel() != 1:
                        raise RuntimeError("only a scalar loss may call backward() inside nn.Graph.build")
                    gradient = torch.ones_like(t) * f
                else:
                    gradient = gradient * f
            pending = graph.__dict__.get("_pending_backward")
            if pending is not None:
                pending.append((t, gradient, a, k))
                return None
            return orig(t, gradient, *a, **k)
        torch.Tensor.backward = backward
        self.__dict__["_orig_backward"] = orig
        try:
            yield
        finally:
            torch.Tensor.backward = orig

    # ------------------------------------------------------------------ plan
    def _stage_layout(self):
        """(number of pipeline stages, this rank's stage index or None, stage placements): stages are the distinct
        ``set_stage`` placements in stage-id order. A rank that belongs to several stages (or to none) gets no
        pipeline schedule: its micro-batches run one after the other."""
        stages = {}
        for proxy in self._blocks.values():
            for p in proxy._walk():
                gm = p._gm
                if gm.stage_placement is not None:
                    stages.setdefault(gm.stage_id if gm.stage_id is not None else len(stages), gm.stage_placement)
        if len(stages) < 2:
            return 1, 0, []
        order = [stages[k] for k in sorted(stages)]
        me = GT._rank()
        mine = [i for i, pl in enumerate(order) if pl.contains(me)]
        return len(order), (mine[0] if len(mine) == 1 else None), order

    def _record_plan(self, trace):
        """The per-rank execution plan built from the first call: pipeline stages with their blocks, the fused
        products and boxing steps each micro-batch issues here (in order), the flat optimizer buffers. It is what
        ``runtime_state_dict`` carries and what ``debug`` / ``repr`` print; the stage table also drives the schedule."""
        n_stages, my_stage, order = self._stage_layout()
        blocks = []
        for name, proxy in self._blocks.items():
            for p in proxy._walk():
                gm = p._gm
                if gm.stage_id is not None or gm.activation_checkpointing:
                    blocks.append({"block": p._name, "stage_id": gm.stage_id,
                                   "placement": None if gm.stage_placement is None else list(gm.stage_placement.ranks_flat),
                                   "activation_checkpointing": gm.activation_checkpointing,
                                   "runs_here": gm.stage_placement is None or gm.stage_placement.contains(GT._rank())})
        ops = [{"op": n, **d} for n, d in (trace or [])]
        flat = [{"optimizer": type(f.optim).__name__, "elements": f.total, "dtype": str(getattr(f, "dtype", None)),
                 "zero_stage": f.zero_stage} for f in self._flat]
        self._plan = {"rank": GT._rank(), "stages": n_stages, "stage_of_rank": my_stage,
                      "schedule": "1F1B" if (n_stages > 1 and my_stage is not None) else "sequential",
                      "micro_batches": self.config.grad_acc_steps if self.config.training else 1,
                      "blocks": blocks, "fused_ops_per_micro_batch": ops, "flat_optimizers": flat}
        return self._plan

    # ------------------------------------------------------------------ run
    def _run(self, args, kwargs):
        cfg = self.config
        n = cfg.grad_acc_steps if cfg.training else 1
        micro_args = _unpack(args, n)
        scaler = self._grad_scaler
        loss_scale = float(scaler.get_scale()) if scaler is not None and hasattr(scaler, "get_scale") else 1.0
        outs = [None] * n
        first_call = self.__dict__.get("_plan") is None
        from ...framework import fused_ops
        trace = [] if first_call else None
        Graph._nesting += 1
        try:
            ctx = contextlib.nullcontext()
            if cfg.amp_enabled:
                dev = "cuda" if any(isinstance(a, torch.Tensor) and a.device.type == "cuda" for a in args) else "cpu"
                ctx = torch.autocast(dev, dtype=cfg.amp_dtype if dev == "cuda" or cfg.amp_dtype == torch.bfloat16 else torch.bfloat16)
            grad_ctx = contextlib.nullcontext() if cfg.training else torch.no_grad()
            n_stages, my_stage, _ = self._stage_layout()
            pipelined = cfg.training and n_stages > 1 and my_stage is not None and n > 1
            with ctx, grad_ctx, self._backward_scaling(lambda: loss_scale / n):
                if not pipelined and self._captured_ready(args, kwargs, first_call):
                    for m in range(n):
                        outs[m] = self._replay_captured(micro_args[m])
                elif not pipelined:
                    for m in range(n):
                        fused_ops.op_trace = trace if m == 0 else None
                        outs[m] = self.build(*micro_args[m], **kwargs)
                else:
                    self._run_1f1b(micro_args, kwargs, outs, n_stages, my_stage, trace)
        finally:
            Graph._nesting -= 1
            fused_ops.op_trace = None
            self.__dict__["_pending_backward"] = None
        if cfg.training:
            self._optimizer_step(loss_scale)
        if first_call:
            self._record_plan(trace)
        return _pack(outs)

    # ------------------------------------------------------------------ captured micro-batch (config.enable_cuda_graph)
    def _captured_ready(self, args, kwargs, first_call):
        """``config.enable_cuda_graph``: after the first (eager, plan-recording) call the forward + backward of ONE
        micro-batch is captured into a CUDA graph and every later micro-batch is a replay of it on fresh inputs (the
        reference captures its kernels per stream: oneflow/core/ep/cuda/cuda_stream.h:70-120,
        oneflow/core/kernel/cuda_graph_support.h:29-34). Conditions: one process (kernels that talk to peers take their
        call number by value), CUDA inputs, every trainable parameter in a flat optimizer buffer (gradients then
        accumulate in place in static memory). Anything else raises, so the switch never silently does nothing."""
        if not self.config.cuda_graph or first_call:
            return False
        if self.__dict__.get("_cg") is not None:
            return True
        if self.__dict__.get("_cg_failed"):
            return False
        if dist.is_initialized() and dist.get_world_size() > 1:
            raise NotImplementedError("config.enable_cuda_graph: capture is limited to single-process graphs (the fused "
                                      "collectives take their call number by value)")
        if kwargs or not any(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
            raise NotImplementedError("config.enable_cuda_graph needs positional CUDA tensor inputs")
        flat_ids = {id(sl.param) for f in self._flat for sl in f.slots}
        if self.config.training and any(id(p) not in flat_ids for p in self._all_params() if p.requires_grad):
            raise NotImplementedError("config.enable_cuda_graph needs all trainable parameters in a fused (flat) optimizer")
        return self._capture(args)

    def _capture(self, args):
        n = self.config.grad_acc_steps if self.config.training else 1
        sample = _unpack(args, n)[0]

        def static_copy(a):
            if isinstance(a, GT.GlobalTensor):
                return GT.wrap(a._local.clone(), a.shape, a.placement, a.sbp)
            return a.clone() if isinstance(a, torch.Tensor) else a
        static_args = tuple(static_copy(a) for a in sample)
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self.build(*static_args)
        except Exception as e:           # an op on the path cannot be captured: say so once and stay eager
            import warnings
            torch.cuda.synchronize()
            self.__dict__["_cg_failed"] = True
            warnings.warn(f"nn.Graph {self._name}: CUDA-graph capture failed ({type(e).__name__}: {e}); running eagerly")
            return False
        # the capture only recorded the kernels: it did not run them, so nothing was accumulated yet
        self.__dict__["_cg"] = (g, static_args, out)
        if self._plan is not None:
            self._plan["captured_micro_batch"] = True
        return True

    def _replay_captured(self, margs):
        g, static_args, out = self._cg
        for s, a in zip(static_args, margs):
            if isinstance(s, GT.GlobalTensor):
                s._local.copy_(a._local)
            elif isinstance(s, torch.Tensor):
                s.copy_(a)
        g.replay()
        from torch.utils import _pytree as pytree
        return pytree.tree_map(lambda t: t.detach().clone() if isinstance(t, torch.Tensor) else t, out)

    def _run_1f1b(self, micro_args, kwargs, outs, n_stages, my_stage, trace):
        """One-forward-one-backward order over the micro-batches for this rank's stage (reference: the stage buffers
        of pipeline_buffer_pass.cpp:44-110 let stage s run ``n_stages - s - 1`` forwards ahead of its backwards).
        ``build`` runs once per micro-batch; its ``backward()`` call is held back until the schedule's backward slot.
        Activations and their gradients cross stages inside the stage-boundary ``to_global`` (asynchronous sends on
        the p2p communicator's own stream, the compute stream only waits for what it receives)."""
        from ...framework import fused_ops
        n = len(micro_args)
        orig = self.__dict__["_orig_backward"]
        warm = min(n_stages - my_stage - 1, n)
        queue = []

        def fwd(m):
            self.__dict__["_pending_backward"] = pend = []
            fused_ops.op_trace = trace if m == 0 else None
            outs[m] = self.build(*micro_args[m], **kwargs)
            fused_ops.op_trace = None
            self.__dict__["_pending_backward"] = None
            queue.append(pend)

        def bwd():
            for t, gradient, a, k in queue.pop(0):
                orig(t, gradient, *a, **k)
        for m in range(warm):
            fwd(m)
        for m in range(warm, n):
            fwd(m)
            bwd()
        while queue:
            bwd()

    def _optimizer_step(self, loss_scale):
        scaler = self._grad_scaler
        found_inf = False
        dynamic = scaler is not None and getattr(scaler, "dynamic", False)
        flat_ids = set()
        for f in self._flat:
            flat_ids.update(id(s.param) for s in f.slots)
        params = [p for p in self._all_params() if id(p) not in flat_ids]
        if loss_scale != 1.0:
            inv = 1.0 / loss_scale
            for p in params:
                if p.grad is not None:
                    p.grad.mul_(inv)
        if dynamic:
            # one not-finite count over every local gradient, one read
            grads = [(p.grad._local if isinstance(p.grad, GT.GlobalTensor) else p.grad) for p in params if p.grad is not None]
            grads = [g.reshape(-1) for g in grads if g is not None and g.numel()]
            grads += [f.grad for f in self._flat if f.total]
            bad = torch.zeros((), dtype=torch.float32, device=grads[0].device if grads else "cpu")
            if grads:
                dev_groups = {}
                for g in grads:
                    dev_groups.setdefault((g.device, g.dtype), []).append(g)
                for (_dev, _dt), gs in dev_groups.items():
                    if gs[0].is_cuda and gs[0].dtype in (torch.float32, torch.bfloat16):
                        from ...ops import kernels as K
                        bad = bad + K.multi_tensor_sqsum(gs)[1].to(bad.device)
                    else:
                        bad = bad + sum((~torch.isfinite(g)).sum() for g in gs).to(bad.device, torch.float32)
            if dist.is_initialized():
                dist.all_reduce(bad)
            found_inf = bool(bad.item() > 0)
            scaler.update(found_inf)
        if not found_inf:
            for f in self._flat:
                f.step(loss_scale)
            for o in self._opts:
                opt = o["optim"]
                if o.get("flat") is not None:
                    continue
                if hasattr(opt, "clip_grad"):
                    opt.clip_grad()
                scaled = [(g, g["lr"]) for g in opt.param_groups if g.get("lr_scale", 1.0) != 1.0]
                for g, lr in scaled:                      # per-group ``lr_scale`` takes effect in graph mode
                    g["lr"] = lr * g["lr_scale"]
                try:
                    opt.step()
                finally:
                    for g, lr in scaled:
                        g["lr"] = lr
        if os.getenv("ONEFLOW_DEBUG_MODE"):
            self._log_step_lr()
        for f in self._flat:
            f.zero_grad()
        for o in self._opts:
            if o.get("flat") is None:
                o["optim"].zero_grad(set_to_none=True)
            if o["lr_sch"] is not None and not found_inf:
                o["lr_sch"].step()
        self._train_step += 1

    def _log_step_lr(self):
        """Debug mode keeps ``log/local/<pid>-train_step2lr.csv``: one ``train_step, lr`` line per step (the first
        optimizer's first group), as the reference's runtime writes."""
        path = os.path.join("log", "local", f"{os.getpid()}-train_step2lr.csv")
        if self._opts:
            os.makedirs(os.path.dirname(path), exist_ok=True)
            fresh = not getattr(self, "_lr_log_started", False)
            with open(path, "w" if fresh else "a") as f:
                if fresh:
                    f.write("train_step, lr\n")
                    self._lr_log_started = True
                f.write(f"{self._train_step}, {self._opts[0]['optim'].param_groups[0]['lr']}\n")

    def __repr__(self):
        lines = [f"(GRAPH:{self._name}:{type(self).__name__}): ("]
        for name, proxy in self._blocks.items():
            gm = proxy._gm
            extra = f", stage_id={gm.stage_id}, placement={gm.stage_placement}" if gm.stage_id is not None else ""
            lines.append(f"  (MODULE:{name}:{type(proxy._module).__name__}{extra})")
        lines.append(f"  (CONFIG: training={self.config.training}, amp={self.config.amp_enabled}, "
                     f"zero={self.config.zero_stage}, grad_acc={self.config.grad_acc_steps})")
        lines.append(")")
        return "\n".join(lines)


def _unpack(args, n):
    """dim-0 unpack of every tensor argument into n micro-batches."""
    if n == 1:
        return [args]
    out = [[] for _ in range(n)]
    for a in args:
        if isinstance(a, torch.Tensor) and a.dim() > 0:
            if a.shape[0] % n:
                raise ValueError(f"batch dimension {a.shape[0]} is not divisible by the {n} gradient accumulation steps")
            if isinstance(a, GT.GlobalTensor) and all(sb.kind == "B" or (sb.kind == "S" and sb.axis == 0) for sb in a.sbp) and \
                    (not a.placement.contains(GT._rank()) or a._local.shape[0] % n == 0):
                # every rank cuts its own shard: no traffic (with a split batch axis a micro-batch is then a strided
                # selection of the global batch, which training does not care about)
                m = a.shape[0] // n
                shape = (m,) + tuple(a.shape[1:])
                if a.placement.contains(GT._rank()):
                    pieces = [GT.wrap(c, shape, a.placement, a.sbp) for c in a._local.chunk(n, 0)]
                else:
                    pieces = [GT.wrap(a._local, shape, a.placement, a.sbp) for _ in range(n)]
            elif isinstance(a, GT.GlobalTensor):
                m = a.shape[0] // n
                pieces = [a[i * m:(i + 1) * m] for i in range(n)]
                # keep the original layout for every micro-batch
                pieces = [GT.to_global(p, a.placement, a.sbp) for p in pieces]
            else:
                pieces = list(a.chunk(n, 0))
            for i in range(n):
                out[i].append(pieces[i])
        else:
            for i in range(n):
                out[i].append(a)
    return [tuple(o) for o in out]


def _pack(outs):
    if len(outs) == 1:
        return outs[0]
    first = outs[0]
    if isinstance(first, torch.Tensor):
        dets = [o.detach() for o in outs]
        return torch.stack(dets) if first.dim() == 0 else torch.cat(dets, 0)
    if isinstance(first, (tuple, list)):
        return type(first)(_pack([o[i] for o in outs]) for i in range(len(first)))
    if isinstance(first, dict):
        return {k: _pack([o[k] for o in outs]) for k in first}
    return outs
