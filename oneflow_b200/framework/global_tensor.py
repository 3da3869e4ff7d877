"""Global tensors: (logical shape, placement, n-D SBP) over per-rank local shards.

``GlobalTensor`` is a ``torch.Tensor`` wrapper subclass. Every ATen operator that reaches it goes through
``__torch_dispatch__``: an SBP rule for the operator picks the signature (which input layouts the local
kernel needs and which layout the output gets), inputs whose SBP differs are boxed
(framework/boxing.py), the operator runs on the local shards, and the result is wrapped again. Autograd
runs above this level, so backward formulas dispatch through the same rules: gradients of broadcast
parameters naturally come out as partial-sum (``P``) tensors that are boxed to ``B`` when a consumer
needs it, exactly the data-parallel / tensor-parallel behaviour of the reference
(EagerGlobalInterpreter::Interpret, oneflow/core/framework/op_interpreter/eager_global_op_interpreter.cpp:174-293;
signature choice oneflow/core/operator/operator.cpp:609-663; per-op GetSbp in oneflow/user/ops/*).

Operators without a dedicated rule fall back to the always-valid all-broadcast signature.
Ranks outside a tensor's placement hold an empty placeholder and skip the local computation.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.distributed as dist
from torch.utils import _pytree as pytree

from .. import sbp as S
from . import boxing
from .nd_sbp import copy_cost, local_shape
from .placement import placement as Placement

aten = torch.ops.aten
B, P = S.broadcast, S.partial_sum


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def _contig_strides(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(st))


class GlobalTensor(torch.Tensor):
    _placement: Placement
    _nd_sbp: tuple

    # The local shard. A row-parallel product may hand out a tensor whose shard is still a thunk (a partial sum that
    # nobody has asked for yet, see framework/fused_ops.DeferredPartial): reading ``_local`` then runs the plain GEMM,
    # while a boxing step that wants the reduced rows asks the thunk for the fused GEMM->reduce-scatter instead.
    @property
    def _local(self):
        d = self.__dict__
        loc = d.get("_loc")
        if loc is None:
            th = d.get("_thunk")
            if th is not None:
                loc = th.materialize()
                view = d.get("_thunk_view")
                if view is not None:
                    loc = loc.view(view)
                d["_loc"], d["_thunk"] = loc, None
        return loc

    @_local.setter
    def _local(self, value):
        d = self.__dict__
        d["_loc"] = value
        d["_thunk"] = None

    @staticmethod
    def __new__(cls, local, logical_shape, placement, nd_sbp, requires_grad=False):
        shape = tuple(int(s) for s in logical_shape)
        r = torch.Tensor._make_wrapper_subclass(cls, shape, strides=_contig_strides(shape), dtype=local.dtype,
                                                device=local.device, layout=local.layout, requires_grad=requires_grad)
        r._local = local
        r._placement = placement
        r._nd_sbp = tuple(nd_sbp)
        return r

    def __init__(self, *a, **k):
        pass

    # ---- reference-compatible attributes
    @property
    def is_global(self):
        return True

    @property
    def is_local(self):
        return False

    @property
    def placement(self):
        return self._placement

    @property
    def sbp(self):
        return self._nd_sbp

    def to_local(self, copy=False):
        return to_local(self, copy=copy)

    def to_global(self, placement=None, sbp=None, **kw):
        return to_global(self, placement, sbp, **kw)

    def numpy(self):
        return to_global(self.detach(), self._placement, (B,) * self._placement.ndim)._local.cpu().numpy()

    def tolist(self):
        return self.numpy().tolist()

    def new(self, *args, **kwargs):
        """``x.new()`` / ``x.new(*sizes)`` / ``x.new(data)``: a new tensor of this tensor's dtype, placement and sbp."""
        from . import tensor_api
        if len(args) == 1 and not isinstance(args[0], (int, torch.Size)):
            return tensor_api.tensor(args[0], dtype=self.dtype, placement=self._placement, sbp=self._nd_sbp)
        size = tuple(args[0]) if len(args) == 1 and isinstance(args[0], torch.Size) else tuple(args)
        size = size if size else (0,)
        return tensor_api.empty(size, dtype=self.dtype, placement=self._placement, sbp=self._safe_sbp(size))

    def _safe_sbp(self, size):
        """This tensor's sbp where it fits a tensor of ``size``; axes that cannot be split there are broadcast."""
        return tuple(s if s.kind != "S" or (s.axis < len(size) and size[s.axis] >= self._placement.hierarchy[i]) else B
                     for i, s in enumerate(self._nd_sbp))

    def contiguous(self, memory_format=torch.contiguous_format):
        """The logical tensor always reads as contiguous; what matters to kernels is the local shard, so a shard
        that is a strided view (after ``transpose`` / ``permute``) is copied into dense memory here."""
        if self._local.is_contiguous(memory_format=memory_format):
            return self
        return self.clone(memory_format=memory_format)

    def type_as(self, other):
        if isinstance(other, GlobalTensor):
            return self.to(other.dtype)
        return self.to_local().to(device=other.device, dtype=other.dtype)

    def __repr__(self):
        return (f"GlobalTensor(shape={tuple(self.shape)}, dtype={self.dtype}, placement={self._placement}, "
                f"sbp={tuple(str(s) for s in self._nd_sbp)}, local_shape={tuple(self._local.shape)})")

    def __reduce_ex__(self, proto):
        from .check_point import reduce_tensor
        return reduce_tensor(self)

    __torch_function__ = torch._C._disabled_torch_function_impl

    # matmul with a 1-D operand: torch finishes that case with an in-place ``squeeze_``, which cannot change the logical
    # shape a wrapper tensor was built with, so the method spellings (and ``flow.matmul``) use out-of-place squeezes
    def matmul(self, other):
        return matmul_any(self, other)

    def __matmul__(self, other):
        return matmul_any(self, other)

    def __rmatmul__(self, other):
        return matmul_any(other, self)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        return dispatch(func, args, kwargs or {})


def matmul_any(a, b):
    """``a @ b`` for any ranks, global or local operands."""
    if a.dim() == 1 or b.dim() == 1:
        out = torch.matmul(a.unsqueeze(0) if a.dim() == 1 else a, b.unsqueeze(-1) if b.dim() == 1 else b)
        if b.dim() == 1:
            out = out.squeeze(-1)
        if a.dim() == 1:
            out = out.squeeze(-1 if b.dim() == 1 else -2)
        return out
    return torch.matmul(a, b)


def is_global(x):
    return isinstance(x, GlobalTensor)


# ------------------------------------------------------------------------------------------------ helpers
def _in_placement(pl):
    return pl.contains(_rank())


def _coords(pl):
    return pl.coords(_rank())


def wrap(local, logical_shape, pl, nd, requires_grad=False):
    return GlobalTensor(local, logical_shape, pl, nd, requires_grad=requires_grad)


def wrap_deferred(thunk, local_view, logical_shape, dtype, device, pl, nd):
    """A global tensor whose local shard is computed on first use by ``thunk`` (``materialize`` / ``reduce_scatter``)."""
    g = GlobalTensor(torch.empty((0,), dtype=dtype, device=device), logical_shape, pl, nd)
    d = g.__dict__
    d["_loc"], d["_thunk"], d["_thunk_view"] = None, thunk, tuple(local_view)
    return g


def rebox(x: GlobalTensor, nd) -> GlobalTensor:
    nd = tuple(nd)
    if nd == x._nd_sbp:
        return x
    if x.__dict__.get("_thunk") is not None:
        from .fused_ops import take_deferred_reduce_scatter
        local = take_deferred_reduce_scatter(x, nd)
        if local is not None:
            return wrap(local, x.shape, x._placement, nd)
    local = boxing.convert_same_placement(x._local, tuple(x.shape), x._placement, x._nd_sbp, nd)
    return wrap(local, x.shape, x._placement, nd)


def _meta_of(x):
    if isinstance(x, GlobalTensor):
        return torch.empty(tuple(x.shape), dtype=x.dtype, device="meta")
    return x


def _local_of(x):
    return x._local if isinstance(x, GlobalTensor) else x


def _meta_of_any(x):
    if isinstance(x, GlobalTensor):
        return torch.empty(tuple(x.shape), dtype=x.dtype, device="meta")
    if isinstance(x, torch.Tensor) and x.dim() > 0:
        return torch.empty(tuple(x.shape), dtype=x.dtype, device="meta")
    return x


def _infer_meta(func, args, kwargs):
    """Output meta (shape / dtype) of ``func`` on the logical shapes.  Local tensor operands next to global ones stay
    real at first (their values may matter, e.g. 0-dim scalars); when the op then complains about mixed devices they
    become meta tensors as well."""
    margs, mkwargs = pytree.tree_map(_meta_of, (args, kwargs))
    try:
        return func(*margs, **mkwargs)
    except RuntimeError as e:
        if "meta" not in str(e):
            raise
        margs, mkwargs = pytree.tree_map(_meta_of_any, (args, kwargs))
        return func(*margs, **mkwargs)


def _placeholder(meta, pl, nd):
    dev = pl.device()
    return wrap(torch.empty((0,), dtype=meta.dtype, device=dev), meta.shape, pl, nd)


def _finish(func, args, kwargs, pl, out_nds, local_args=None, local_kwargs=None, meta_out=None, shapes_from_result=False):
    """Runs func on the local shards and wraps the outputs. out_nds: one nd-sbp per tensor output (a single
    nd-sbp is applied to every output).  ``shapes_from_result``: every input is broadcast, so the local result IS the
    logical result and its shapes are taken from it — no shape inference on meta tensors, which data-dependent ops
    (nonzero, unique, masked_select, bincount) and ops reading values do not support."""
    if shapes_from_result and _in_placement(pl):
        if local_args is None:
            local_args, local_kwargs = pytree.tree_map(_local_of, (args, kwargs))
        res = func(*local_args, **(local_kwargs or {}))
        flat, spec = pytree.tree_flatten(res)
        nd = tuple(out_nds[0]) if out_nds and isinstance(out_nds[0], (tuple, list)) else tuple(out_nds)
        outs = [wrap(t, t.shape, pl, nd) if isinstance(t, torch.Tensor) else t for t in flat]
        return pytree.tree_unflatten(outs, spec)
    if meta_out is None:
        meta_out = _infer_meta(func, args, kwargs)
    metas, spec = pytree.tree_flatten(meta_out)
    tensor_idx = [i for i, m in enumerate(metas) if isinstance(m, torch.Tensor)]
    if out_nds and not isinstance(out_nds[0], (tuple, list)):
        out_nds = [tuple(out_nds)] * len(tensor_idx)
    elif len(out_nds) == 1 and len(tensor_idx) > 1:
        out_nds = [tuple(out_nds[0])] * len(tensor_idx)       # one nd-sbp given for an op with several outputs
    if not _in_placement(pl):
        outs = list(metas)
        for k, i in enumerate(tensor_idx):
            outs[i] = _placeholder(metas[i], pl, out_nds[k])
        return pytree.tree_unflatten(outs, spec)
    if local_args is None:
        local_args, local_kwargs = pytree.tree_map(_local_of, (args, kwargs))
    res = func(*local_args, **(local_kwargs or {}))
    flat, _ = pytree.tree_flatten(res)
    outs = list(flat)
    for k, i in enumerate(tensor_idx):
        if isinstance(flat[i], torch.Tensor):
            outs[i] = wrap(flat[i], metas[i].shape, pl, out_nds[k])
    return pytree.tree_unflatten(outs, spec)


def _globals(args, kwargs):
    flat, _ = pytree.tree_flatten((args, kwargs))
    return [a for a in flat if isinstance(a, GlobalTensor)]


def _common_placement(gs):
    pl = gs[0]._placement
    for g in gs[1:]:
        if g._placement != pl:
            raise RuntimeError(f"global tensors of one op must share a placement: {pl} vs {g._placement} "
                               "(use to_global to move one of them)")
    return pl


def _replace(args, kwargs, mapping):
    def f(x):
        return mapping.get(id(x), x) if isinstance(x, GlobalTensor) else x
    return pytree.tree_map(f, (args, kwargs))


# ------------------------------------------------------------------------------------------------ rules
RULES = {}


def rule(*ops):
    def deco(fn):
        for op in ops:
            RULES[op] = fn
        return fn
    return deco


def fallback_all_broadcast(func, args, kwargs):
    gs = _globals(args, kwargs)
    pl = _common_placement(gs)
    nd = (B,) * pl.ndim
    mapping = {id(g): rebox(g, nd) for g in gs}
    a2, k2 = _replace(args, kwargs, mapping)
    if func._schema.is_mutable and isinstance(args[0], GlobalTensor):
        self_t = args[0]
        boxed = mapping[id(self_t)]
        out = _finish(func, a2, k2, pl, [nd], shapes_from_result=True)
        self_t._local, self_t._nd_sbp = boxed._local, nd  # the mutation happened on the boxed shard
        return self_t if isinstance(out, GlobalTensor) else out
    return _finish(func, a2, k2, pl, [nd], shapes_from_result=True)


_LINEAR_UNARY = {aten.neg.default, aten.clone.default, aten.detach.default, aten.alias.default, aten._to_copy.default,
                 aten.contiguous.default, aten.view_as_real.default}
_ADD_LIKE = {aten.add.Tensor, aten.sub.Tensor, aten.add_.Tensor, aten.sub_.Tensor}
_MUL_LIKE = {aten.mul.Tensor, aten.mul_.Tensor, aten.div.Tensor, aten.div_.Tensor, aten.mul.Scalar, aten.div.Scalar,
             aten.mul_.Scalar, aten.div_.Scalar}


def _pointwise_fast(func, args, kwargs):
    """The common case without any inference: every tensor operand is a global tensor of ONE logical shape, dtype, placement
    and SBP (scalars beside them are fine), nothing is a partial sum unless the op is linear in them. The op then runs on
    the local shards as they are and the result carries the operands' description (gradient accumulation of a residual
    stream, optimizer arithmetic). Returns NotImplemented when the case does not apply."""
    first = None
    for a in args:
        if isinstance(a, GlobalTensor):
            if first is None:
                first = a
            elif a._placement != first._placement or a._nd_sbp != first._nd_sbp or a.shape != first.shape or a.dtype != first.dtype:
                return NotImplemented
        elif isinstance(a, torch.Tensor) or isinstance(a, (list, tuple)):
            return NotImplemented
    if first is None or kwargs and any(isinstance(v, torch.Tensor) for v in kwargs.values()):
        return NotImplemented
    n_glob = sum(isinstance(a, GlobalTensor) for a in args)
    if any(s_.kind == "P" for s_ in first._nd_sbp):
        if not ((func in _ADD_LIKE and n_glob == 2 and "alpha" not in kwargs) or (func in _LINEAR_UNARY and n_glob == 1)):
            return NotImplemented
    if func._schema.is_mutable:
        if not isinstance(args[0], GlobalTensor):
            return NotImplemented
        if _in_placement(first._placement):
            func(*[a._local if isinstance(a, GlobalTensor) else a for a in args], **kwargs)
        return args[0]
    if not _in_placement(first._placement):
        return NotImplemented
    res = func(*[a._local if isinstance(a, GlobalTensor) else a for a in args], **kwargs)
    if not isinstance(res, torch.Tensor) or res.shape != first._local.shape:
        return NotImplemented      # not an element-wise result after all: the general rule decides
    return wrap(res, first.shape, first._placement, first._nd_sbp)


def pointwise_rule(func, args, kwargs):
    fast = _pointwise_fast(func, args, kwargs)
    if fast is not NotImplemented:
        return fast
    gs = _globals(args, kwargs)
    pl = _common_placement(gs)
    try:
        meta_out = _infer_meta(func, args, kwargs)
        mflat, _ = pytree.tree_flatten(meta_out)
        out_meta = next(m for m in mflat if isinstance(m, torch.Tensor))
        out_shape = tuple(out_meta.shape)
    except (NotImplementedError, RuntimeError):
        # the op reads operand values while inferring (0-dim operands): a pointwise result has the broadcast shape
        meta_out = None
        flat_in, _ = pytree.tree_flatten((args, kwargs))
        out_shape = tuple(torch.broadcast_shapes(*[tuple(t.shape) for t in flat_in if isinstance(t, torch.Tensor)]))
    ond = len(out_shape)
    mutable = func._schema.is_mutable and isinstance(args[0], GlobalTensor)
    targets = {id(g): list(g._nd_sbp) for g in gs}
    out_nd = []
    for axis in range(pl.ndim):
        kinds = [g._nd_sbp[axis] for g in gs]
        chosen = None
        split = next((g for g in gs if g._nd_sbp[axis].kind == "S"), None)
        if mutable and args[0]._nd_sbp[axis].kind == "S":
            split = args[0]
        if split is not None:
            D = split._nd_sbp[axis].axis + (ond - split.dim())  # output dimension that is split
            ok = True
            for g in gs:
                d = D - (ond - g.dim())
                if d >= 0 and g.shape[d] == out_shape[D]:
                    targets[id(g)][axis] = S.split(d)
                elif d < 0 or g.shape[d] == 1:
                    targets[id(g)][axis] = B
                else:
                    ok = False
            if ok and not (mutable and targets[id(args[0])][axis] != args[0]._nd_sbp[axis] and args[0]._nd_sbp[axis].kind == "S"):
                chosen = S.split(D)
        if chosen is None and any(k.kind == "P" for k in kinds):
            lin = False
            if func in _LINEAR_UNARY:
                lin = True
            elif func in _ADD_LIKE:
                lin = all(isinstance(a, GlobalTensor) and a._nd_sbp[axis].kind == "P" for a in args[:2])
            elif func in _MUL_LIKE:
                others = [a for a in args[1:2] if isinstance(a, GlobalTensor)]
                lin = isinstance(args[0], GlobalTensor) and args[0]._nd_sbp[axis].kind == "P" and \
                    all(o._nd_sbp[axis].kind == "B" for o in others)
            if lin:
                for g in gs:
                    targets[id(g)][axis] = g._nd_sbp[axis]
                chosen = P
        if chosen is None:
            for g in gs:
                targets[id(g)][axis] = B
            chosen = B
        out_nd.append(chosen)
    mapping = {}
    for g in gs:
        mapping[id(g)] = rebox(g, targets[id(g)])
    if mutable:
        self_t = args[0]
        boxed = mapping[id(self_t)]
        if boxed is not self_t:
            self_t._local, self_t._nd_sbp = boxed._local, boxed._nd_sbp
            mapping[id(self_t)] = self_t
    a2, k2 = _replace(args, kwargs, mapping)
    if mutable:
        if _in_placement(pl):
            la, lk = pytree.tree_map(_local_of, (a2, k2))
            func(*la, **lk)
        return args[0]
    if meta_out is None:
        if not _in_placement(pl):
            return _placeholder(torch.empty(out_shape, dtype=gs[0].dtype, device="meta"), pl, tuple(out_nd))
        la, lk = pytree.tree_map(_local_of, (a2, k2))
        res = func(*la, **lk)
        flat, spec = pytree.tree_flatten(res)
        return pytree.tree_unflatten([wrap(t, out_shape, pl, tuple(out_nd)) if isinstance(t, torch.Tensor) else t for t in flat], spec)
    return _finish(func, a2, k2, pl, [tuple(out_nd)], meta_out=meta_out)


def _score(cands, ins, pl, axis):
    """Pick the candidate (tuple of required input sbp..., out sbp) with the lowest order value: -10 for every
    input already in the required layout, ties broken by copy cost (reference operator.cpp:609-663)."""
    best, best_key = None, None
    n = pl.hierarchy[axis]
    for c in cands:
        req = c[:-1]
        key0, cost = 0, 0.0
        feasible = True
        for g, r in zip(ins, req):
            if g is None:
                continue
            if r.kind == "S" and (r.axis >= g.dim() or g.shape[r.axis] < n):
                feasible = False
                break
            cur = g._nd_sbp[axis]
            if cur == r:
                key0 -= 10
            cost += copy_cost(cur, r, g.numel() * g.element_size(), n)
        if not feasible:
            continue
        key = (key0, cost)
        if best_key is None or key < best_key:
            best, best_key = c, key
    return best


def _matmul_like(func, args, kwargs, cands_fn, tensor_pos):
    gs = _globals(args, kwargs)
    pl = _common_placement(gs)
    ins = [args[i] if i < len(args) and isinstance(args[i], GlobalTensor) else None for i in tensor_pos]
    targets = {id(g): list(g._nd_sbp) for g in gs}
    out_nd = []
    for axis in range(pl.ndim):
        c = _score(cands_fn(ins), ins, pl, axis)
        for g, r in zip(ins, c[:-1]):
            if g is not None:
                targets[id(g)][axis] = r
        out_nd.append(c[-1])
    mapping = {id(g): rebox(g, targets[id(g)]) for g in gs}
    a2, k2 = _replace(args, kwargs, mapping)
    return _finish(func, a2, k2, pl, [tuple(out_nd)])


@rule(aten.mm.default)
def mm_rule(func, args, kwargs):
    s0, s1 = S.split(0), S.split(1)
    return _matmul_like(func, args, kwargs,
                        lambda ins: [(s0, B, s0), (B, s1, s1), (s1, s0, P), (P, B, P), (B, P, P), (B, B, B)], (0, 1))


@rule(aten.addmm.default)
def addmm_rule(func, args, kwargs):
    s0, s1 = S.split(0), S.split(1)
    bias = args[0]
    one_d = isinstance(bias, GlobalTensor) and bias.dim() == 1

    def cands(ins):
        if one_d:
            return [(B, s0, B, s0), (s0, B, s1, s1), (P, s1, s0, P), (P, P, B, P), (P, B, P, P), (B, B, B, B)]
        return [(s0, s0, B, s0), (s1, B, s1, s1), (P, s1, s0, P), (P, P, B, P), (P, B, P, P), (B, B, B, B)]
    return _matmul_like(func, args, kwargs, cands, (0, 1, 2))


@rule(aten.bmm.default)
def bmm_rule(func, args, kwargs):
    s0, s1, s2 = S.split(0), S.split(1), S.split(2)
    return _matmul_like(func, args, kwargs,
                        lambda ins: [(s0, s0, s0), (s1, B, s1), (B, s2, s2), (s2, s1, P), (P, B, P), (B, P, P), (B, B, B)], (0, 1))


def _remap_dim_rule(func, args, kwargs, dim_map):
    """View-like op whose output dims are a permutation / insertion / removal of the input dims.
    dim_map(in_dim) -> out dim or None (if the dim disappears: then the split must be dropped first)."""
    x = args[0]
    pl = x._placement
    nd_in, nd_out = list(x._nd_sbp), []
    for axis, s in enumerate(x._nd_sbp):
        if s.kind == "S":
            d = dim_map(s.axis)
            if d is None:
                nd_in[axis] = B
                nd_out.append(B)
            else:
                nd_out.append(S.split(d))
        else:
            nd_out.append(s)
    xb = rebox(x, nd_in)
    return _finish(func, (xb,) + tuple(args[1:]), kwargs, pl, [tuple(nd_out)])


@rule(aten.t.default)
def t_rule(func, args, kwargs):
    return _remap_dim_rule(func, args, kwargs, lambda d: 1 - d if args[0].dim() == 2 else d)


@rule(aten.transpose.int)
def transpose_rule(func, args, kwargs):
    nd = args[0].dim()
    a, b = args[1] % nd, args[2] % nd
    return _remap_dim_rule(func, args, kwargs, lambda d: b if d == a else (a if d == b else d))


@rule(aten.permute.default)
def permute_rule(func, args, kwargs):
    perm = [p % args[0].dim() for p in args[1]]
    return _remap_dim_rule(func, args, kwargs, lambda d: perm.index(d))


@rule(aten.unsqueeze.default)
def unsqueeze_rule(func, args, kwargs):
    nd = args[0].dim() + 1
    u = args[1] % nd
    return _remap_dim_rule(func, args, kwargs, lambda d: d + 1 if d >= u else d)


@rule(aten.squeeze.dim)
def squeeze_rule(func, args, kwargs):
    x = args[0]
    q = args[1] % max(x.dim(), 1)
    if x.dim() == 0 or x.shape[q] != 1:
        return _remap_dim_rule(func, args, kwargs, lambda d: d)
    return _remap_dim_rule(func, args, kwargs, lambda d: None if d == q else (d - 1 if d > q else d))


@rule(aten.view.default, aten._unsafe_view.default, aten.reshape.default)
def view_rule(func, args, kwargs):
    x = args[0]
    pl = x._placement
    in_shape = tuple(x.shape)
    meta = _infer_meta(func, args, kwargs)
    out_shape = tuple(meta.shape)
    coords = _coords(pl)
    nd_in, nd_out = list(x._nd_sbp), []
    local_out = list(out_shape)
    for axis, s in enumerate(x._nd_sbp):
        if s.kind != "S":
            nd_out.append(s)
            continue
        d = s.axis
        pre = math.prod(in_shape[:d])
        target = None
        acc = 1
        for j, o in enumerate(out_shape):
            if acc == pre and o == 1 and in_shape[d] != 1:
                continue                       # a size-1 axis inserted in front of the split dimension
            if acc == pre and o != 0:
                n = pl.hierarchy[axis]
                # d is the leading factor of output dim j (trailing dims merged in) or is itself cut in two
                if (o % in_shape[d] == 0 or in_shape[d] % o == 0) and in_shape[d] % n == 0 and o % n == 0:
                    target = j
                break
            acc *= o
        if target is None or any(k.kind == "S" and k.axis == d for a2, k in enumerate(x._nd_sbp) if a2 != axis):
            nd_in[axis] = B
            nd_out.append(B)
        else:
            nd_out.append(S.split(target))
            local_out[target] = local_out[target] // pl.hierarchy[axis]
    xb = rebox(x, nd_in)
    if not _in_placement(pl):
        return _placeholder(meta, pl, tuple(nd_out))
    try:
        res = func(xb._local, local_out)
    except RuntimeError:
        # the logical tensor is viewable but this shard's strides are not (it came out of a permute or a slice)
        res = xb._local.reshape(local_out)
    return wrap(res, out_shape, pl, tuple(nd_out))


@rule(aten.expand.default)
def expand_rule(func, args, kwargs):
    x = args[0]
    pl = x._placement
    meta = _infer_meta(func, args, kwargs)
    out_shape = list(meta.shape)
    shift = len(out_shape) - x.dim()
    local_size = list(args[1])
    nd_out = []
    for axis, s in enumerate(x._nd_sbp):
        if s.kind == "S":
            nd_out.append(S.split(s.axis + shift))
            if _in_placement(pl):
                local_size[s.axis + shift] = x._local.shape[s.axis]
        else:
            nd_out.append(s)
    if not _in_placement(pl):
        return _placeholder(meta, pl, tuple(nd_out))
    return wrap(func(x._local, local_size), out_shape, pl, tuple(nd_out))


def _reduce_rule(func, args, kwargs, is_mean=False):
    x = args[0]
    pl = x._placement
    dims = args[1] if len(args) > 1 and args[1] is not None else list(range(x.dim()))
    if isinstance(dims, int):
        dims = [dims]
    dims = sorted(d % max(x.dim(), 1) for d in dims) if x.dim() else []
    keepdim = (args[2] if len(args) > 2 else kwargs.get("keepdim", False))
    nd_out = []
    for s in x._nd_sbp:
        if s.kind == "S":
            if s.axis in dims:
                nd_out.append(P)
            else:
                nd_out.append(S.split(s.axis if keepdim else s.axis - sum(1 for d in dims if d < s.axis)))
        else:
            nd_out.append(s)
    meta = _infer_meta(func, args, kwargs)
    if not _in_placement(pl):
        return _placeholder(meta, pl, tuple(nd_out))
    if is_mean:
        count = math.prod(x.shape[d] for d in dims) if dims else 1
        local = torch.sum(x._local, dims, keepdim=keepdim, dtype=kwargs.get("dtype")) / count
    else:
        local = func(x._local, *args[1:], **kwargs)
    return wrap(local, meta.shape, pl, tuple(nd_out))


@rule(aten.sum.dim_IntList, aten.sum.default)
def sum_rule(func, args, kwargs):
    return _reduce_rule(func, args, kwargs)


@rule(aten.mean.dim, aten.mean.default)
def mean_rule(func, args, kwargs):
    return _reduce_rule(func, args, kwargs, is_mean=True)


def _keep_unless_dim(func, args, kwargs, dim, n_tensor_inputs=1):
    """Ops that work row-wise along `dim` (softmax family): any split except along `dim` passes through."""
    gs = [a for a in args[:n_tensor_inputs] if isinstance(a, GlobalTensor)]
    pl = _common_placement(gs)
    x = gs[0]
    dim = dim % max(x.dim(), 1)
    nd = []
    for axis in range(pl.ndim):
        s = x._nd_sbp[axis]
        nd.append(s if (s.kind == "S" and s.axis != dim) else B)
    mapping = {id(g): rebox(g, nd) for g in gs}
    a2, k2 = _replace(args, kwargs, mapping)
    return _finish(func, a2, k2, pl, [tuple(nd)])


@rule(aten._log_softmax.default, aten._softmax.default)
def softmax_rule(func, args, kwargs):
    return _keep_unless_dim(func, args, kwargs, args[1])


@rule(aten._log_softmax_backward_data.default, aten._softmax_backward_data.default)
def softmax_bwd_rule(func, args, kwargs):
    return _keep_unless_dim(func, args, kwargs, args[2], n_tensor_inputs=2)


@rule(aten.nll_loss_forward.default)
def nll_forward_rule(func, args, kwargs):
    logp, target, weight, reduction, ignore_index = args
    pl = logp._placement
    nd = [s if (s.kind == "S" and s.axis == 0) else B for s in logp._nd_sbp]
    lp, tg = rebox(logp, nd), rebox(target, nd)
    if weight is not None and isinstance(weight, GlobalTensor):
        weight = rebox(weight, (B,) * pl.ndim)
    if reduction == 0:  # none
        return _finish(func, (lp, tg, weight, reduction, ignore_index), {}, pl, [tuple(nd), (B,) * pl.ndim])
    split = any(s.kind == "S" for s in nd)
    if not split:
        return _finish(func, (lp, tg, weight, reduction, ignore_index), {}, pl, [(B,) * pl.ndim] * 2)
    # batch-split: local sums are partial sums; the mean divides by the global weight total
    part_nd = tuple(P if s.kind == "S" else B for s in nd)
    out, total = _finish(func, (lp, tg, weight, 2, ignore_index), {}, pl, [part_nd, part_nd])
    total_b = rebox(total, (B,) * pl.ndim)
    if reduction == 1:
        out = wrap(out._local / total_b._local if _in_placement(pl) else out._local, out.shape, pl, part_nd)
    return out, total_b


@rule(aten.nll_loss_backward.default)
def nll_backward_rule(func, args, kwargs):
    grad_out, logp, target, weight, reduction, ignore_index, total_weight = args
    pl = logp._placement
    nd = [s if (s.kind == "S" and s.axis == 0) else B for s in logp._nd_sbp]
    allb = (B,) * pl.ndim
    go = rebox(grad_out, nd if reduction == 0 else allb)
    lp, tg = rebox(logp, nd), rebox(target, nd)
    tw = rebox(total_weight, allb) if isinstance(total_weight, GlobalTensor) else total_weight
    if weight is not None and isinstance(weight, GlobalTensor):
        weight = rebox(weight, allb)
    return _finish(func, (go, lp, tg, weight, reduction, ignore_index, tw), {}, pl, [tuple(nd)])


@rule(aten.embedding.default)
def embedding_rule(func, args, kwargs):
    weight, idx = args[0], args[1]
    pl = weight._placement
    nd_w, nd_i, nd_o = [], [], []
    vocab_parallel = False
    for axis in range(pl.ndim):
        sw, si = weight._nd_sbp[axis], idx._nd_sbp[axis]
        if sw.kind == "S" and sw.axis == 0:     # vocabulary-parallel: out is a partial sum
            nd_w.append(sw); nd_i.append(B); nd_o.append(P)
            vocab_parallel = True
        elif si.kind == "S":
            nd_w.append(B); nd_i.append(si); nd_o.append(si)
        else:
            nd_w.append(B); nd_i.append(B); nd_o.append(B)
    w, i = rebox(weight, nd_w), rebox(idx, nd_i)
    if not vocab_parallel:
        return _finish(func, (w, i) + tuple(args[2:]), kwargs, pl, [tuple(nd_o)])
    meta = _infer_meta(func, args, kwargs)
    if not _in_placement(pl):
        return _placeholder(meta, pl, tuple(nd_o))
    from .nd_sbp import slice_view
    lo, hi = slice_view(weight.shape, pl.hierarchy, nd_w, _coords(pl))[0]
    li = i._local - lo
    mine = (li >= 0) & (li < hi - lo)
    out = torch.nn.functional.embedding(li.clamp(0, max(hi - lo - 1, 0)), w._local) * mine.unsqueeze(-1).to(w.dtype)
    return wrap(out, meta.shape, pl, tuple(nd_o))


@rule(aten.embedding_dense_backward.default)
def embedding_bwd_rule(func, args, kwargs):
    grad, idx = args[0], args[1]
    pl = grad._placement
    nd_g, nd_o = [], []
    for axis in range(pl.ndim):
        si = idx._nd_sbp[axis]
        if si.kind == "S":
            nd_g.append(si); nd_o.append(P)
        else:
            nd_g.append(B); nd_o.append(B)
    g = rebox(grad, nd_g)
    i = rebox(idx, nd_g)
    return _finish(func, (g, i) + tuple(args[2:]), kwargs, pl, [tuple(nd_o)])


@rule(aten.native_layer_norm.default)
def layer_norm_rule(func, args, kwargs):
    x, normalized_shape, w, b, eps = args
    pl = x._placement
    begin = x.dim() - len(normalized_shape)
    nd = [s if (s.kind == "S" and s.axis < begin) else B for s in x._nd_sbp]
    allb = (B,) * pl.ndim
    xb = rebox(x, nd)
    w = rebox(w, allb) if isinstance(w, GlobalTensor) else w
    b = rebox(b, allb) if isinstance(b, GlobalTensor) else b
    return _finish(func, (xb, normalized_shape, w, b, eps), {}, pl, [tuple(nd)] * 3)


@rule(aten.native_layer_norm_backward.default)
def layer_norm_bwd_rule(func, args, kwargs):
    go, x, normalized_shape, mean, rstd, w, b, mask = args
    pl = x._placement
    begin = x.dim() - len(normalized_shape)
    nd = [s if (s.kind == "S" and s.axis < begin) else B for s in x._nd_sbp]
    allb = (B,) * pl.ndim
    param_nd = tuple(P if s.kind == "S" else B for s in nd)  # gamma/beta grads are partial over the split rows
    go, x, mean, rstd = (rebox(t, nd) for t in (go, x, mean, rstd))
    w = rebox(w, allb) if isinstance(w, GlobalTensor) else w
    b = rebox(b, allb) if isinstance(b, GlobalTensor) else b
    return _finish(func, (go, x, normalized_shape, mean, rstd, w, b, mask), {}, pl, [tuple(nd), param_nd, param_nd])


@rule(aten.convolution.default)
def conv_rule(func, args, kwargs):
    x, w, bias = args[0], args[1], args[2]
    pl = x._placement
    nd = [s if (s.kind == "S" and s.axis == 0) else B for s in x._nd_sbp]
    allb = (B,) * pl.ndim
    xb, wb = rebox(x, nd), rebox(w, allb)
    bias = rebox(bias, allb) if isinstance(bias, GlobalTensor) else bias
    return _finish(func, (xb, wb, bias) + tuple(args[3:]), kwargs, pl, [tuple(nd)])


@rule(aten.convolution_backward.default)
def conv_bwd_rule(func, args, kwargs):
    go, x, w = args[0], args[1], args[2]
    pl = x._placement
    nd = [s if (s.kind == "S" and s.axis == 0) else B for s in x._nd_sbp]
    allb = (B,) * pl.ndim
    param_nd = tuple(P if s.kind == "S" else B for s in nd)
    return _finish(func, (rebox(go, nd), rebox(x, nd), rebox(w, allb)) + tuple(args[3:]), kwargs, pl,
                   [tuple(nd), param_nd, param_nd])


# ------------------------------------------------------------------------------------------------ dimension-preserving ops
def _keep_splits(func, args, kwargs, x_pos, blocked, like_pos=(), out_dim_map=None, n_out=1, partial_ok=False):
    """Signature family "a split passes through unless it is on a dimension the op works along": the tensors at
    ``x_pos`` (same rank, aligned dims) keep every split whose dimension is not in ``blocked`` and are broadcast on the
    other mesh axes; ``like_pos`` tensors are broadcast. ``out_dim_map(d)`` gives the output dimension of input dimension
    d (None: identity). The reference declares these per op (e.g. concat: oneflow/user/ops/concat_op.cpp, slice:
    slice_op.cpp, pooling: max_pool_op.cpp, dropout: dropout_op.cpp, normalization: normalization_op.cpp)."""
    flat = list(args)
    xs = [flat[i] for i in x_pos]
    tensors = []
    for x in xs:
        tensors += list(x) if isinstance(x, (list, tuple)) else [x]
    gs = [t for t in tensors if isinstance(t, GlobalTensor)]
    pl = _common_placement(gs + [flat[i] for i in like_pos if i < len(flat) and isinstance(flat[i], GlobalTensor)])
    ref = gs[0]
    nd_in, nd_out = [], []
    for axis in range(pl.ndim):
        kinds = [g._nd_sbp[axis] for g in gs]
        s0 = kinds[0]
        same = all(k == s0 for k in kinds)
        if same and s0.kind == "S" and (s0.axis % max(ref.dim(), 1)) not in blocked:
            nd_in.append(s0)
            d = s0.axis if out_dim_map is None else out_dim_map(s0.axis)
            nd_out.append(S.split(d))
        elif same and s0.kind == "P" and partial_ok:
            nd_in.append(P)
            nd_out.append(P)
        else:
            nd_in.append(B)
            nd_out.append(B)
    mapping = {id(g): rebox(g, nd_in) for g in gs}
    allb = (B,) * pl.ndim
    for i in like_pos:
        if i < len(flat) and isinstance(flat[i], GlobalTensor):
            mapping[id(flat[i])] = rebox(flat[i], allb)
    a2, k2 = _replace(args, kwargs, mapping)
    return _finish(func, a2, k2, pl, [tuple(nd_out)] * n_out if n_out > 1 else [tuple(nd_out)])


@rule(aten.select.int)
def select_rule(func, args, kwargs):
    x, dim = args[0], args[1] % args[0].dim()
    return _keep_splits(func, args, kwargs, (0,), {dim}, out_dim_map=lambda d: d - 1 if d > dim else d, partial_ok=True)


@rule(aten.slice.Tensor)
def slice_rule(func, args, kwargs):
    x = args[0]
    dim = (args[1] if len(args) > 1 else 0) % max(x.dim(), 1)
    start = args[2] if len(args) > 2 and args[2] is not None else 0
    end = args[3] if len(args) > 3 and args[3] is not None else x.shape[dim]
    step = args[4] if len(args) > 4 else 1
    whole = start == 0 and end >= x.shape[dim] and step == 1
    return _keep_splits(func, args, kwargs, (0,), set() if whole else {dim}, partial_ok=True)


@rule(aten.narrow.default)
def narrow_rule(func, args, kwargs):
    x, dim = args[0], args[1] % args[0].dim()
    return _keep_splits(func, args, kwargs, (0,), {dim}, partial_ok=True)


@rule(aten.cat.default)
def cat_rule(func, args, kwargs):
    ts = args[0]
    dim = (args[1] if len(args) > 1 else kwargs.get("dim", 0)) % max(ts[0].dim(), 1)
    if not all(isinstance(t, GlobalTensor) and t.dim() == ts[0].dim() for t in ts):
        return fallback_all_broadcast(func, args, kwargs)
    return _keep_splits(func, args, kwargs, (0,), {dim}, partial_ok=True)


@rule(aten.stack.default)
def stack_rule(func, args, kwargs):
    ts = args[0]
    if not all(isinstance(t, GlobalTensor) for t in ts):
        return fallback_all_broadcast(func, args, kwargs)
    dim = (args[1] if len(args) > 1 else kwargs.get("dim", 0)) % (ts[0].dim() + 1)
    return _keep_splits(func, args, kwargs, (0,), set(), out_dim_map=lambda d: d + 1 if d >= dim else d, partial_ok=True)


@rule(aten.split.Tensor, aten.split_with_sizes.default, aten.unsafe_split.Tensor, aten.unsafe_split_with_sizes.default)
def split_rule(func, args, kwargs):
    x = args[0]
    dim = (args[2] if len(args) > 2 else kwargs.get("dim", 0)) % max(x.dim(), 1)
    return _keep_splits(func, args, kwargs, (0,), {dim}, partial_ok=True)


@rule(aten.unbind.int)
def unbind_rule(func, args, kwargs):
    x = args[0]
    dim = (args[1] if len(args) > 1 else 0) % max(x.dim(), 1)
    return _keep_splits(func, args, kwargs, (0,), {dim}, out_dim_map=lambda d: d - 1 if d > dim else d, partial_ok=True)


@rule(aten.index_select.default)
def index_select_rule(func, args, kwargs):
    dim = args[1] % max(args[0].dim(), 1)
    return _keep_splits(func, args, kwargs, (0,), {dim}, like_pos=(2,), partial_ok=True)


@rule(aten.gather.default)
def gather_rule(func, args, kwargs):
    # input and index have the same rank and are walked together on every dimension but `dim`
    dim = args[1] % max(args[0].dim(), 1)
    return _keep_splits(func, args, kwargs, (0, 2), {dim})


@rule(aten.native_dropout.default)
def dropout_rule(func, args, kwargs):
    # every shard draws its own mask: any split passes through, a partial sum has to be completed first
    return _keep_splits(func, args, kwargs, (0,), set(), n_out=2)


@rule(aten.native_dropout_backward.default)
def dropout_bwd_rule(func, args, kwargs):
    return _keep_splits(func, args, kwargs, (0, 1), set())


@rule(aten.max_pool2d_with_indices.default, aten.max_pool3d_with_indices.default)
def max_pool_rule(func, args, kwargs):
    x = args[0]
    spatial = set(range(x.dim() - (2 if "2d" in func._schema.name else 3), x.dim()))
    return _keep_splits(func, args, kwargs, (0,), spatial, n_out=2)


@rule(aten.max_pool2d_with_indices_backward.default, aten.max_pool3d_with_indices_backward.default)
def max_pool_bwd_rule(func, args, kwargs):
    x = args[1]
    spatial = set(range(x.dim() - (2 if "2d" in func._schema.name else 3), x.dim()))
    idx_pos = len(args) - 1
    return _keep_splits(func, args, kwargs, (0, 1, idx_pos), spatial)


@rule(aten.avg_pool2d.default, aten.avg_pool3d.default, aten._adaptive_avg_pool2d.default, aten._adaptive_avg_pool3d.default,
      aten.upsample_nearest2d.default, aten.upsample_bilinear2d.default)
def spatial_rule(func, args, kwargs):
    x = args[0]
    nsp = 3 if "3d" in func._schema.name else 2
    return _keep_splits(func, args, kwargs, (0,), set(range(x.dim() - nsp, x.dim())))


@rule(aten.avg_pool2d_backward.default, aten._adaptive_avg_pool2d_backward.default)
def spatial_bwd_rule(func, args, kwargs):
    x = args[1]
    return _keep_splits(func, args, kwargs, (0, 1), set(range(x.dim() - 2, x.dim())))


@rule(aten._native_batch_norm_legit.default, aten._native_batch_norm_legit_no_training.default, aten.native_batch_norm.default,
      aten._native_batch_norm_legit_functional.default)
def batch_norm_rule(func, args, kwargs):
    """Inference keeps batch and spatial splits (the statistics are given). Training needs the statistics of the whole
    batch: the input is gathered unless only the channel dimension is split (per-channel statistics are then local)."""
    x = args[0]
    name = func._schema.name
    training = False if name.endswith("no_training") else bool(args[5])
    pl = x._placement
    allb = (B,) * pl.ndim
    params = [a for a in args[1:5] if isinstance(a, GlobalTensor)]
    nd = []
    for s_ in x._nd_sbp:
        if s_.kind == "S" and s_.axis != 1 and not training:
            nd.append(s_)
        else:
            nd.append(B)
    mapping = {id(x): rebox(x, nd)}
    for p_ in params:
        mapping[id(p_)] = rebox(p_, allb)
    a2, k2 = _replace(args, kwargs, mapping)
    meta = _infer_meta(func, args, kwargs)
    n_t = len([m for m in pytree.tree_flatten(meta)[0] if isinstance(m, torch.Tensor)])
    return _finish(func, a2, k2, pl, [tuple(nd)] + [allb] * (n_t - 1), meta_out=meta)


@rule(aten._scaled_dot_product_flash_attention.default, aten._scaled_dot_product_efficient_attention.default,
      aten._scaled_dot_product_flash_attention_for_cpu.default, aten._scaled_dot_product_cudnn_attention.default)
def sdpa_rule(func, args, kwargs):
    """[B, H, S, D] attention: batch and head splits are independent problems (the reference declares exactly these two,
    oneflow/user/ops/scaled_dot_product_flash_attention_op.cpp:71-100); a sequence or feature split is gathered."""
    q = args[0]
    pl = q._placement
    gs = [a for a in args[:3] if isinstance(a, GlobalTensor)]
    nd = []
    for axis in range(pl.ndim):
        s0 = q._nd_sbp[axis]
        ok = s0.kind == "S" and s0.axis in (0, 1) and all(g._nd_sbp[axis] == s0 for g in gs)
        nd.append(s0 if ok else B)
    mapping = {id(g): rebox(g, nd) for g in gs}
    for a in list(args[3:]) + list(kwargs.values()):
        if isinstance(a, GlobalTensor):
            mapping[id(a)] = rebox(a, (B,) * pl.ndim)
    a2, k2 = _replace(args, kwargs, mapping)
    meta = _infer_meta(func, args, kwargs)
    flat = [m for m in pytree.tree_flatten(meta)[0] if isinstance(m, torch.Tensor)]
    out_nds = []
    for m in flat:
        # outputs that carry batch and head dimensions keep the split; scalars (rng state, offsets) are broadcast
        out_nds.append(tuple(s_ if (s_.kind == "S" and m.dim() > s_.axis and m.shape[s_.axis] == q.shape[s_.axis]) else B for s_ in nd))
    return _finish(func, a2, k2, pl, out_nds, meta_out=meta)


@rule(aten.copy_.default)
def copy_rule(func, args, kwargs):
    dst, src = args[0], args[1]
    if isinstance(dst, GlobalTensor):
        if isinstance(src, GlobalTensor):
            src_local = boxing.convert(src._local, tuple(src.shape), src.dtype, src._placement, src._nd_sbp,
                                       dst._placement, dst._nd_sbp)
        else:
            coords = _coords(dst._placement)
            src_local = boxing.from_all_broadcast(src.expand(dst.shape).to(dst._local.device), dst._placement,
                                                  dst._nd_sbp, coords) if coords is not None else None
        if _in_placement(dst._placement):
            dst._local.copy_(src_local)
        return dst
    src_b = rebox(src, (B,) * src._placement.ndim)
    return dst.copy_(src_b._local)


@rule(aten._local_scalar_dense.default, aten.equal.default, aten.is_nonzero.default)
def scalar_rule(func, args, kwargs):
    gs = _globals(args, kwargs)
    pl = _common_placement(gs)
    mapping = {id(g): rebox(g, (B,) * pl.ndim) for g in gs}
    a2, k2 = _replace(args, kwargs, mapping)
    la, lk = pytree.tree_map(_local_of, (a2, k2))
    if not _in_placement(pl):
        raise RuntimeError("cannot read the value of a global tensor on a rank outside its placement")
    return func(*la, **lk)


_LIKE_FACTORIES = {aten.ones_like.default, aten.zeros_like.default, aten.empty_like.default, aten.full_like.default,
                   aten.rand_like.default, aten.randn_like.default, aten.new_zeros.default, aten.new_ones.default,
                   aten.new_empty.default, aten.new_full.default}


def like_rule(func, args, kwargs):
    x = args[0]
    pl = x._placement
    nd = tuple(B if s.kind == "P" else s for s in x._nd_sbp)
    if func in (aten.new_zeros.default, aten.new_ones.default, aten.new_empty.default, aten.new_full.default):
        return fallback_all_broadcast(func, args, kwargs)
    xb = rebox(x, nd)
    return _finish(func, (xb,) + tuple(args[1:]), kwargs, pl, [nd])


def dispatch(func, args, kwargs):
    r = RULES.get(func)
    if r is not None:
        return r(func, args, kwargs)
    if func in _LIKE_FACTORIES:
        return like_rule(func, args, kwargs)
    if torch.Tag.pointwise in func.tags or func in _LINEAR_UNARY:
        return pointwise_rule(func, args, kwargs)
    return fallback_all_broadcast(func, args, kwargs)


# ------------------------------------------------------------------------------------------------ to_global / to_local
def _norm_sbp(sbp, pl):
    if sbp is None:
        raise ValueError("sbp is required")
    return S.normalize(sbp, pl.ndim)


class _LocalToGlobal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, local, pl, nd, logical_shape):
        ctx.nd, ctx.pl = nd, pl
        return wrap(local.detach(), logical_shape, pl, nd)

    @staticmethod
    def backward(ctx, grad):
        # dual SBP: a broadcast input was used on every rank, so its gradient is the partial sum of theirs
        dual = tuple(P if s.kind == "B" else (B if s.kind == "P" else s) for s in ctx.nd)
        g = grad if isinstance(grad, GlobalTensor) else None
        if g is None:
            return grad, None, None, None
        g = rebox(g, dual) if any(a.kind != b.kind for a, b in zip(g._nd_sbp, dual)) and False else g
        # every rank only needs its own local gradient: S -> the shard, B(out-grad) -> full copy
        want = tuple(s if s.kind == "S" else B for s in ctx.nd)
        return rebox(g, want)._local, None, None, None


class _GlobalToLocal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g):
        ctx.pl, ctx.nd, ctx.shape = g._placement, g._nd_sbp, tuple(g.shape)
        return g._local.detach().clone() if False else g._local.detach()

    @staticmethod
    def backward(ctx, grad_local):
        dual = tuple(P if s.kind == "B" else (B if s.kind == "P" else s) for s in ctx.nd)
        return wrap(grad_local, ctx.shape, ctx.pl, dual)


class _GlobalToGlobal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, pl, nd, grad_nd):
        ctx.in_pl, ctx.in_nd, ctx.grad_nd = g._placement, g._nd_sbp, grad_nd
        ctx.out_nd = tuple(nd)
        if pl == g._placement:
            out = rebox(g, nd)                 # same ranks: a deferred partial sum can take its fused reduce-scatter
            return wrap(out._local, g.shape, pl, nd) if out is g else out
        local = boxing.convert(g._local, tuple(g.shape), g.dtype, g._placement, g._nd_sbp, pl, nd)
        return wrap(local, g.shape, pl, nd)

    @staticmethod
    def backward(ctx, grad):
        # the gradient returns to the input's placement, with grad_sbp if given else its own sbp
        # (reference: oneflow/core/autograd/gradient_funcs/global_to_global.cpp:52-75)
        if grad._placement != ctx.in_pl and ctx.grad_nd is None and grad._placement.hierarchy == ctx.in_pl.hierarchy:
            # a placement change between equal meshes (pipeline stage boundary): first bring the gradient to the layout
            # the forward tensor had, inside its own placement. Both sides of the transfer then agree on the layout
            # without exchanging it (the rank that skipped this stage only holds a placeholder), and each rank sends
            # its shard to its counterpart.
            want = tuple(B if s_.kind == "P" else s_ for s_ in ctx.out_nd)
            grad = rebox(grad, want)
        nd = ctx.grad_nd if ctx.grad_nd is not None else grad._nd_sbp
        if len(nd) != ctx.in_pl.ndim:
            nd = (B,) * ctx.in_pl.ndim
        local = boxing.convert(grad._local, tuple(grad.shape), grad.dtype, grad._placement, grad._nd_sbp, ctx.in_pl, nd)
        return wrap(local, grad.shape, ctx.in_pl, nd), None, None, None


def _infer_logical_shape(local, pl, nd, check_meta):
    coords = _coords(pl)
    shape = list(local.shape)
    for axis, s in enumerate(nd):
        if s.kind != "S":
            continue
        n = pl.hierarchy[axis]
        if check_meta and dist.is_initialized() and n > 1:
            sizes = [None] * n
            dist.all_gather_object(sizes, int(local.shape[s.axis]) if coords is not None else 0, group=pl.axis_group(axis))
            shape[s.axis] = sum(sizes)
        else:
            shape[s.axis] = shape[s.axis] * n
    return tuple(shape)


def to_global(x, placement=None, sbp=None, *, grad_sbp=None, check_meta=True, copy=False, sync_data=True):
    """local -> global, or global -> global (SBP and/or placement change)."""
    if isinstance(x, GlobalTensor):
        pl = placement if placement is not None else x._placement
        nd = _norm_sbp(sbp, pl) if sbp is not None else (x._nd_sbp if pl.ndim == x._placement.ndim else None)
        if nd is None:
            raise ValueError("sbp is required when the placement hierarchy changes")
        gnd = _norm_sbp(grad_sbp, x._placement) if grad_sbp is not None else None
        if pl == x._placement and nd == x._nd_sbp and not copy:
            return x
        if x.requires_grad and torch.is_grad_enabled():
            return _GlobalToGlobal.apply(x, pl, nd, gnd)
        if pl == x._placement:
            return rebox(x, nd)
        local = boxing.convert(x._local, tuple(x.shape), x.dtype, x._placement, x._nd_sbp, pl, nd)
        return wrap(local, x.shape, pl, nd)
    if placement is None or sbp is None:
        raise ValueError("to_global of a local tensor needs placement and sbp")
    pl = placement
    nd = _norm_sbp(sbp, pl)
    me_in = _in_placement(pl)
    if me_in and pl.size > 1 and dist.is_initialized():
        # local -> global is collective over the placement (shape agreement, broadcast of B data): with
        # ONEFLOW_TIMEOUT_SECONDS set, a rank that never arrives here is reported instead of waited for
        from . import control_plane
        if control_plane.consistency_timeout() is not None:
            control_plane.check_consistency(list(pl.ranks_flat), f"local_to_global {tuple(x.shape)} {x.dtype} {tuple(str(s_) for s_ in nd)}")
    local = x
    if me_in:
        dev = pl.device()
        if local.device != dev:
            local = local.to(dev)
    shape = _infer_logical_shape(local, pl, nd, check_meta)
    if me_in and sync_data and dist.is_initialized() and pl.size > 1 and any(s.kind == "B" for s in nd) and not x.requires_grad:
        # broadcast sbp: every rank must hold the same data; take the first rank's along each B axis
        for axis, s in enumerate(nd):
            if s.kind == "B" and pl.hierarchy[axis] > 1:
                src = pl.axis_ranks(axis, _rank())[0]
                local = local.contiguous().clone() if local.data_ptr() == x.data_ptr() else local
                dist.broadcast(local, src, group=pl.axis_group(axis))
    if not me_in:
        local = torch.empty((0,), dtype=x.dtype, device=pl.device() if pl.type == "cpu" else x.device)
    if x.requires_grad and torch.is_grad_enabled():
        return _LocalToGlobal.apply(local, pl, nd, shape)
    return wrap(local, shape, pl, nd, requires_grad=False)


def to_local(x, copy=False):
    if not isinstance(x, GlobalTensor):
        return x
    if x.requires_grad and torch.is_grad_enabled():
        out = _GlobalToLocal.apply(x)
    else:
        out = x._local
    return out.clone() if copy else out
