"""The hot ops of the flow API on the hand-written sm_100a kernels, for local AND global tensors.

Every function here is what a user reaches through ``flow.nn.Linear`` / ``flow.nn.LayerNorm`` /
``flow.nn.Embedding`` / ``flow.nn.functional.*`` / ``flow._C.fused_*``. Each op carries

* its SBP signatures (which layouts of its operands it can consume and what layout the result gets), chosen
  per mesh axis from the operands' current SBP as the reference's ``GetSbp`` functions do
  (matmul: oneflow/user/ops/matmul_op.cpp:123-175, layer_norm: oneflow/user/ops/layer_norm_op.cpp,
  embedding / gather: oneflow/user/ops/gather_op.cpp, sparse_softmax_cross_entropy:
  oneflow/user/ops/sparse_softmax_cross_entropy_op.cpp, attention:
  oneflow/user/ops/scaled_dot_product_flash_attention_op.cpp:71-100);
* the boxing its signature needs, FUSED into the GEMM where the pattern is tensor parallelism with
  sequence-split activations: ``S(0)`` rows -> all-gather -> column-parallel product runs as the one-kernel
  all-gather->GEMM, a row-parallel product whose partial-sum result is wanted as ``S(0)`` rows runs as the
  one-kernel GEMM->reduce-scatter (csrc/comm/gemm_comm.cu) -- what the reference inserts as separate
  ``_nccl_logical_*`` ops (oneflow/core/job_rewriter/insert_nccl_logical_op_pass.cpp:192-296);
* its backward written with the same kernels (data gradient, weight gradient without transposes, bias
  gradient as a column sum), so gradients of tensor-parallel layers use the fused products as well.

A row-parallel product returns a *deferred* partial-sum tensor: the local GEMM only runs when somebody needs
the partial values; ``to_global(sbp=split(0))`` on it (or any consumer that boxes it to ``S(0)``) runs the fused
GEMM->reduce-scatter instead, so ``matmul`` followed by ``to_global`` costs one kernel.

Parameters that carry a ``_main_grad`` view (set by ``nn.Graph`` for its fused optimizers) receive their
gradient by accumulation in fp32 straight from the GEMM epilogue; the autograd gradient is then ``None``.
bf16 CUDA tensors always run the native kernels; CPU tensors and other dtypes run the PyTorch statements of
``ops`` (the same call sites, used by the gloo-rank tests).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from .. import sbp as S
from ..ops import embedding as E
from ..ops import gemm as G
from ..ops import kernels as K
from . import global_tensor as GT

B_, P_ = S.broadcast, S.partial_sum
_TP_CTX = {}
op_trace = None          # a list while nn.Graph records its plan: (op name, detail dict) tuples are appended


def _trace(name, **kw):
    if op_trace is not None:
        op_trace.append((name, kw))


def _is_g(t):
    return isinstance(t, GT.GlobalTensor)


def _loc(t):
    return t._local if _is_g(t) else t


def _native(*ts):
    """True when every given tensor can go to the kernels (bf16 on CUDA) or all of them are CPU tensors (statements)."""
    ts = [t for t in ts if t is not None]
    if all(not t.is_cuda for t in ts):
        return True
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def _kind(t, axis, n):
    """SBP of ``t`` on a mesh axis; an axis of size 1 reads as broadcast."""
    if t is None or n == 1:
        return B_
    return t._nd_sbp[axis]


def _in_pl(pl):
    return pl.contains(GT._rank())


def tp_context(pl, axis, device, tokens, hidden):
    """The fused-product context (symmetric arena + in-kernel collectives) of this rank's sub-group along one mesh
    axis, grown (collectively: every rank of the group sees the same shapes) when a larger problem arrives."""
    me = GT._rank()
    ranks = tuple(pl.axis_ranks(axis, me))
    key = (ranks, str(device))
    ctx = _TP_CTX.get(key)
    if ctx is None or ctx.max_tokens < tokens or ctx.hidden_cap < hidden:
        from ..parallel.tensor_parallel import TPContext
        if ctx is not None:
            tokens, hidden = max(tokens, ctx.max_tokens), max(hidden, ctx.hidden_cap)
            if device.type == "cuda":
                torch.cuda.synchronize()
        ctx = TPContext(pl.axis_group(axis), list(ranks), device, max_tokens=tokens, max_cols=hidden, hidden=hidden)
        if ctx.cuda is False:
            ctx.hidden_cap = hidden
        _TP_CTX[key] = ctx
    return ctx


def _fusable(t, rows_full, n, *dims):
    """The fused GEMM+collective kernels take bf16 CUDA operands, row counts that are multiples of 128 per rank and
    8-aligned columns; everything else runs the collective and the product as two steps."""
    return t.is_cuda and t.dtype == torch.bfloat16 and rows_full % (n * 128) == 0 and all(d % 8 == 0 for d in dims)


def _gemm(a, b, **kw):
    """ops.gemm; the CPU statement keeps the operands' dtype (the kernel path is bf16 by construction)."""
    if a.is_cuda:
        return G.gemm(a, b, **kw)
    if "out" not in kw:
        kw["out_dtype"] = a.dtype
    if kw.get("want_aux"):
        # the statement's pre-activation output in the operands' dtype: product + bias first, the rest on top
        act, residual = kw.pop("act", 0), kw.pop("residual", None)
        kw.pop("want_aux")
        aux = G.gemm(a, b, **kw)
        y = G._act_ref(aux.float(), G._act_code(act))
        if residual is not None:
            y = y + residual.float()
        return y.to(a.dtype), aux
    return G.gemm(a, b, **kw)


# ------------------------------------------------------------------------------------------------ deferred partial sums
class DeferredPartial:
    """The not-yet-computed local value of a partial-sum (``P``) result of a row-parallel product.

    ``materialize`` runs the plain GEMM (what any consumer of the partial values gets); ``reduce_scatter`` runs the
    fused GEMM->reduce-scatter, giving this rank's rows of the sum directly."""

    def __init__(self, a, w, b_layout, bias, pl, axis, idx, logical_rows):
        self.a, self.w, self.b_layout, self.bias = a, w, b_layout, bias
        self.pl, self.axis, self.idx, self.rows = pl, axis, idx, logical_rows

    def materialize(self):
        # the bias belongs to the sum, not to every addend: only the first rank of the axis adds it
        return _gemm(self.a, self.w, b_layout=self.b_layout, bias=self.bias if self.idx == 0 else None)

    def reduce_scatter(self, residual=None):
        n = self.pl.hierarchy[self.axis]
        N = self.w.shape[0] if self.b_layout == "nk" else self.w.shape[1]
        Kd = self.a.shape[1]
        if _fusable(self.a, self.a.shape[0], n, N, Kd):
            tp = tp_context(self.pl, self.axis, self.a.device, self.a.shape[0], max(N, Kd))
            _trace("gemm_reduce_scatter", T=self.a.shape[0], N=N, K=Kd, n=n)
            return tp.gemm_rs(self.a, self.w, b_layout=self.b_layout, bias=self.bias, residual=residual)
        from . import boxing
        part = _gemm(self.a, self.w, b_layout=self.b_layout)
        ranks = self.pl.axis_ranks(self.axis, GT._rank())
        out = boxing.p_to_s(part, 0, self.pl.axis_group(self.axis), ranks, self.idx)
        if self.bias is not None:
            out = out + self.bias
        return out if residual is None else out + residual


def take_deferred_reduce_scatter(x, nd):
    """If ``x`` is a deferred partial sum and ``nd`` only differs from its SBP by ``P -> S(0)`` on the deferred axis,
    returns the local result of the fused GEMM->reduce-scatter, else None (called by ``global_tensor.rebox``)."""
    th = x.__dict__.get("_thunk")
    if th is None or x.dim() != 2:
        return None
    cur = x._nd_sbp
    for a, (c, t) in enumerate(zip(cur, nd)):
        if a == th.axis:
            if not (t.kind == "S" and t.axis == 0):
                return None
        elif c != t:
            return None
    # rows may already be split on other mesh axes (data parallel): only an outer split of dim 0 composes with this one
    for a, c in enumerate(cur):
        if a != th.axis and c.kind == "S" and c.axis == 0 and a > th.axis:
            return None
    return th.reduce_scatter()


# ------------------------------------------------------------------------------------------------ parameter gradients
def _param_grad(param, nd, value_fn, accumulate_fn):
    """Delivers a parameter gradient. With a ``_main_grad`` buffer on the parameter the gradient is accumulated there in
    fp32 (``accumulate_fn(buffer)``) and autograd gets None; otherwise ``value_fn()`` is returned for autograd."""
    if param is None or not param.requires_grad:
        return None
    mg = getattr(param, "_main_grad", None)
    if mg is not None:
        accumulate_fn(mg)
        if nd is not None:
            param._grad_nd_sbp = tuple(nd)
        return None
    v = value_fn()
    if _is_g(param):
        return GT.wrap(v.to(param.dtype), param.shape, param._placement, tuple(nd))
    return v.to(param.dtype)


def _wgrad(param, nd, dy2, x2):
    """d/dW of y = x W^T: dy^T x, [N, K] (weights with more dims keep their own shape)."""
    def acc(mg):
        G.gemm(dy2, x2, a_layout="km", b_layout="kn", out=mg.view(dy2.shape[1], x2.shape[1]), accumulate=True)

    def val():
        return _gemm(dy2, x2, a_layout="km", b_layout="kn").view(_loc(param).shape)
    return _param_grad(param, nd, val, acc)


def _bgrad(param, nd, dy2):
    def acc(mg):
        K.column_sum(dy2, out=mg.view(-1))

    def val():
        return K.column_sum(dy2).view(_loc(param).shape)
    return _param_grad(param, nd, val, acc)


# ------------------------------------------------------------------------------------------------ linear
class _LinearPlan:
    """SBP signature of one ``linear`` call: per mesh axis data / column / row, plus what the fused paths need."""
    __slots__ = ("pl", "nd_x", "nd_w", "mode", "axis", "n", "idx", "x_gather", "out_nd", "out_rs", "in_pl")


def _plan_linear(x, w, bias, residual, out_rs):
    """Returns a _LinearPlan, or None when the operands' SBP fits none of the signatures handled here (the caller then
    falls back to the ATen-level rules)."""
    pl = w._placement if _is_g(w) else x._placement
    if (_is_g(x) and x._placement != pl) or not _is_g(w) or not _is_g(x):
        return None
    p = _LinearPlan()
    p.pl, p.mode, p.axis, p.n, p.idx, p.x_gather, p.out_rs = pl, "data", -1, 1, 0, False, False
    p.in_pl = _in_pl(pl)
    coords = pl.coords(GT._rank())
    out_nd = []
    last = x.dim() - 1
    wcol = w.dim() - 2                    # the out-features axis of the weight ([N, K] or [G, N, K])
    for a, n in enumerate(pl.hierarchy):
        xs, ws = _kind(x, a, n), _kind(w, a, n)
        bs = _kind(bias, a, n) if _is_g(bias) else B_
        if ws.kind == "B":
            if xs.kind == "P" or (xs.kind == "S" and xs.axis == last) or bs.kind != "B":
                return None
            out_nd.append(xs)
        elif ws.kind == "S" and ws.axis == wcol:
            if p.mode != "data" or (bias is not None and not (bs.kind == "S" and bs.axis == bias.dim() - 1)):
                return None
            if xs.kind == "S" and xs.axis == 0 and x.dim() == 2:
                p.x_gather = True
            elif xs.kind != "B":
                return None
            p.mode, p.axis, p.n = "col", a, n
            out_nd.append(S.split(last + (w.dim() - 2)))
        elif ws.kind == "S" and ws.axis == w.dim() - 1 and w.dim() == 2:
            if p.mode != "data" or not (xs.kind == "S" and xs.axis == last) or bs.kind != "B":
                return None
            p.mode, p.axis, p.n = "row", a, n
            rs = out_rs or (residual is not None and _is_g(residual) and _kind(residual, a, n).kind == "S"
                            and _kind(residual, a, n).axis == 0)
            p.out_rs = bool(rs) and x.dim() == 2
            out_nd.append(S.split(0) if p.out_rs else P_)
        else:
            return None
    if p.axis >= 0 and coords is not None:
        p.idx = coords[p.axis]
    p.out_nd = tuple(out_nd)
    return p


class _Linear(torch.autograd.Function):
    """y = act(x W^T + b) + residual on local shards, with the tensor-parallel exchange fused into the products."""

    @staticmethod
    def forward(ctx, x, w, bias, residual, act, plan, link=None):
        ctx.plan, ctx.act = plan, act
        ctx.link = link            # (link this call produces for, link it consumes) when the call is a layer of ``mlp``
        ctx.x_shape, ctx.has_res = tuple(x.shape), residual is not None
        ctx.params = (w, bias)
        g = plan is not None
        xl, wl, bl, rl = _loc(x), _loc(w), _loc(bias), _loc(residual)
        out_shape = tuple(x.shape[:-1]) + tuple(w.shape[:-2]) + (w.shape[-2],)
        if g and not plan.in_pl:
            ctx.skip = True
            return GT._placeholder(torch.empty(out_shape, dtype=x.dtype, device="meta"), plan.pl, plan.out_nd)
        ctx.skip = False
        x2 = xl.reshape(-1, xl.shape[-1])
        if not x2.is_contiguous() or (x2.is_cuda and x2.data_ptr() % 16):
            x2 = x2.contiguous() if not x2.is_contiguous() else x2.clone()
        w2 = wl.reshape(-1, wl.shape[-1])
        _trace("linear", mode=(plan.mode if g else "local"), M=x2.shape[0], N=w2.shape[0], K=w2.shape[1], act=int(act),
               residual=residual is not None)
        b1 = bl.reshape(-1) if bl is not None else None
        r2 = rl.reshape(-1, rl.shape[-1]) if rl is not None else None
        aux, x_saved, thunk = None, x2, None
        mode = plan.mode if g else "data"
        if mode == "col" and plan.x_gather:
            n = plan.n
            T = x2.shape[0] * n
            if _fusable(x2, T, n, w2.shape[0], x2.shape[1]):
                tp = tp_context(plan.pl, plan.axis, x2.device, T, max(x2.shape[1], 8))
                _trace("all_gather_gemm", T=T, N=w2.shape[0], K=x2.shape[1], n=n)
                res = tp.ag_gemm(x2, w2, bias=b1, act=act, want_aux=bool(act), return_gathered=True)
                gathered, y = res[0], res[1]
                aux = res[2] if act else None
                # the gathered rows live in the exchange buffer, which later calls overwrite: keep a copy for the
                # weight gradient (cheaper than gathering again in the backward)
                x_saved = gathered.clone() if gathered.is_cuda else gathered
            else:
                from . import boxing
                ranks = plan.pl.axis_ranks(plan.axis, GT._rank())
                x_saved = boxing.s_to_b(x2, 0, plan.pl.axis_group(plan.axis), ranks, plan.idx, T)
                y, aux = _gemm_act(x_saved, w2, b1, act, r2)
        elif mode == "row":
            if act:
                raise ValueError("linear: an activation on a row-parallel product needs the reduced sum first")
            n = plan.n
            if plan.out_rs:
                th = DeferredPartial(x2, w2, "nk", b1, plan.pl, plan.axis, plan.idx, x2.shape[0])
                y = th.reduce_scatter(r2)
            else:
                thunk = DeferredPartial(x2, w2, "nk", b1, plan.pl, plan.axis, plan.idx, x2.shape[0])
                y = None
        else:
            y, aux = _gemm_act(x2, w2, b1, act, r2)
        ctx.save_for_backward(x_saved, w2, aux)
        if link is not None and link[0] is not None:
            link[0].aux, link[0].act = aux, act
        if not g:
            return y.view(out_shape)
        lshape = _local_shape_of(out_shape, plan.pl, plan.out_nd)
        if thunk is not None:
            return GT.wrap_deferred(thunk, lshape, out_shape, x.dtype, x2.device, plan.pl, plan.out_nd)
        return GT.wrap(y.view(lshape), out_shape, plan.pl, plan.out_nd)

    @staticmethod
    def backward(ctx, dy):
        plan, act = ctx.plan, ctx.act
        w, bias = ctx.params
        g = plan is not None
        if ctx.skip:
            dxp = GT._placeholder(torch.empty(ctx.x_shape, dtype=dy.dtype, device="meta"), plan.pl, (B_,) * plan.pl.ndim)
            return dxp, None, None, (dy if ctx.has_res else None), None, None, None
        x2, w2, aux = ctx.saved_tensors
        link = ctx.link
        # the consumer half of ``mlp``: its input is the producer's activation output and nothing else reads that, so the
        # activation's gradient rides in the epilogue of this call's data-gradient GEMM
        fuse = {}
        prod, cons = link if link is not None else (None, None)
        if cons is not None and cons.aux is not None and cons.act:
            fuse = {"aux_in": cons.aux, "act": cons.act}
        mode = plan.mode if g else "data"
        dres = dy if ctx.has_res else None
        if g:
            # bring the incoming gradient to the layout this signature's backward consumes
            want = list(plan.out_nd)
            if mode == "row":
                cur = dy._nd_sbp[plan.axis] if plan.n > 1 else B_
                want[plan.axis] = cur if (cur.kind == "B" or (cur.kind == "S" and cur.axis == 0)) else B_
            dy = GT.rebox(dy, want)
            dyl = dy._local
        else:
            dyl = dy
        dy2 = dyl.reshape(-1, w2.shape[0]) if mode != "row" or not g else dyl.reshape(-1, dyl.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if act and not (prod is not None and prod.fused):
            dy2 = K.bias_act_bwd(aux, None, dy2, act)
        # a link outlives the nodes' saved tensors (it hangs on the context objects until the whole graph is freed): drop its
        # reference to the pre-activation values as soon as nobody needs it (the dict above keeps them for this call)
        if prod is not None:
            prod.aux = None
        if cons is not None and fuse:
            cons.aux = None
        nd_w = w._nd_sbp if _is_g(w) else None
        nd_b = bias._nd_sbp if _is_g(bias) else None
        x_nd = None
        if mode == "data":
            dx2 = _gemm(dy2, w2, b_layout="kn", **fuse) if ctx.needs_input_grad[0] else None
            if fuse and dx2 is not None:
                cons.fused = True
            gw = _wgrad(w, _param_nd(plan, nd_w, None), dy2, x2)
            gb = _bgrad(bias, _param_nd(plan, nd_b, None), dy2)
            x_nd = tuple(plan.out_nd[:]) if g else None
            if g:
                x_nd = tuple(_x_nd_data(plan))
        elif mode == "col":
            gw = _wgrad(w, _param_nd(plan, nd_w, plan.axis), dy2, x2)
            gb = _bgrad(bias, _param_nd(plan, nd_b, plan.axis), dy2)
            dx2, thunk = None, None
            if ctx.needs_input_grad[0]:
                if plan.x_gather:
                    th = DeferredPartial(dy2, w2, "kn", None, plan.pl, plan.axis, plan.idx, dy2.shape[0])
                    dx2 = th.reduce_scatter()
                    x_nd = tuple(_x_nd_data(plan, axis_sbp=S.split(0)))
                else:
                    thunk = DeferredPartial(dy2, w2, "kn", None, plan.pl, plan.axis, plan.idx, dy2.shape[0])
                    x_nd = tuple(_x_nd_data(plan, axis_sbp=P_))
            if thunk is not None:
                out = GT.wrap_deferred(thunk, _local_shape_of(ctx.x_shape, plan.pl, x_nd), ctx.x_shape, dy2.dtype, dy2.device,
                                       plan.pl, x_nd)
                return out, gw, gb, dres, None, None, None
        else:  # row
            cur = dy._nd_sbp[plan.axis] if plan.n > 1 else B_
            dy_full = dy2
            if cur.kind == "S":
                n = plan.n
                T = dy2.shape[0] * n
                if _fusable(dy2, T, n, w2.shape[1], dy2.shape[1]):
                    tp = tp_context(plan.pl, plan.axis, dy2.device, T, max(dy2.shape[1], 8))
                    _trace("all_gather_gemm", T=T, N=w2.shape[1], K=dy2.shape[1], n=n, grad=True)
                    dy_full, dx2 = tp.ag_gemm(dy2, w2, b_layout="kn", return_gathered=True, **fuse)
                else:
                    from . import boxing
                    ranks = plan.pl.axis_ranks(plan.axis, GT._rank())
                    dy_full = boxing.s_to_b(dy2, 0, plan.pl.axis_group(plan.axis), ranks, plan.idx, T)
                    dx2 = _gemm(dy_full, w2, b_layout="kn", **fuse)
                if fuse:
                    cons.fused = True
                # the bias was added once to the reduced rows: its gradient is the column sum over this rank's rows,
                # a partial sum over the axis
                gb = _bgrad(bias, _param_nd(plan, nd_b, None, partial_axis=plan.axis), dy2)
            else:
                dx2 = _gemm(dy2, w2, b_layout="kn", **fuse)
                if fuse:
                    cons.fused = True
                gb = _bgrad(bias, _param_nd(plan, nd_b, None), dy2)
            gw = _wgrad(w, _param_nd(plan, nd_w, plan.axis), dy_full, x2)
            x_nd = tuple(_x_nd_data(plan, axis_sbp=S.split(len(ctx.x_shape) - 1)))
        if dx2 is None:
            return None, gw, gb, dres, None, None, None
        if not g:
            return dx2.view(ctx.x_shape), gw, gb, dres, None, None, None
        return GT.wrap(dx2.view(_local_shape_of(ctx.x_shape, plan.pl, x_nd)), ctx.x_shape, plan.pl, x_nd), gw, gb, dres, None, None, None


def _gemm_act(x2, w2, b1, act, r2):
    if act:
        y, aux = _gemm(x2, w2, bias=b1, act=act, want_aux=True, residual=r2)
        return y, aux
    return _gemm(x2, w2, bias=b1, residual=r2), None


def _local_shape_of(shape, pl, nd):
    from .nd_sbp import local_shape
    coords = pl.coords(GT._rank())
    return tuple(local_shape(shape, pl.hierarchy, nd, coords))


def _x_nd_data(plan, axis_sbp=None):
    """SBP of the input gradient: what the input had on the data axes, ``axis_sbp`` on the model-parallel axis."""
    nd = []
    for a, s in enumerate(plan.out_nd):
        if a == plan.axis:
            nd.append(axis_sbp)
        else:
            nd.append(s)
    return nd


def _param_nd(plan, nd_param, model_axis, partial_axis=None):
    """SBP of a parameter gradient: the parameter's own split on the model-parallel axis, a partial sum on every axis
    along which the rows of the activations were split (data parallelism, sequence parallelism)."""
    if plan is None or nd_param is None:
        return None
    nd = []
    for a, s in enumerate(nd_param):
        n = plan.pl.hierarchy[a]
        if a == model_axis:
            nd.append(s)
        elif a == partial_axis:
            nd.append(P_ if n > 1 else B_)
        elif a == plan.axis:
            nd.append(s if s.kind == "S" else B_)
        else:
            o = plan.out_nd[a]
            nd.append(P_ if (o.kind == "S" and n > 1) else B_)
    return tuple(nd)


class _ActLink:
    """What the two halves of ``mlp`` share: the producer's pre-activation values and activation code, and whether the
    consumer's backward already applied the activation's gradient."""
    __slots__ = ("aux", "act", "fused")

    def __init__(self):
        self.aux, self.act, self.fused = None, 0, False


def mlp(x, w1, b1, w2, b2, *, act="gelu", residual=None, out_sbp=None):
    """``linear(act(linear(x, w1, b1)), w2, b2) + residual`` as one unit: the hidden activation is private to the call, so
    in backward the activation's gradient is folded into the epilogue of the second layer's data-gradient GEMM (one pass
    over the [tokens, ffn] hidden gradient less). SBP handling, fused tensor-parallel products and parameter gradients
    are those of ``linear`` (column-parallel first layer, row-parallel second layer is the Megatron MLP).
    Reference: the fused MLP family (oneflow/user/kernels/cublas_fused_mlp_kernel.cu, cublas_bias_add_relu_matmul_grad)."""
    link = _ActLink()
    h = linear(x, w1, b1, act=act, _link=(link, None))
    return linear(h, w2, b2, residual=residual, out_sbp=out_sbp, _link=(None, link))


def mlp_chain(x, weights, biases, *, act="relu", skip_final_activation=False):
    """A stack of linear layers with one activation between them (the reference's ``fused_mlp``): every hidden activation is
    private to the call, so each layer's backward folds the previous layer's activation gradient into its data-gradient GEMM."""
    n = len(weights)
    prev = None
    for i, (w, b) in enumerate(zip(weights, biases)):
        last = i == n - 1
        a = 0 if (last and skip_final_activation) else act
        nxt = _ActLink() if (not last and a) else None
        x = linear(x, w, b, act=a, _link=(nxt, prev))
        prev = nxt
    return x


def linear(x, weight, bias=None, *, act=0, residual=None, out_sbp=None, _link=None):
    """``act(x @ weight^T + bias) + residual``.

    weight: ``[N, K]``, or ``[G, N, K]`` for G stacked projections (the result then has shape ``[..., G, N]``: a packed
    QKV projection is ``G = 3`` with the heads split on axis 1, so each tensor-parallel rank holds whole heads of q, k
    and v). ``act``: 0 / "gelu" / "gelu_tanh" / "relu". ``residual`` is added after the activation (the reference's
    ``_add_to_output``). For a row-parallel product ``out_sbp=split(0)`` (or a ``split(0)`` residual) selects the fused
    GEMM->reduce-scatter; without it the result is a deferred partial sum."""
    act = G._act_code(act)
    if _is_g(x) or _is_g(weight):
        if not _is_g(x) or not _is_g(weight):
            raise TypeError("linear: x and weight must both be global or both be local")
        want_rs = out_sbp is not None and any(s.kind == "S" and s.axis == 0 for s in S.normalize(out_sbp, weight._placement.ndim)
                                              if s is not None)
        plan = _plan_linear(x, weight, bias, residual, want_rs)
        if plan is not None and _native(_loc(x), _loc(weight)) and _aligned(weight):
            return _Linear.apply(x, weight, bias, residual, act, plan, _link)
        w2 = weight if weight.dim() == 2 else weight.reshape(-1, weight.shape[-1])
        y = torch.nn.functional.linear(x, w2, bias.reshape(-1) if bias is not None and bias.dim() > 1 else bias)
        if weight.dim() == 3:
            y = y.reshape(*x.shape[:-1], weight.shape[0], weight.shape[1])
        y = G._act_ref(y, act) if act else y
        return y if residual is None else y + residual
    if x.is_cuda and _native(x, weight) and _aligned(weight) and x.numel() > 0:
        return _Linear.apply(x, weight, bias, residual, act, None, _link)
    w2 = weight if weight.dim() == 2 else weight.reshape(-1, weight.shape[-1])
    y = torch.nn.functional.linear(x, w2, bias.reshape(-1) if bias is not None and bias.dim() > 1 else bias)
    if weight.dim() == 3:
        y = y.reshape(*x.shape[:-1], weight.shape[0], weight.shape[1])
    y = G._act_ref(y, act) if act else y
    return y if residual is None else y + residual


def _aligned(weight):
    wl = _loc(weight)
    if wl.numel() == 0:
        return True
    return wl.shape[-1] % 8 == 0 and wl.shape[-2] % 8 == 0 and (not wl.is_cuda or wl.data_ptr() % 16 == 0)


# ------------------------------------------------------------------------------------------------ layer norm
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, pl, nd, passthrough=False):
        ctx.pl, ctx.nd, ctx.shape = pl, nd, tuple(x.shape)
        ctx.params = (gamma, beta)
        ctx.passthrough = passthrough
        if pl is not None and not _in_pl(pl):
            ctx.skip = True
            ph = GT._placeholder(torch.empty(x.shape, dtype=x.dtype, device="meta"), pl, nd)
            return (ph, GT._placeholder(torch.empty(x.shape, dtype=x.dtype, device="meta"), pl, nd)) if passthrough else ph
        ctx.skip = False
        xl = _loc(x)
        x2 = xl.reshape(-1, xl.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        _trace("layer_norm", rows=x2.shape[0], cols=x2.shape[1])
        y, mean, rstd = K.layer_norm_fwd(x2, _loc(gamma), _loc(beta), eps)
        ctx.save_for_backward(x2, _loc(gamma), mean, rstd)
        y = y.view(xl.shape)
        yo = GT.wrap(y, x.shape, pl, nd) if pl is not None else y
        if not passthrough:
            return yo
        # the input handed on for the residual branch: whatever gradient reaches it comes back to THIS node, which adds it
        # inside the LayerNorm backward kernel instead of leaving the sum of the two branches to a separate add
        xo = GT.wrap(xl.view(xl.shape), x.shape, pl, nd) if pl is not None else xl.view(xl.shape)
        return yo, xo

    @staticmethod
    def backward(ctx, dy, dx_pass=None):
        gamma, beta = ctx.params
        pl, nd = ctx.pl, ctx.nd
        if ctx.skip:
            return (dy if dy is not None else dx_pass), None, None, None, None, None, None
        x2, gl, mean, rstd = ctx.saved_tensors
        addend = None
        if dx_pass is not None:
            if pl is not None:
                dx_pass = GT.rebox(dx_pass, nd)
            addend = _loc(dx_pass).reshape(x2.shape)
            if not addend.is_contiguous():
                addend = addend.contiguous()
        if dy is None:         # only the passed-through input was used
            dx = addend.view(_loc(dx_pass).shape)
            return (GT.wrap(dx, ctx.shape, pl, nd) if pl is not None else dx), None, None, None, None, None, None
        if pl is not None:
            dy = GT.rebox(dy, nd)
        dyl = _loc(dy)
        dy2 = dyl.reshape(x2.shape)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # parameter gradients are partial sums over every mesh axis that splits the rows
        pnd = tuple(P_ if (s.kind == "S" and pl.hierarchy[a] > 1) else B_ for a, s in enumerate(nd)) if pl is not None else None
        mg, mb = getattr(gamma, "_main_grad", None), getattr(beta, "_main_grad", None)
        want = gamma is not None and gamma.requires_grad
        if want and mg is not None and mb is not None:
            dx, _, _ = K.layer_norm_bwd(dy2, x2, gl, mean, rstd, add_to_dx=addend, dgamma=mg.view(-1), dbeta=mb.view(-1))
            gamma._grad_nd_sbp = beta._grad_nd_sbp = pnd
            dg = db = None
        else:
            dx, dg, db = K.layer_norm_bwd(dy2, x2, gl, mean, rstd, add_to_dx=addend, want_param_grads=want)
            if want:
                dg, db = dg.to(gl.dtype), db.to(gl.dtype)
                if pl is not None:
                    dg = GT.wrap(dg, gamma.shape, pl, pnd)
                    db = GT.wrap(db, beta.shape, pl, pnd)
            else:
                dg = db = None
        dx = dx.view(dyl.shape)
        if pl is not None:
            dx = GT.wrap(dx, ctx.shape, pl, nd)
        return dx, dg, (db if beta is not None else None), None, None, None, None


def layer_norm_residual(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    """``(layer_norm(x), x)`` for a pre-norm residual block: use the returned ``x`` for the residual branch. The gradients of
    the two branches then meet inside the LayerNorm backward kernel (its ``add_to_dx`` input) instead of in a separate add."""
    return layer_norm(x, normalized_shape, weight, bias, eps, _passthrough=True)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5, _passthrough=False):
    """LayerNorm over the last axis on the native kernels (rows may be split on any mesh axis; parameters broadcast);
    other forms go to the ATen path."""
    ns = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    ok = len(ns) == 1 and weight is not None and bias is not None and x.shape[-1] % 8 == 0 and x.shape[-1] <= 32768
    if ok and _is_g(x):
        pl = x._placement
        last = x.dim() - 1
        ok = _native(_loc(x)) and _is_g(weight) and _is_g(bias) and weight._placement == pl and all(
            _kind(x, a, n).kind == "B" or (_kind(x, a, n).kind == "S" and _kind(x, a, n).axis != last) for a, n in enumerate(pl.hierarchy)) \
            and all(_kind(weight, a, n).kind == "B" and _kind(bias, a, n).kind == "B" for a, n in enumerate(pl.hierarchy))
        if ok:
            return _LayerNorm.apply(x, weight, bias, eps, pl, x._nd_sbp, _passthrough)
    elif ok and not _is_g(weight) and _native(x, weight, bias) and (x.is_cuda or x.dtype == torch.bfloat16) and x.numel() > 0:
        return _LayerNorm.apply(x, weight, bias, eps, None, None, _passthrough)
    y = torch.nn.functional.layer_norm(x, ns, weight, bias, eps)
    return (y, x) if _passthrough else y


# ------------------------------------------------------------------------------------------------ attention
class _PackedAttention(torch.autograd.Function):
    """Causal / full self-attention on a packed QKV activation ``[tokens, 3, heads * head_dim]`` (``heads`` split over
    the tensor-parallel axis: SBP ``S(2)``; tokens of whole sequences may be split over a data-parallel axis)."""

    @staticmethod
    def forward(ctx, qkv, seq, head_dim, causal, scale, pl, nd_out):
        ctx.pl, ctx.nd_in, ctx.shape = pl, (qkv._nd_sbp if pl is not None else None), tuple(qkv.shape)
        ctx.causal, ctx.scale = causal, scale
        out_shape = (qkv.shape[0], qkv.shape[2])
        if pl is not None and not _in_pl(pl):
            ctx.skip = True
            return GT._placeholder(torch.empty(out_shape, dtype=qkv.dtype, device="meta"), pl, nd_out)
        ctx.skip = False
        q = _loc(qkv)
        T, _, HD = q.shape
        Hl = HD // head_dim
        q5 = q.view(T // seq, seq, 3, Hl, head_dim)
        _trace("fused_attention", batch=T // seq, seq=seq, heads=Hl, head_dim=head_dim, causal=bool(causal))
        out, lse = K.fmha_fwd(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], causal=causal, scale=scale)
        ctx.save_for_backward(q5, out, lse)
        y = out.view(T, HD)
        return GT.wrap(y, out_shape, pl, nd_out) if pl is not None else y

    @staticmethod
    def backward(ctx, d_o):
        if ctx.skip:
            return (GT._placeholder(torch.empty(ctx.shape, dtype=d_o.dtype, device="meta"), ctx.pl, ctx.nd_in),) + (None,) * 6
        q5, out, lse = ctx.saved_tensors
        pl = ctx.pl
        if pl is not None:
            want = tuple(S.split(1) if (s.kind == "S" and s.axis == 2) else s for s in ctx.nd_in)
            d_o = GT.rebox(d_o, want)
        dl = _loc(d_o)
        Bq, Sq, _, Hl, D = q5.shape
        d4 = dl.reshape(Bq, Sq, Hl, D)
        if not d4.is_contiguous():
            d4 = d4.contiguous()
        dqkv = torch.empty_like(q5)
        K.fmha_bwd(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], out, d4, lse, causal=ctx.causal, scale=ctx.scale, dqkv=dqkv)
        d = dqkv.view(Bq * Sq, 3, Hl * D)
        return (GT.wrap(d, ctx.shape, pl, ctx.nd_in) if pl is not None else d,) + (None,) * 6


def fused_attention_qkv_packed(qkv, *, seq_len, head_size, causal=True, scale=None):
    """Self-attention over a packed projection ``qkv [tokens, 3, hidden]`` (tokens = batch * seq_len, sequences
    contiguous); returns ``[tokens, hidden]``. Head-split ``S(2)`` inputs give a column-split ``S(1)`` result, ready for
    a row-parallel output projection. Runs the fused tcgen05 attention kernels for head sizes 64 / 128."""
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(head_size)
    if _is_g(qkv):
        pl = qkv._placement
        nd_out = []
        for a, n in enumerate(pl.hierarchy):
            s = _kind(qkv, a, n)
            if s.kind == "S" and s.axis == 2:
                nd_out.append(S.split(1))
            elif s.kind == "B" or (s.kind == "S" and s.axis == 0):
                nd_out.append(s)
            else:
                qkv = GT.rebox(qkv, tuple(B_ if i == a else t for i, t in enumerate(qkv._nd_sbp)))
                nd_out.append(B_)
        return _PackedAttention.apply(qkv, seq_len, head_size, causal, sc, pl, tuple(nd_out))
    return _PackedAttention.apply(qkv, seq_len, head_size, causal, sc, None, None)


# ------------------------------------------------------------------------------------------------ embedding
class _Embedding(torch.autograd.Function):
    """Row lookup. Vocabulary-parallel tables (weight ``S(0)``) give partial-sum rows (ids outside the shard read zero)."""

    @staticmethod
    def forward(ctx, ids, weight, pl, nd_ids, nd_out, vocab_start):
        ctx.pl, ctx.nd_out, ctx.vocab_start = pl, nd_out, vocab_start
        ctx.weight = weight
        out_shape = tuple(ids.shape) + (weight.shape[1],)
        ctx.out_shape = out_shape
        if pl is not None and not _in_pl(pl):
            ctx.skip = True
            return GT._placeholder(torch.empty(out_shape, dtype=weight.dtype, device="meta"), pl, nd_out)
        ctx.skip = False
        il, wl = _loc(ids), _loc(weight)
        ctx.save_for_backward(il)
        _trace("embedding", ids=il.numel(), rows=wl.shape[0], vocab_start=int(vocab_start))
        y = E.embedding_fwd(il, wl, None, seq=1, vocab_start=vocab_start).view(tuple(il.shape) + (wl.shape[1],))
        return GT.wrap(y, out_shape, pl, nd_out) if pl is not None else y

    @staticmethod
    def backward(ctx, dy):
        weight, pl = ctx.weight, ctx.pl
        if ctx.skip:
            return None, None, None, None, None, None
        (il,) = ctx.saved_tensors
        if pl is not None:
            # every rank needs the gradient rows of all the ids it looked up: P (the forward's partial rows) reads as B
            want = tuple(B_ if s.kind == "P" else s for s in ctx.nd_out)
            dy = GT.rebox(dy, want)
        dyl = _loc(dy).reshape(-1, weight.shape[1])
        if not dyl.is_contiguous():
            dyl = dyl.contiguous()
        wl = _loc(weight)
        nd_w = None
        if pl is not None:
            nd_w = tuple(s if s.kind == "S" else (P_ if (o.kind == "S" and pl.hierarchy[a] > 1) else B_)
                         for a, (s, o) in enumerate(zip(weight._nd_sbp, ctx.nd_out)))

        def acc(mg):
            E.embedding_bwd(il, dyl, mg.view(wl.shape), None, seq=1, vocab_start=ctx.vocab_start)

        def val():
            g = torch.zeros(wl.shape, dtype=torch.float32, device=wl.device)
            E.embedding_bwd(il, dyl, g, None, seq=1, vocab_start=ctx.vocab_start)
            return g
        gw = _param_grad(weight, nd_w, val, acc)
        return None, gw, None, None, None, None


def embedding(ids, weight):
    """``weight[ids]``; native kernels for bf16 CUDA tables. Global tensors: a table split on the vocabulary (``S(0)``)
    yields partial-sum rows (each rank contributes the ids of its shard), a broadcast table follows the ids' SBP."""
    if _is_g(weight):
        pl = weight._placement
        if not _is_g(ids) or ids._placement != pl or not _native(_loc(weight)) or weight.shape[1] % 8:
            return torch.nn.functional.embedding(ids, weight)
        nd_ids, nd_out, vocab_start = list(ids._nd_sbp), [], 0
        coords = pl.coords(GT._rank())
        from .nd_sbp import slice_view
        for a, n in enumerate(pl.hierarchy):
            ws, isb = _kind(weight, a, n), _kind(ids, a, n)
            if ws.kind == "S" and ws.axis == 0:
                nd_ids[a] = B_
                nd_out.append(P_)
            elif ws.kind == "B":
                nd_ids[a] = isb if isb.kind != "P" else B_
                nd_out.append(nd_ids[a])
            else:
                return torch.nn.functional.embedding(ids, weight)
        ids = GT.rebox(ids, nd_ids)
        if coords is not None:
            vocab_start = slice_view(weight.shape, pl.hierarchy, weight._nd_sbp, coords)[0][0]
        return _Embedding.apply(ids, weight, pl, tuple(nd_ids), tuple(nd_out), vocab_start)
    if weight.is_cuda and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0 and ids.numel() > 0 and not _is_g(ids):
        return _Embedding.apply(ids, weight, None, None, None, 0)
    return torch.nn.functional.embedding(ids, weight)


# ------------------------------------------------------------------------------------------------ cross entropy
class _SparseXent(torch.autograd.Function):
    """Per-row softmax cross entropy of integer labels; the class axis may be split over one mesh axis (the row
    statistics of the shards are merged, as the reference's vocabulary-parallel kernel does with all-reduces)."""

    @staticmethod
    def forward(ctx, logits, labels, pl, nd_rows, vaxis, vocab_start):
        ctx.pl, ctx.nd_rows, ctx.nd_logits = pl, nd_rows, (logits._nd_sbp if pl is not None else None)
        ctx.shape = tuple(logits.shape)
        if pl is not None and not _in_pl(pl):
            ctx.skip = True
            return GT._placeholder(torch.empty(logits.shape[:1], dtype=torch.float32, device="meta"), pl, nd_rows)
        ctx.skip = False
        ll, lab = _loc(logits), _loc(labels).reshape(-1)
        _trace("sparse_softmax_cross_entropy", rows=ll.shape[0], classes=ll.shape[1], vocab_parallel=vaxis is not None)
        stats = K.xent_stats(ll, lab, vocab_start=vocab_start)
        if vaxis is not None:
            from . import boxing
            n = pl.hierarchy[vaxis]
            ranks = pl.axis_ranks(vaxis, GT._rank())
            allp = boxing.s_to_b(stats.reshape(1, -1), 0, pl.axis_group(vaxis), ranks, pl.coords(GT._rank())[vaxis], n)
            stats = K.xent_merge(allp.view(n, ll.shape[0], 3))
        loss, _ = K.xent_grad(ll, lab, stats, vocab_start=vocab_start, want_grad=False)
        ctx.save_for_backward(ll, lab, stats)
        ctx.vocab_start = vocab_start
        return GT.wrap(loss, logits.shape[:1], pl, nd_rows) if pl is not None else loss

    @staticmethod
    def backward(ctx, dloss):
        if ctx.skip:
            return GT._placeholder(torch.empty(ctx.shape, dtype=torch.bfloat16, device="meta"), ctx.pl, ctx.nd_logits), None, None, None, None, None
        ll, lab, stats = ctx.saved_tensors
        pl = ctx.pl
        if pl is not None:
            dloss = GT.rebox(dloss, ctx.nd_rows)
        dl = _loc(dloss).reshape(-1, 1).to(torch.float32)
        # (softmax - onehot) written over the logits' own storage (they are not needed again), then the row scale
        _, d = K.xent_grad(ll, lab, stats, vocab_start=ctx.vocab_start, inplace=True)
        d.mul_(dl.to(d.dtype))
        return (GT.wrap(d, ctx.shape, pl, ctx.nd_logits) if pl is not None else d), None, None, None, None, None


def sparse_softmax_cross_entropy(logits, labels):
    """loss[row] = logsumexp(logits[row]) - logits[row, labels[row]] as fp32, for 2-D ``logits``. Global logits may be
    split on the class axis (vocabulary parallel). The backward reuses the logits' storage for their gradient."""
    if _is_g(logits):
        pl = logits._placement
        if logits.dim() != 2 or not _is_g(labels) or labels._placement != pl or not _native(_loc(logits)):
            return _xent_fallback(logits, labels)
        nd_rows, nd_lab, vaxis, vocab_start = [], [], None, 0
        for a, n in enumerate(pl.hierarchy):
            s = _kind(logits, a, n)
            if s.kind == "S" and s.axis == 1:
                if vaxis is not None:
                    return _xent_fallback(logits, labels)
                vaxis = a
                nd_rows.append(B_)
            elif s.kind == "P":
                return _xent_fallback(logits, labels)
            else:
                nd_rows.append(s)
        labels = GT.rebox(labels, tuple(nd_rows))
        if vaxis is not None:
            from .nd_sbp import slice_view
            coords = pl.coords(GT._rank())
            if coords is not None:
                vocab_start = slice_view(logits.shape, pl.hierarchy, logits._nd_sbp, coords)[1][0]
        return _SparseXent.apply(logits, labels, pl, tuple(nd_rows), vaxis, vocab_start)
    if logits.dim() == 2 and not _is_g(labels) and logits.is_cuda and logits.dtype == torch.bfloat16 and logits.is_contiguous():
        return _SparseXent.apply(logits, labels, None, None, None, 0)
    return _xent_fallback(logits, labels)


def _xent_fallback(logits, labels):
    nc = logits.shape[-1]
    return torch.nn.functional.cross_entropy(logits.reshape(-1, nc).float(), labels.reshape(-1).long(), reduction="none").reshape(labels.shape)
