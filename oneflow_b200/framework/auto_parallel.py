"""Auto-parallel: choose the SBP signature of every layer of a network so that compute plus boxing cost is minimal.

The network is given as a chain of matmul-like layers (the dominant case: Linear / attention projections / MLPs).
Every layer has the three classic candidates
    data parallel    x S(0), w B     -> y S(0)      (weight gradient needs an all-reduce)
    column parallel  x B,    w S(0)  -> y S(1)      (weights split over the output features)
    row parallel     x S(1), w S(1)  -> y P         (weights split over the input features)
and consecutive layers are joined by the boxing that turns the produced SBP into the consumed one, priced by the
same copy-cost model the boxing planner uses (csrc/core/sbp_math.cpp). A dynamic programme over the chain finds the
cheapest assignment; memory is a hard constraint (weights + optimizer state per rank must fit).

Reference: oneflow/core/auto_parallel/{sbp_graph,sbp_node,sbp_edge,sbp_constructor,sbp_collector}.cpp and
oneflow/core/job_rewriter/auto_parallel.cpp (graph of ops with candidate signatures, edge costs = boxing cost,
node/edge elimination to find the minimum); nn.Graph ``config.enable_auto_parallel``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

from .. import sbp as _sbp


@dataclass
class LinearSpec:
    name: str
    in_features: int
    out_features: int
    tokens: int                 # rows of the activation (batch x sequence)
    bytes_per_elem: int = 2


@dataclass
class Choice:
    name: str
    kind: str                   # "data", "column", "row"
    x_sbp: object
    w_sbp: object
    y_sbp: object


_CANDIDATES = (
    ("data", _sbp.split(0), _sbp.broadcast, _sbp.split(0)),
    ("column", _sbp.broadcast, _sbp.split(0), _sbp.split(1)),
    ("row", _sbp.split(1), _sbp.split(1), _sbp.partial_sum),
)


def _copy_cost(a, b, nbytes, n):
    if a == b or n == 1:
        return 0.0
    try:
        from ..runtime import core
        return float(core.copy_cost(a, b, nbytes, n))
    except Exception:
        # same formulas as the native model: bytes that cross the links per rank
        f = (n - 1) / n
        if a.kind == "P":
            return nbytes * (2 * f if b.kind == "B" else f)
        if a.kind == "S" and b.kind == "B":
            return nbytes * f
        if a.kind == "S" and b.kind == "S":
            return nbytes * f / n
        return 0.0        # B -> S / B -> P: local slicing


def solve_chain(layers: Sequence[LinearSpec], world: int, *, flops_per_s: float = 1.4e15, link_bytes_per_s: float = 7.7e11,
                mem_bytes_per_rank: Optional[float] = None, state_bytes_per_param: float = 16.0, input_sbp=None,
                output_sbp=None, train: bool = True) -> List[Choice]:
    """Returns one Choice per layer minimising estimated step time (seconds)."""
    input_sbp = input_sbp or _sbp.split(0)
    INF = float("inf")
    best = {0: (0.0, [])}          # key: index of the produced-SBP candidate of the previous layer (0 = the input)
    prev_out = {0: input_sbp}
    mem_used = {0: 0.0}
    for spec in layers:
        act_in = spec.tokens * spec.in_features * spec.bytes_per_elem
        act_out = spec.tokens * spec.out_features * spec.bytes_per_elem
        w_bytes = spec.in_features * spec.out_features * spec.bytes_per_elem
        flops = 2.0 * spec.tokens * spec.in_features * spec.out_features * (3 if train else 1)
        nxt, nxt_out, nxt_mem = {}, {}, {}
        for ci, (kind, xs, ws, ys) in enumerate(_CANDIDATES):
            compute = flops / world / flops_per_s
            comm = 0.0
            if kind == "data" and train:
                comm += _copy_cost(_sbp.partial_sum, _sbp.broadcast, w_bytes, world) / link_bytes_per_s   # grad all-reduce
            params = spec.in_features * spec.out_features / (1 if kind == "data" else world)
            for pk, (cost, path) in best.items():
                mem = mem_used[pk] + params * state_bytes_per_param
                if mem_bytes_per_rank is not None and mem > mem_bytes_per_rank:
                    continue
                box = _copy_cost(prev_out[pk], xs, act_in, world) / link_bytes_per_s
                if train:   # the backward boxing is the transpose of the forward one
                    box += _copy_cost(xs if xs.kind != "B" else _sbp.partial_sum, prev_out[pk] if prev_out[pk].kind != "P" else _sbp.broadcast,
                                      act_in, world) / link_bytes_per_s
                total = cost + compute + comm + box
                key = ci + 1
                if key not in nxt or total < nxt[key][0]:
                    nxt[key] = (total, path + [Choice(spec.name, kind, xs, ws, ys)])
                    nxt_out[key] = ys
                    nxt_mem[key] = mem
        if not nxt:
            raise RuntimeError(f"auto-parallel: layer {spec.name} does not fit in memory under any signature")
        best, prev_out, mem_used = nxt, nxt_out, nxt_mem
    final = None
    for k, (cost, path) in best.items():
        act = layers[-1].tokens * layers[-1].out_features * layers[-1].bytes_per_elem
        if output_sbp is not None:
            cost = cost + _copy_cost(prev_out[k], output_sbp, act, world) / link_bytes_per_s
        elif prev_out[k].kind == "P":
            cost = cost + _copy_cost(prev_out[k], _sbp.split(0), act, world) / link_bytes_per_s
        if final is None or cost < final[0]:
            final = (cost, path)
    return final[1]


def apply_to_module(module, choices: Sequence[Choice], placement):
    """Re-distributes the ``weight`` / ``bias`` of the named Linear sub-modules according to ``choices``."""
    mods = dict(module.named_modules())
    for c in choices:
        m = mods[c.name]
        m.weight.data = m.weight.data.to_global(placement, c.w_sbp) if hasattr(m.weight.data, "to_global") else m.weight.data
        if getattr(m, "bias", None) is not None and hasattr(m.bias.data, "to_global"):
            b_sbp = _sbp.split(0) if c.kind == "column" else _sbp.broadcast
            m.bias.data = m.bias.data.to_global(placement, b_sbp)
    return module


# ------------------------------------------------------------------------------------------------ general SBP graphs
class SbpGraph:
    """A graph of operators, each with candidate SBP signatures, joined by tensors whose boxing has a price.

    ``add_node(name, costs)``: ``costs[i]`` = seconds of compute + the operator's own communication under candidate ``i``.
    ``add_edge(u, v, matrix)``: ``matrix[i][j]`` = seconds to box u's output under u's candidate ``i`` into what v's
    candidate ``j`` consumes. ``solve()`` returns the assignment with the least total cost, exactly, by the elimination
    scheme of the reference (oneflow/core/auto_parallel/sbp_graph.cpp: node elimination for nodes with one or two
    neighbours, edge elimination for parallel edges, node merging when neither applies):
      * parallel edges between the same two nodes add up;
      * a node with one neighbour folds into that neighbour's cost vector (minimum over its own candidates);
      * a node with two neighbours becomes an edge between them (minimum over its candidates of edge + node + edge);
      * if every remaining node has three or more neighbours, the node with the fewest candidates is merged into a
        neighbour (the pair becomes one node whose candidates are the pairs);
    every step records its argmin table, and the choices are read back in reverse order."""

    def __init__(self):
        self.costs = {}          # node -> list of float
        self.edges = {}          # frozenset({u, v}) -> (u, v, matrix[i_u][j_v])
        self.order = []

    def add_node(self, name, costs):
        if name in self.costs:
            raise ValueError(f"duplicate node {name}")
        self.costs[name] = [float(c) for c in costs]
        self.order.append(name)

    def add_edge(self, u, v, matrix):
        if u == v:
            raise ValueError("self edges are not allowed")
        m = [[float(x) for x in row] for row in matrix]
        if len(m) != len(self.costs[u]) or any(len(r) != len(self.costs[v]) for r in m):
            raise ValueError(f"edge {u}->{v}: matrix shape does not match the candidate counts")
        key = frozenset((u, v))
        if key in self.edges:
            a, b, old = self.edges[key]
            if a != u:
                m = [[m[j][i] for j in range(len(m))] for i in range(len(m[0]))]
            self.edges[key] = (a, b, [[x + y for x, y in zip(r0, r1)] for r0, r1 in zip(old, m)])
        else:
            self.edges[key] = (u, v, m)

    def _matrix(self, edges, u, v):
        """Cost matrix indexed [candidate of u][candidate of v]."""
        a, b, m = edges[frozenset((u, v))]
        return m if a == u else [[m[j][i] for j in range(len(m))] for i in range(len(m[0]))]

    def solve(self):
        costs = {k: list(v) for k, v in self.costs.items()}
        edges = dict(self.edges)
        members = {k: [k] for k in costs}            # merged nodes: which original nodes a node stands for
        decode = {k: [(i,) for i in range(len(v))] for k, v in costs.items()}   # candidate -> tuple of original choices
        trail = []

        def neighbours(n):
            return [next(iter(k - {n})) for k in edges if n in k]

        while len(costs) > 1:
            n = next((x for x in costs if len(neighbours(x)) == 0), None)
            if n is not None:                         # an isolated component: settle it on its own
                best = min(range(len(costs[n])), key=costs[n].__getitem__)
                trail.append(("fixed", n, best, costs[n][best]))
                del costs[n]
                continue
            n = next((x for x in costs if len(neighbours(x)) == 1), None)
            if n is not None:
                u = neighbours(n)[0]
                m = self._matrix(edges, u, n)
                arg = []
                for i in range(len(costs[u])):
                    j = min(range(len(costs[n])), key=lambda j: m[i][j] + costs[n][j])
                    costs[u][i] += m[i][j] + costs[n][j]
                    arg.append(j)
                trail.append(("leaf", n, u, arg))
                del edges[frozenset((u, n))], costs[n]
                continue
            n = next((x for x in costs if len(neighbours(x)) == 2), None)
            if n is not None:
                u, w = neighbours(n)
                mu, mw = self._matrix(edges, u, n), self._matrix(edges, n, w)
                new = [[0.0] * len(costs[w]) for _ in costs[u]]
                arg = [[0] * len(costs[w]) for _ in costs[u]]
                for i in range(len(costs[u])):
                    for k in range(len(costs[w])):
                        j = min(range(len(costs[n])), key=lambda j: mu[i][j] + costs[n][j] + mw[j][k])
                        new[i][k] = mu[i][j] + costs[n][j] + mw[j][k]
                        arg[i][k] = j
                trail.append(("series", n, u, w, arg))
                del edges[frozenset((u, n))], edges[frozenset((n, w))], costs[n]
                key = frozenset((u, w))
                if key in edges:
                    old = self._matrix(edges, u, w)
                    new = [[x + y for x, y in zip(r0, r1)] for r0, r1 in zip(old, new)]
                edges[key] = (u, w, new)
                continue
            # every node has >= 3 neighbours: merge the one with the fewest candidates into one of its neighbours
            n = min(costs, key=lambda x: (len(costs[x]), len(neighbours(x))))
            u = min(neighbours(n), key=lambda x: len(costs[x]))
            m = self._matrix(edges, u, n)
            name = ("merged", u, n)
            pairs = [(i, j) for i in range(len(costs[u])) for j in range(len(costs[n]))]
            costs[name] = [costs[u][i] + costs[n][j] + m[i][j] for i, j in pairs]
            del edges[frozenset((u, n))]
            for old_node, pos in ((u, 0), (n, 1)):
                for x in neighbours(old_node):
                    mx = self._matrix(edges, old_node, x)
                    del edges[frozenset((old_node, x))]
                    add = [[mx[p[pos]][k] for k in range(len(costs[x]))] for p in pairs]
                    key = frozenset((name, x))
                    if key in edges:
                        prev = self._matrix(edges, name, x)
                        add = [[a + b for a, b in zip(r0, r1)] for r0, r1 in zip(prev, add)]
                    edges[key] = (name, x, add)
            trail.append(("merge", name, u, n, pairs))
            del costs[u], costs[n]
        choice = {}
        total = 0.0
        if costs:
            last = next(iter(costs))
            choice[last] = min(range(len(costs[last])), key=costs[last].__getitem__)
            total = costs[last][choice[last]]
        for step in reversed(trail):
            if step[0] == "fixed":
                choice[step[1]] = step[2]
                total += step[3]
            elif step[0] == "leaf":
                _, n, u, arg = step
                choice[n] = arg[choice[u]]
            elif step[0] == "series":
                _, n, u, w, arg = step
                choice[n] = arg[choice[u]][choice[w]]
            else:
                _, name, u, n, pairs = step
                choice[u], choice[n] = pairs[choice.pop(name)]
        return {k: choice[k] for k in self.order}, total

    def cost_of(self, choice):
        total = sum(self.costs[n][choice[n]] for n in self.costs)
        for u, v, m in self.edges.values():
            total += m[choice[u]][choice[v]]
        return total


@dataclass
class Signature:
    kind: str                    # "data", "column", "row", "split0", "broadcast", "split_last", "partial", "vocab"
    ins: tuple                   # SBP each tensor input must arrive in
    out: object                  # SBP of the output
    params: dict                 # parameter name -> SBP
    cost: float = 0.0            # seconds: compute + the signature's own communication (gradient all-reduce)


def plan_module(module, example_inputs, world, *, flops_per_s=1.4e15, link_bytes_per_s=7.7e11, train=True, bytes_per_elem=2,
                input_sbp=None, output_sbp=None):
    """Auto-parallel for an arbitrary ``torch.nn.Module``: traces it (torch.fx) on the example inputs, gives every operator
    its candidate SBP signatures, prices every tensor between two operators with the boxing cost model, and solves the
    resulting SBP graph exactly. Returns ``(plan, total_seconds)`` where ``plan`` maps each node name of the trace to its
    ``Signature``; ``plan.param_sbp`` maps parameter names (``"fc1.weight"``) to their SBP. 1-D placement of ``world`` ranks.

    Reference: oneflow/core/auto_parallel/sbp_constructor.cpp (one SbpNode per op with its signature list, one SbpEdge per
    consumed tensor with the copy cost between every pair of signatures), sbp_collector.cpp."""
    import operator

    import torch
    import torch.fx
    from torch.fx.passes.shape_prop import ShapeProp

    if torch.is_tensor(example_inputs):
        example_inputs = (example_inputs,)
    leaf_types = (torch.nn.Linear, torch.nn.Embedding, torch.nn.LayerNorm, torch.nn.Softmax, torch.nn.ReLU, torch.nn.GELU, torch.nn.Tanh,
                  torch.nn.Sigmoid, torch.nn.SiLU, torch.nn.Dropout, torch.nn.Identity)

    class _Tracer(torch.fx.Tracer):
        def is_leaf_module(self, m, qualname):
            # this framework's own layers derive from torch's: they are leaves too, whatever module they are defined in
            return isinstance(m, leaf_types) or super().is_leaf_module(m, qualname)

    gm = torch.fx.GraphModule(module, _Tracer().trace(module))
    ShapeProp(gm).propagate(*example_inputs)
    S0, B, P = _sbp.split(0), _sbp.broadcast, _sbp.partial_sum
    mult = 3.0 if train else 1.0
    mods = dict(gm.named_modules())

    def meta(n):
        tm = n.meta.get("tensor_meta")
        return tm if hasattr(tm, "shape") else None

    def nbytes(n):
        tm = meta(n)
        if tm is None:
            return 0
        k = 1
        for d in tm.shape:
            k *= int(d)
        return k * bytes_per_elem

    def last(n):
        return _sbp.split(len(meta(n).shape) - 1)

    def grad_sync(param_bytes):
        return _copy_cost(P, B, param_bytes, world) / link_bytes_per_s if train else 0.0

    def tensor_args(n):
        return [a for a in n.all_input_nodes if meta(a) is not None]

    pointwise_fn = {torch.relu, torch.tanh, torch.sigmoid, torch.nn.functional.relu, torch.nn.functional.gelu, torch.nn.functional.silu,
                    torch.nn.functional.dropout, operator.neg}
    pointwise_mod = (torch.nn.ReLU, torch.nn.GELU, torch.nn.Tanh, torch.nn.Sigmoid, torch.nn.SiLU, torch.nn.Dropout, torch.nn.Identity)
    rowwise_mod = (torch.nn.LayerNorm, torch.nn.Softmax)
    binary_fn = {operator.add: True, torch.add: True, operator.sub: True, torch.sub: True, operator.mul: False, torch.mul: False,
                 operator.truediv: False}

    sigs = {}
    for n in gm.graph.nodes:
        if n.op == "output" or (n.op != "placeholder" and meta(n) is None):
            continue
        ins = tensor_args(n)
        rank = len(meta(n).shape) if meta(n) is not None else 0
        cands = []
        if n.op == "placeholder":
            fixed = input_sbp if input_sbp is not None else None
            for s in ([fixed] if fixed is not None else [S0, B]):
                cands.append(Signature("input", (), s, {}, 0.0))
        elif n.op == "get_attr":
            cands.append(Signature("broadcast", (), B, {}, 0.0))
        elif n.op == "call_module" and isinstance(mods[n.target], torch.nn.Linear):
            m = mods[n.target]
            tokens = nbytes(n) // bytes_per_elem // m.out_features
            fl = 2.0 * tokens * m.in_features * m.out_features * mult / world / flops_per_s
            wb = m.in_features * m.out_features * bytes_per_elem
            pw, pb = f"{n.target}.weight", f"{n.target}.bias"
            has_b = m.bias is not None
            cands.append(Signature("data", (S0,), S0, {pw: B, **({pb: B} if has_b else {})}, fl + grad_sync(wb)))
            cands.append(Signature("column", (B,), last(n), {pw: S0, **({pb: S0} if has_b else {})}, fl))
            cands.append(Signature("row", (_sbp.split(len(meta(ins[0]).shape) - 1),), P, {pw: _sbp.split(1), **({pb: B} if has_b else {})}, fl))
        elif n.op == "call_module" and isinstance(mods[n.target], torch.nn.Embedding):
            m = mods[n.target]
            tb = m.num_embeddings * m.embedding_dim * bytes_per_elem
            pw = f"{n.target}.weight"
            cands.append(Signature("data", (S0,), S0, {pw: B}, grad_sync(tb)))
            cands.append(Signature("vocab", (B,), P, {pw: S0}, 0.0))
            cands.append(Signature("column", (B,), last(n), {pw: _sbp.split(1)}, 0.0))
        elif (n.op == "call_module" and isinstance(mods[n.target], rowwise_mod)) or \
                (n.op == "call_function" and n.target in (torch.softmax, torch.nn.functional.softmax, torch.nn.functional.layer_norm)):
            params = {}
            if n.op == "call_module":
                params = {f"{n.target}.{k}": B for k, _ in mods[n.target].named_parameters(recurse=False)}
                pbytes = sum(p.numel() for p in mods[n.target].parameters(recurse=False)) * bytes_per_elem
            else:
                pbytes = 0
            cands.append(Signature("split0", (S0,) * len(ins), S0, params, grad_sync(pbytes)))
            cands.append(Signature("broadcast", (B,) * len(ins), B, params, 0.0))
        elif (n.op == "call_module" and isinstance(mods[n.target], pointwise_mod)) or (n.op == "call_function" and n.target in pointwise_fn) or \
                (n.op == "call_method" and n.target in ("relu", "tanh", "sigmoid", "contiguous", "clone", "float", "to")):
            cands.append(Signature("split0", (S0,) * len(ins), S0, {}, 0.0))
            cands.append(Signature("broadcast", (B,) * len(ins), B, {}, 0.0))
            if rank >= 2:
                cands.append(Signature("split_last", (last(n),) * len(ins), last(n), {}, 0.0))
        elif n.op == "call_function" and n.target in binary_fn and len(ins) == 2 and tuple(meta(ins[0]).shape) == tuple(meta(ins[1]).shape):
            cands.append(Signature("split0", (S0, S0), S0, {}, 0.0))
            cands.append(Signature("broadcast", (B, B), B, {}, 0.0))
            if rank >= 2:
                cands.append(Signature("split_last", (last(n), last(n)), last(n), {}, 0.0))
            if binary_fn[n.target]:
                cands.append(Signature("partial", (P, P), P, {}, 0.0))
        else:
            # anything else (reshapes, attention cores, reductions ...) keeps the batch split or runs replicated
            cands.append(Signature("split0", (S0,) * len(ins), S0, {}, 0.0))
            cands.append(Signature("broadcast", (B,) * len(ins), B, {}, 0.0))
        sigs[n] = cands

    g = SbpGraph()
    for n, cands in sigs.items():
        g.add_node(n.name, [c.cost for c in cands])
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    results = [a for a in out_node.all_input_nodes if a in sigs]
    for n, cands in sigs.items():
        for k, a in enumerate(tensor_args(n)):
            if a not in sigs:
                continue
            nb = nbytes(a)
            mat = []
            for ca in sigs[a]:
                row = []
                for cn in cands:
                    want = cn.ins[k] if k < len(cn.ins) else B
                    c = _copy_cost(ca.out, want, nb, world) / link_bytes_per_s
                    if train and ca.out != want:       # the gradient travels the transposed route
                        back_from = P if want.kind == "B" else want
                        back_to = B if ca.out.kind == "P" else ca.out
                        c += _copy_cost(back_from, back_to, nb, world) / link_bytes_per_s
                    row.append(c)
                mat.append(row)
            g.add_edge(a.name, n.name, mat)
    # the results leave as output_sbp (default: whatever is not a partial sum)
    for r in results:
        extra = []
        for c in sigs[r]:
            want = output_sbp if output_sbp is not None else (S0 if c.out.kind == "P" else c.out)
            extra.append(_copy_cost(c.out, want, nbytes(r), world) / link_bytes_per_s)
        g.costs[r.name] = [a + b for a, b in zip(g.costs[r.name], extra)]
    choice, total = g.solve()

    class Plan(dict):
        pass
    plan = Plan()
    plan.param_sbp = {}
    plan.graph = g
    for n, cands in sigs.items():
        s = cands[choice[n.name]]
        plan[n.name] = s
        plan.param_sbp.update(s.params)
    return plan, total


def apply_plan(module, plan, placement):
    """Distributes the parameters of ``module`` as ``plan.param_sbp`` says. Parameters that are global tensors already (on a 1-D
    placement) are re-boxed in place; local parameters become global tensors on ``placement``."""
    from . import global_tensor as GT
    params = dict(module.named_parameters())
    for name, s in plan.param_sbp.items():
        p = params.get(name)
        if p is None:
            continue
        if isinstance(p, GT.GlobalTensor):
            if list(p.sbp) != [s]:
                new = GT.rebox(p.detach(), [s])
                p._local, p._nd_sbp = new._local, new._nd_sbp
        else:
            p.data = GT.rebox(GT.to_global(p.data, placement, [_sbp.broadcast]), [s])
    return module
