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
