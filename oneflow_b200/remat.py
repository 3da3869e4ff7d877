"""``flow.remat``: the memory budget of rematerialisation (reference: python/oneflow/remat/__init__.py:21-54).
Activation memory is bounded here by explicit recomputation (``flow.utils.checkpoint`` and the engines' layer-wise
recompute), not by dynamic eviction, so the budget is recorded and reported and nothing is evicted behind the caller's back."""
import re

_state = {"budget": None, "small_pieces": True}


def parse_size(size):
    units = {"B": 1, "KB": 2 ** 10, "MB": 2 ** 20, "GB": 2 ** 30, "TB": 2 ** 40, "": 1,
             "KIB": 10 ** 3, "MIB": 10 ** 6, "GIB": 10 ** 9, "TIB": 10 ** 12}
    m = re.match(r"^([\d\.]+)\s*([a-zA-Z]{0,3})$", str(size).strip())
    if m is None or m.group(2).upper() not in units:
        raise ValueError(f"cannot parse size {size!r}")
    return int(float(m.group(1)) * units[m.group(2).upper()])


def set_budget(budget):
    _state["budget"] = parse_size(budget)


def get_budget():
    return _state["budget"]


def set_small_pieces_optimization(mode=True):
    _state["small_pieces"] = bool(mode)


def is_small_pieces_optimization_enabled():
    return _state["small_pieces"]


def is_enabled():
    return _state["budget"] is not None
