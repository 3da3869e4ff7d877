"""``flow.sbp``: split(axis) / broadcast / partial_sum descriptors of how a global tensor is laid out
over one axis of its placement (reference: python/oneflow/sbp.py:17-22,
oneflow/core/job/sbp_parallel.proto:47-72). Instances are interned; they pickle as
``("S", axis) | ("B", -1) | ("P", -1)`` like the reference's sbp symbols
(oneflow/api/python/symbol/sbp_symbol.cpp:62-106)."""
from __future__ import annotations


class sbp:
    _cache = {}
    __slots__ = ("kind", "axis")

    def __new__(cls, kind, axis=-1):
        key = (kind, axis if kind == "S" else -1)
        inst = cls._cache.get(key)
        if inst is None:
            inst = object.__new__(cls)
            object.__setattr__(inst, "kind", key[0])
            object.__setattr__(inst, "axis", key[1])
            cls._cache[key] = inst
        return inst

    def __setattr__(self, *a):
        raise AttributeError("sbp objects are immutable")

    def __reduce__(self):
        return (_rebuild, (self.kind, self.axis))

    def __getstate__(self):
        return (self.kind, self.axis)

    def __call__(self):
        """``flow.sbp.broadcast()`` / ``flow.sbp.split(0)()``: the symbol itself (both spellings are in use)."""
        return self

    def is_split(self):
        return self.kind == "S"

    def is_broadcast(self):
        return self.kind == "B"

    def is_partial_sum(self):
        return self.kind == "P"

    def __repr__(self):
        if self.kind == "S":
            return f"oneflow.sbp.split(dim={self.axis})"
        return "oneflow.sbp.broadcast" if self.kind == "B" else "oneflow.sbp.partial_sum"

    def __str__(self):
        return f"S({self.axis})" if self.kind == "S" else self.kind


def _rebuild(kind, axis):
    return sbp(kind, axis)


def split(dim=None, axis=None):
    d = dim if dim is not None else axis
    if d is None or int(d) < 0:
        raise ValueError("split needs a non-negative axis")
    return sbp("S", int(d))


broadcast = sbp("B")
partial_sum = sbp("P")


def normalize(s, ndim_mesh=1):
    """Accepts one sbp, a sequence of sbp, or strings like "S(0)"/"B"/"P"; returns a tuple of length ndim_mesh."""
    if isinstance(s, (sbp, str)):
        s = (s,)
    out = []
    for x in s:
        if isinstance(x, str):
            x = x.strip()
            if x in ("B", "broadcast"):
                x = broadcast
            elif x in ("P", "partial_sum"):
                x = partial_sum
            elif x.startswith("S(") and x.endswith(")"):
                x = split(int(x[2:-1]))
            else:
                raise ValueError(f"cannot parse sbp {x!r}")
        if not isinstance(x, sbp):
            raise TypeError(f"expected an sbp, got {type(x)}")
        out.append(x)
    if len(out) != ndim_mesh:
        raise ValueError(f"placement has {ndim_mesh} mesh axes but {len(out)} sbp were given")
    return tuple(out)
