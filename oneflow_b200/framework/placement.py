"""``flow.placement(type, ranks)``: device type + ranks, a nested rank list giving an n-D hierarchy
(reference: oneflow/api/python/symbol/placement_symbol.cpp:143-185, oneflow/core/job/placement.proto).
Process groups for a placement and for each of its mesh axes are created lazily and cached; creation is
collective over the world, as the reference's communicator manager requires every participating rank to
take part in the same order (oneflow/core/job/eager_nccl_comm_manager.cpp:54-80)."""
from __future__ import annotations

import itertools

import torch
import torch.distributed as dist


def _shape_of(nested):
    shape = []
    cur = nested
    while isinstance(cur, (list, tuple)):
        shape.append(len(cur))
        cur = cur[0] if len(cur) else None
    return tuple(shape)


def _flatten(nested):
    if isinstance(nested, (list, tuple)):
        for x in nested:
            yield from _flatten(x)
    else:
        yield int(nested)


_GROUP_CACHE = {}


def group_for_ranks(ranks):
    """Process group over exactly these global ranks. Only the member ranks create it (group-local synchronisation), each
    when it first needs it: ranks outside a placement (other pipeline stages) never have to take part. The members
    reach the creation in the same order because they run the same program on the same global tensors."""
    ranks = tuple(ranks)
    if not dist.is_initialized():
        return None
    if ranks == tuple(range(dist.get_world_size())):
        return dist.group.WORLD
    if dist.get_rank() not in ranks:
        return None
    g = _GROUP_CACHE.get(ranks)
    if g is None:
        g = dist.new_group(list(ranks), use_local_synchronization=True)
        _GROUP_CACHE[ranks] = g
    return g


class placement:
    def __init__(self, type="cpu", ranks=None, device_type=None):
        if device_type is not None:
            type = device_type
        if isinstance(type, torch.device):
            type = type.type
        if getattr(type, "type", None) == "mock":
            type = "mock"
        if type not in ("cpu", "cuda", "mock"):      # "mock": the pseudo device kind for tests, host memory behind it
            raise ValueError(f"unknown device type {type!r}")
        if ranks is None:
            ranks = list(range(dist.get_world_size() if dist.is_initialized() else 1))
        if isinstance(ranks, range):
            ranks = list(ranks)
        if hasattr(ranks, "tolist"):
            ranks = ranks.tolist()
        self.type = type
        self.hierarchy = _shape_of(ranks) or (1,)
        self.ranks_flat = tuple(_flatten(ranks))
        if len(set(self.ranks_flat)) != len(self.ranks_flat):
            raise ValueError("placement ranks must be unique")
        n = 1
        for d in self.hierarchy:
            n *= d
        if n != len(self.ranks_flat):
            raise ValueError("ragged rank list")
        self._nested = ranks

    # -- reference-compatible surface
    @property
    def ranks(self):
        import numpy as np
        return np.array(self.ranks_flat).reshape(self.hierarchy)

    @property
    def device_type(self):
        return self.type

    @staticmethod
    def all(device_type="cpu"):
        return placement(device_type, list(range(dist.get_world_size() if dist.is_initialized() else 1)))

    @property
    def ndim(self):
        return len(self.hierarchy)

    @property
    def size(self):
        return len(self.ranks_flat)

    def __eq__(self, other):
        return (isinstance(other, placement) and self.type == other.type and self.hierarchy == other.hierarchy
                and self.ranks_flat == other.ranks_flat)

    def __hash__(self):
        return hash((self.type, self.hierarchy, self.ranks_flat))

    def __repr__(self):
        return f'oneflow.placement(type="{self.type}", ranks={self.ranks.tolist()})'

    def __getstate__(self):
        return {"type": self.type, "ranks": self.ranks.tolist()}

    def __setstate__(self, st):
        self.__init__(st["type"], st["ranks"])

    # -- mesh helpers
    def contains(self, rank):
        return rank in self.ranks_flat

    def coords(self, rank):
        """Mesh coordinates of a global rank (None if it is outside the placement)."""
        if rank not in self.ranks_flat:
            return None
        idx = self.ranks_flat.index(rank)
        out = []
        for d in reversed(self.hierarchy):
            out.append(idx % d)
            idx //= d
        return tuple(reversed(out))

    def rank_at(self, coords):
        idx = 0
        for c, d in zip(coords, self.hierarchy):
            idx = idx * d + c
        return self.ranks_flat[idx]

    def axis_ranks(self, axis, rank):
        """Global ranks that differ from `rank` only in mesh coordinate `axis` (the 1-D sub-group)."""
        c = list(self.coords(rank))
        out = []
        for i in range(self.hierarchy[axis]):
            c[axis] = i
            out.append(self.rank_at(c))
        return out

    def group(self):
        return group_for_ranks(self.ranks_flat)

    def axis_group(self, axis):
        """Sub-group of the calling rank along one mesh axis (None on ranks outside the placement)."""
        if not dist.is_initialized():
            return None
        me = dist.get_rank()
        if me not in self.ranks_flat:
            return None
        return group_for_ranks(self.axis_ranks(axis, me))

    def device(self):
        if self.type in ("cpu", "mock"):
            return torch.device("cpu")
        return torch.device("cuda", torch.cuda.current_device())
