"""Lazy random values for tests: a generator is drawn once per test iteration (``value()``), combines with ``+ - * |``
and takes the type it should produce from ``.to(type)`` or from the annotation of the parameter it is passed to."""
from __future__ import annotations

import os
import typing

import numpy as np
import torch as _torch

_seed = os.getenv("ONEFLOW_TEST_SEED")
rng = np.random.default_rng(int(_seed) if _seed else None)

_state = {"global": False}


def is_global():
    return _state["global"]


def _broadcast_obj(v):
    """In global tests every rank must draw the same values: rank 0's are sent to all."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        return v
    box = [v]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class generator:
    def __init__(self, children=()):
        self.children = [c for c in children if isinstance(c, generator)]
        self._value, self._has = None, False

    def reset(self):
        self._value, self._has = None, False
        for c in self.children:
            c.reset()

    def eval(self):
        self.reset()
        return self.value()

    def value(self):
        if not self._has:
            v = self._draw()
            self._value, self._has = (_broadcast_obj(v) if is_global() else v), True
        return self._value

    def _draw(self):
        raise NotImplementedError

    def size(self):
        return 1

    def to(self, annotation):
        self._to(annotation)
        for c in self.children:
            c.to(annotation)
        return self

    def _to(self, annotation):
        pass

    def __or__(self, other):
        other = pack(other)
        return oneof(self, other, possibility=self.size() / (self.size() + other.size()))

    __ror__ = __or__

    def __add__(self, other):
        return _binary(self, other, lambda a, b: a + b)

    __radd__ = __add__

    def __sub__(self, other):
        return _binary(self, other, lambda a, b: a - b)

    def __rsub__(self, other):
        return _binary(other, self, lambda a, b: a - b)

    def __mul__(self, other):
        return _binary(self, other, lambda a, b: a * b)

    __rmul__ = __mul__

    def __neg__(self):
        return _binary(0, self, lambda a, b: a - b)


def pack(x):
    if isinstance(x, generator):
        return x
    if isinstance(x, (list, tuple)):
        return tuple_(*x)
    return constant(x)


class _binary(generator):
    def __init__(self, a, b, fn):
        self.a, self.b, self.fn = pack(a), pack(b), fn
        super().__init__([self.a, self.b])

    def _draw(self):
        return self.fn(self.a.value(), self.b.value())


class constant(generator):
    def __init__(self, x):
        super().__init__()
        self.x = x

    def _draw(self):
        return self.x


class Nothing:
    """Marks an argument that is to be left out of the call."""


class nothing(generator):
    def _draw(self):
        return Nothing()


class tuple_(generator):
    def __init__(self, *items):
        self.items = [pack(i) for i in items]
        super().__init__(self.items)

    def _draw(self):
        return tuple(i.value() for i in self.items)


class oneof(generator):
    def __init__(self, *args, possibility=None):
        self.args = [pack(a) for a in args]
        super().__init__(self.args)
        if isinstance(possibility, float):
            if len(args) != 2:
                raise ValueError("a single possibility needs exactly two alternatives")
            possibility = [possibility, 1 - possibility]
        if possibility is None:
            possibility = [1 / len(args)] * len(args)
        self.possibility = [p.value() if isinstance(p, generator) else p for p in possibility]

    def _draw(self):
        i = int(rng.choice(len(self.args), p=np.asarray(self.possibility) / np.sum(self.possibility)))
        return self.args[i].value()

    def size(self):
        return sum(a.size() for a in self.args)


def _concrete(annotation):
    """Reduce typing constructs to something ``random`` can draw: Optional[int] -> int, Union -> first member,
    Tuple[int, int] -> ("tuple", [int, int])."""
    origin = typing.get_origin(annotation)
    if origin is typing.Union:
        args = [a for a in typing.get_args(annotation) if a is not type(None)]
        return _concrete(args[int(rng.integers(0, len(args)))]) if args else None
    if origin in (tuple, typing.Tuple):
        return ("tuple", [_concrete(a) for a in typing.get_args(annotation) if a is not Ellipsis])
    return annotation


class random(generator):
    def __init__(self, low=1, high=6):
        self.low, self.high = pack(low), pack(high)
        super().__init__([self.low, self.high])
        self.annotation = None

    def _to(self, annotation):
        if self.annotation is None:
            self.annotation = annotation

    def _one(self, ann):
        low, high = self.low.value(), self.high.value()
        if isinstance(ann, tuple) and ann and ann[0] == "tuple":
            return [self._one(a) for a in ann[1]]
        if ann is int:
            return int(rng.integers(low, high))
        if ann is bool:
            return bool(rng.integers(0, 2))
        if ann is complex:
            return complex(rng.random() * (high - low) + low, rng.random() * (high - low) + low)
        if ann is None or ann is type(None):
            return None              # no type known (an un-annotated parameter): the argument is passed as None
        if ann is float:
            return float(rng.random() * (high - low) + low)
        raise NotImplementedError(f"random values of type {ann}")

    def _draw(self):
        return self._one(_concrete(self.annotation))


def random_or_nothing(low, high):
    return oneof(random(low, high), nothing(), possibility=2 / 3)


def random_bool():
    return random().to(bool)


_DEFAULT_RANGE = {int: (-10, 11), float: (0, 1), complex: (-10, 10)}


class random_pytorch_tensor(generator):
    def __init__(self, ndim=None, dim0=1, dim1=None, dim2=None, dim3=None, dim4=None, low=None, high=None, dtype=float,
                 pin_memory=False):
        dims = [dim0, dim1, dim2, dim3, dim4]
        self.ndim = pack(random(1, 6) if ndim is None else ndim).to(int)
        self.dims = [pack(random(1, 8) if d is None else d).to(int) for d in dims]
        self.low, self.high, self.dtype, self.pin_memory = pack(low).to(float), pack(high).to(float), pack(dtype), pin_memory
        super().__init__([self.ndim] + self.dims + [self.low, self.high, self.dtype])

    def _draw(self):
        ndim, dtype = self.ndim.value(), self.dtype.value()
        low, high = self.low.value(), self.high.value()
        low = _DEFAULT_RANGE[dtype][0] if low is None else low
        high = _DEFAULT_RANGE[dtype][1] if high is None else high
        shape = [self.dims[i].value() if i < 5 else int(rng.integers(1, 8)) for i in range(ndim)]
        if dtype is float:
            return _torch.tensor(rng.uniform(low, high, size=shape), dtype=_torch.float32)
        if dtype is int:
            return _torch.tensor(rng.integers(int(low), int(high), size=shape), dtype=_torch.int64)
        if dtype is complex:
            return _torch.tensor(rng.uniform(low, high, size=shape) + 1j * rng.uniform(low, high, size=shape), dtype=_torch.complex64)
        raise NotImplementedError(f"random tensors of {dtype}")


class choice_pytorch_tensor(generator):
    def __init__(self, a, size=None, replace=True, p=None, dtype=int):
        super().__init__()
        self.a, self.size_, self.replace, self.p, self.dtype = a, size, replace, p, dtype

    def _draw(self):
        arr = rng.choice(self.a, self.size_, self.replace, self.p)
        return _torch.tensor(arr, dtype={int: _torch.int64, float: _torch.float32}.get(self.dtype, self.dtype))


class random_device(generator):
    def _draw(self):
        if os.getenv("ONEFLOW_TEST_CPU_ONLY") or not _torch.cuda.is_available():
            return "cpu"
        return ["cpu", "cuda"][int(rng.integers(0, 2))]


class cpu_device(generator):
    def _draw(self):
        return "cpu"


class gpu_device(generator):
    def _draw(self):
        return "cuda" if _torch.cuda.is_available() and not os.getenv("ONEFLOW_TEST_CPU_ONLY") else "cpu"


_DTYPE_SEQS = {
    "int": [_torch.int8, _torch.int16, _torch.int32, _torch.int64], "unsigned": [_torch.uint8], "signed": [_torch.int8, _torch.int16, _torch.int32, _torch.int64],
    "arithmetic": [_torch.int8, _torch.int32, _torch.int64, _torch.float32, _torch.float64], "float": [_torch.float32, _torch.float64],
    "half": [_torch.float16], "bfloat16": [_torch.bfloat16], "bool": [_torch.bool], "complex": [_torch.complex64, _torch.complex128],
    "pod": [_torch.int8, _torch.uint8, _torch.int32, _torch.int64, _torch.float32, _torch.float64, _torch.bool],
}
_DTYPE_SEQS["index"] = [_torch.int32, _torch.int64]
_DTYPE_SEQS["image"] = [_torch.uint8, _torch.float32]


class random_pytorch_dtype(generator):
    def __init__(self, seq_names):
        super().__init__()
        self.choices = [d for n in seq_names for d in _DTYPE_SEQS[n]]

    def _draw(self):
        return self.choices[int(rng.integers(0, len(self.choices)))]


# ------------------------------------------------------------------------------------------------ placements and sbp
def _all_ranks():
    import torch.distributed as dist
    return list(range(dist.get_world_size())) if dist.is_available() and dist.is_initialized() else [0]


class all_placement(generator):
    """Iterable of placements over all ranks: 1-D, and 2-D when the world factors as 2 x n."""

    def __init__(self):
        super().__init__()
        self.devices = ["cpu"] + (["cuda"] if _torch.cuda.is_available() and not os.getenv("ONEFLOW_TEST_CPU_ONLY") else [])

    def _all(self):
        import oneflow_b200 as flow
        ranks = _all_ranks()
        out = []
        for dev in self.devices:
            out.append(flow.placement(dev, ranks))
            if len(ranks) >= 4 and len(ranks) % 2 == 0:
                out.append(flow.placement(dev, [ranks[:len(ranks) // 2], ranks[len(ranks) // 2:]]))
        return out

    def __iter__(self):
        return iter(self._all())

    def _draw(self):
        return self._all()


class all_cpu_placement(all_placement):
    def __init__(self):
        super().__init__()
        self.devices = ["cpu"]


class all_cuda_placement(all_placement):
    def __init__(self):
        super().__init__()
        self.devices = ["cuda"]


class random_placement(all_placement):
    def _draw(self):
        a = self._all()
        return a[int(rng.integers(0, len(a)))]


class random_cpu_placement(random_placement):
    def __init__(self):
        super().__init__()
        self.devices = ["cpu"]


class random_gpu_placement(random_placement):
    def __init__(self):
        super().__init__()
        self.devices = ["cuda"]


class all_sbp(generator):
    """All nd-sbp tuples for a placement: per mesh axis one of split(i) for i < ``max_dim`` (restricted to
    ``valid_split_axis`` when given), broadcast and partial-sum, minus the kinds excluded.  ``max_dim`` 0 (a scalar)
    leaves broadcast only.  Iterable, indexable and sized."""

    def __init__(self, placement=None, dim=1, max_dim=0, except_split=False, except_broadcast=False, except_partial_sum=False,
                 valid_split_axis=None):
        super().__init__()
        if placement is not None:
            pl = placement.value() if isinstance(placement, generator) else placement
            self.dim = len(pl.hierarchy)
        else:
            self.dim = dim
        self.max_dim = max_dim
        self.except_split, self.except_broadcast, self.except_partial_sum = except_split, except_broadcast, except_partial_sum
        if valid_split_axis is None:
            self.valid_split_axis = list(range(max_dim))
        else:
            self.valid_split_axis = [valid_split_axis] if isinstance(valid_split_axis, int) else list(valid_split_axis)

    def _all(self):
        import itertools
        import oneflow_b200 as flow
        if self.max_dim == 0:
            return [tuple(flow.sbp.broadcast for _ in range(self.dim))]
        kinds = []
        if not self.except_split:
            kinds += [flow.sbp.split(i) for i in range(self.max_dim) if i in self.valid_split_axis]
        if not self.except_broadcast:
            kinds.append(flow.sbp.broadcast)
        if not self.except_partial_sum:
            kinds.append(flow.sbp.partial_sum)
        return [tuple(c) for c in itertools.product(kinds, repeat=self.dim)]

    def __iter__(self):
        return iter(self._all())

    def __len__(self):
        return len(self._all())

    def __getitem__(self, key):
        return self._all()[key]

    def _draw(self):
        return self._all()


class random_sbp(all_sbp):
    def _draw(self):
        a = self._all()
        return a[int(rng.integers(0, len(a)))]


__all__ = ["random_pytorch_tensor", "random_bool", "random_device", "random_pytorch_dtype", "cpu_device", "gpu_device",
           "random_placement", "random_cpu_placement", "random_gpu_placement", "all_placement", "all_cpu_placement",
           "all_cuda_placement", "random_sbp", "all_sbp", "random", "random_or_nothing", "oneof", "constant", "nothing",
           "choice_pytorch_tensor", "generator", "Nothing", "rng", "is_global"]
