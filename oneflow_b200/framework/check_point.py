"""``flow.save`` / ``flow.load`` in the reference's checkpoint format.

* single file: pickle of ``{"protocol_version": 1, "__oneflow__": None, "data": obj}``; tensors are
  pickled as ``oneflow.Tensor`` / ``oneflow.nn.Parameter`` objects whose state is
  ``{"data": ndarray, "dtype", "device"}`` (local) or ``{"data", "dtype", "placement", "sbp"}`` (global);
* ``save_as_external_data=True``: ``path`` is a directory with ``pickled_data`` plus one sub-directory
  per tensor holding the raw bytes (``out``) and a text-proto ``meta`` (``shape { dim: .. } data_type: kFloat``);
  tensor states are then ``{"path": <sub-directory>}``;
* legacy directories (``snapshot_done`` marker, one directory per variable) and ``torch.save`` files load too.

Class paths in the pickle stream (``oneflow.Tensor``, ``oneflow.nn.Parameter``,
``oneflow._oneflow_internal.dtype|placement|sbp.sbp``) are the reference's, provided by the ``oneflow``
alias package of this repository, so files written here load in the reference and vice versa.
Reference: python/oneflow/framework/check_point_v2.py (:53-58 meta, :197-210 tensor directories,
:300-355 tensor state, :435-459 legacy loader, :596-643 load, :683-741 save).
"""
from __future__ import annotations

import copyreg
import io
import os
import pickle
import re
import uuid
from collections import OrderedDict
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from .. import sbp as S
from . import dtype as D
from .placement import placement as Placement

PROTOCOL_VERSION = 1
PICKLE_FILENAME = "pickled_data"
DATA_FILENAME = "out"
META_FILENAME = "meta"
SNAPSHOT_DONE = "snapshot_done"


def _alias():
    """The ``oneflow`` alias package carries the classes named in the pickle stream."""
    import oneflow  # noqa: F401  (repository-local alias of oneflow_b200)
    import oneflow._oneflow_internal as internal
    return oneflow, internal


# ------------------------------------------------------------------------------------------------ tensors on disk
def _tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def _tensor_from_bytes(raw: bytes, shape, dt):
    if dt == torch.bfloat16:
        arr = np.frombuffer(raw, dtype=np.int16).copy()
        return torch.from_numpy(arr).view(torch.bfloat16).reshape(tuple(shape))
    arr = np.frombuffer(raw, dtype=D.to_numpy_dtype(dt)).copy()
    return torch.from_numpy(arr).reshape(tuple(shape))


def write_meta(path: Path, shape, dt):
    lines = ["shape {"] + [f"  dim: {int(d)}" for d in shape] + ["}", f"data_type: {D.PROTO_NAME_OF[dt]}", ""]
    path.write_text("\n".join(lines))


def read_meta(path: Path):
    txt = path.read_text()
    dims = [int(x) for x in re.findall(r"dim:\s*(-?\d+)", txt)]
    m = re.search(r"data_type:\s*(\w+)", txt)
    if not m:
        raise ValueError(f"{path}: no data_type")
    return tuple(dims), D.DTYPE_OF_PROTO_NAME[m.group(1)]


def save_tensor_dir(t: torch.Tensor, d: Path):
    d.mkdir(parents=True, exist_ok=True)
    (d / DATA_FILENAME).write_bytes(_tensor_bytes(t))
    write_meta(d / META_FILENAME, t.shape, t.dtype)


def load_tensor_dir(d: Path):
    shape, dt = read_meta(d / META_FILENAME)
    return _tensor_from_bytes((d / DATA_FILENAME).read_bytes(), shape, dt)


# ------------------------------------------------------------------------------------------------ pickling
class _Ctx:
    def __init__(self, path, global_rank, external, map_location=None):
        self.path, self.global_rank, self.external, self.map_location = path, global_rank, external, map_location
        self.counter = 0


def _to_numpy(t):
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.float().numpy()  # the reference's numpy() of a bfloat16 tensor yields float32 as well
    return t.numpy()


def _gather_global(t, dst_rank):
    from .global_tensor import to_global
    cpu_pl = Placement("cpu", t.placement.ranks.tolist())
    x = to_global(t.detach(), cpu_pl, t.sbp)
    x = to_global(x, Placement("cpu", [dst_rank]), (S.broadcast,))
    return x._local


def tensor_state(t, ctx: _Ctx):
    from .global_tensor import GlobalTensor
    _, internal = _alias()
    is_global = isinstance(t, GlobalTensor)
    if ctx is not None:
        if ctx.global_rank is None:
            if is_global:
                raise ValueError("Please set global_dst_rank in `flow.save` to save global tensor")
            local = t
        else:
            # local tensors inside a globally saved object (step counters, scalars) are taken from the
            # destination rank as they are
            local = _gather_global(t, ctx.global_rank) if is_global else t
        if ctx.external:
            if ctx.global_rank is None:
                rel = f"tensor_{uuid.uuid4().hex[:12]}"
            else:
                rel = f"global_tensor_{ctx.counter}"
                ctx.counter += 1
            if ctx.global_rank is None or ctx.global_rank == _rank():
                save_tensor_dir(local, ctx.path / rel)
            return {"path": rel}
        return {"data": _to_numpy(local), "dtype": internal.dtype.of(local.dtype), "device": "cpu"}
    if not is_global:
        return {"data": _to_numpy(t), "dtype": internal.dtype.of(t.dtype), "device": "cuda" if t.is_cuda else "cpu"}
    return {"data": t.numpy(), "dtype": internal.dtype.of(t.dtype), "placement": internal.placement.of(t.placement),
            "sbp": tuple(internal.sbp.sbp.of(s) for s in t.sbp)}


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def _standin(t, ctx=None):
    """An instance of the class named ``oneflow.Tensor`` / ``oneflow.nn.Parameter`` in the stream, carrying the
    reference's tensor state; pickled by the default protocol-2 reduce as NEWOBJ + BUILD."""
    oneflow, _ = _alias()
    is_param = isinstance(t, torch.nn.Parameter) or getattr(t, "_is_param", False)
    cls = oneflow.nn._ParameterStandin if is_param else oneflow.Tensor
    obj = object.__new__(cls)
    object.__setattr__(obj, "_pickle_state", tensor_state(t, ctx))
    return obj


def reduce_tensor(t, ctx=None):
    """``pickle.dumps(tensor)`` outside flow.save (e.g. multiprocessing): a self-contained rebuild."""
    return (_rebuild_from_state, (tensor_state(t, None), isinstance(t, torch.nn.Parameter)))


def _rebuild_from_state(state, is_param):
    p = _PendingParam() if is_param else _PendingTensor()
    p.state = state
    return _resolve(p, None, {})


class _Pickler(pickle._Pickler):
    """Pure-Python pickler so that ``save`` can swap tensors / dtypes / placements / sbp for the stand-in
    objects whose class paths the reference expects, before the normal reduce machinery sees them."""

    def __init__(self, f, ctx):
        super().__init__(f, protocol=2)
        self.ctx = ctx
        self._swapped = {}

    def save(self, obj, save_persistent_id=True):
        if isinstance(obj, torch.Tensor):
            key = id(obj)
            rep = self._swapped.get(key)
            if rep is None:
                rep = (_standin(obj, self.ctx), obj)  # keep obj alive: ids must stay unique while pickling
                self._swapped[key] = rep
            obj = rep[0]
        elif isinstance(obj, torch.dtype):
            _, internal = _alias()
            obj = internal.dtype(D.ENUM_OF[obj])
        elif isinstance(obj, Placement):
            _, internal = _alias()
            if not isinstance(obj, internal.placement):
                obj = internal.placement.of(obj)
        elif isinstance(obj, S.sbp):
            _, internal = _alias()
            obj = internal.sbp.sbp.of(obj)
        elif isinstance(obj, torch.Size):
            obj = tuple(obj)
        return super().save(obj, save_persistent_id)

    def save_global(self, obj, name=None):
        # numpy >= 2 names its internals ``numpy._core``; the reference pins numpy < 2, which only knows
        # ``numpy.core`` (an alias numpy 2 still resolves), so write the portable spelling.
        module = getattr(obj, "__module__", None)
        if module == "oneflow.nn" and getattr(obj, "__name__", "") == "Parameter":
            # the stand-in class of parameters: named by its class path, which resolves to the parameter class on load
            self.write(pickle.GLOBAL + b"oneflow.nn\nParameter\n")
            self.memoize(obj)
            return
        if isinstance(module, str) and module.startswith("numpy._core"):
            qual = name or getattr(obj, "__qualname__", obj.__name__)
            self.write(pickle.GLOBAL + module.replace("numpy._core", "numpy.core").encode() + b"\n" + qual.encode() + b"\n")
            self.memoize(obj)
            return
        return super().save_global(obj, name)

    dispatch = dict(pickle._Pickler.dispatch)
    import types as _types
    dispatch[_types.FunctionType] = save_global
    dispatch[_types.BuiltinFunctionType] = save_global
    dispatch[type] = lambda self, obj: (pickle._Pickler.save_type(self, obj) if obj in (type(None), type(NotImplemented), type(...))
                                        else self.save_global(obj))


class _PendingTensor:
    """What ``NEWOBJ oneflow.Tensor`` + ``BUILD state`` leaves behind; resolved once the whole object is loaded."""
    is_param = False
    state = None

    def __setstate__(self, state):
        self.state = state


class _PendingParam(_PendingTensor):
    is_param = True


def _resolve_tensor(p: _PendingTensor, ctx: _Ctx):
    from .global_tensor import to_global
    st = p.state
    if "path" in st:
        d = ctx.path / st["path"]
        if ctx.global_rank is None:
            t = load_tensor_dir(d)
        else:
            src = ctx.global_rank
            if _rank() == src:
                t = load_tensor_dir(d)
                meta = [(tuple(t.shape), t.dtype)]
            else:
                t, meta = None, [None]
            if dist.is_initialized():
                dist.broadcast_object_list(meta, src=src)
            if t is None:
                t = torch.empty((0,), dtype=meta[0][1])
            from .global_tensor import wrap
            t = wrap(t, meta[0][0], Placement("cpu", [src]), (S.broadcast,))
    else:
        dt = st["dtype"]
        dt = dt.torch_dtype if hasattr(dt, "torch_dtype") else dt
        t = torch.as_tensor(np.asarray(st["data"])).to(dt)
        if "placement" in st:
            pl = st["placement"]
            nd = tuple(x.to_sbp() if hasattr(x, "to_sbp") else x for x in st["sbp"])
            from .global_tensor import wrap
            coords = pl.coords(_rank())
            from . import boxing
            local = boxing.from_all_broadcast(t.to(pl.device()), pl, nd, coords) if coords is not None else torch.empty((0,), dtype=dt)
            t = wrap(local, t.shape, pl, nd)
        elif ctx is None or ctx.map_location is None:
            dev = st.get("device", "cpu")
            if dev == "cuda" and torch.cuda.is_available():
                t = t.cuda()
    if ctx is not None and ctx.map_location is not None:
        ml = ctx.map_location
        if isinstance(ml, Placement):
            from .global_tensor import GlobalTensor
            t = to_global(t, ml, (S.broadcast,) * ml.ndim) if not isinstance(t, GlobalTensor) or True else t
        else:
            from .global_tensor import GlobalTensor
            if isinstance(t, GlobalTensor):
                t = t._local
            t = t.to(ml)
    if p.is_param:
        t = torch.nn.Parameter(t, requires_grad=t.is_floating_point())
    return t


def _resolve(obj, ctx, memo):
    oid = id(obj)
    if oid in memo:
        return memo[oid]
    if isinstance(obj, _PendingTensor):
        r = _resolve_tensor(obj, ctx)
    elif isinstance(obj, OrderedDict):
        r = OrderedDict()
        memo[oid] = r
        for k, v in obj.items():
            r[k] = _resolve(v, ctx, memo)
        if hasattr(obj, "_metadata"):
            r._metadata = obj._metadata
        return r
    elif isinstance(obj, dict):
        r = {}
        memo[oid] = r
        for k, v in obj.items():
            r[k] = _resolve(v, ctx, memo)
        return r
    elif isinstance(obj, list):
        r = [_resolve(v, ctx, memo) for v in obj]
    elif isinstance(obj, tuple):
        r = tuple(_resolve(v, ctx, memo) for v in obj)
    elif hasattr(obj, "torch_dtype"):
        r = obj.torch_dtype
    elif hasattr(obj, "to_sbp"):
        r = obj.to_sbp()
    elif isinstance(obj, torch.nn.Module) or (hasattr(obj, "__dict__") and not isinstance(obj, (type, torch.Tensor))
                                              and type(obj).__module__.split(".")[0] not in ("builtins", "torch", "numpy")):
        # an object pickled whole (a module, an optimizer, a user class): its attributes are resolved in place
        memo[oid] = obj
        try:
            attrs = vars(obj)
        except TypeError:
            return obj
        for k, v in list(attrs.items()):
            nv = _resolve(v, ctx, memo)
            if nv is not v:
                attrs[k] = nv
        if isinstance(obj, torch.nn.Module):
            _complete_modules(obj)
        return obj
    else:
        r = obj
    memo[oid] = r
    return r


def _complete_modules(root):
    """A module pickled whole by another version of the library may lack bookkeeping attributes that
    ``Module.__call__`` reads (hook tables and the like): every submodule gets the defaults of a fresh module for
    what it does not carry."""
    defaults = torch.nn.Module().__dict__
    stack, seen = [root], set()
    while stack:
        m = stack.pop()
        if id(m) in seen:
            continue
        seen.add(id(m))
        for k, v in defaults.items():
            if k not in m.__dict__:
                m.__dict__[k] = type(v)() if isinstance(v, (dict, set, list)) else v
        stack.extend(c for c in m.__dict__.get("_modules", {}).values() if isinstance(c, torch.nn.Module))


class _Unpickler(pickle.Unpickler):
    def find_class(self, module, name):
        if module in ("oneflow", "oneflow.framework.tensor", "oneflow._oneflow_internal") and name == "Tensor":
            return _PendingTensor
        if name == "Parameter" and module.startswith("oneflow"):
            return _PendingParam
        if module.startswith("oneflow"):
            _alias()
        return super().find_class(module, name)


# ------------------------------------------------------------------------------------------------ public API
def save(obj, path, global_dst_rank=None, save_as_external_data=False):
    """Saves ``obj`` (tensors, state dicts, arbitrary picklable containers). With ``global_dst_rank`` global
    tensors are gathered to that rank, which alone writes the file(s).  ``path`` may also be a writable binary
    file object (``io.BytesIO``, an open file): the single-file form is written into it."""
    stream = path if hasattr(path, "write") else None
    if stream is not None:
        if save_as_external_data:
            raise ValueError("save_as_external_data needs a directory path, not a file object")
        path = Path(".")
    path = Path(path)
    from ..nn.graph.graph import Graph
    if isinstance(obj, Graph):
        obj = obj.state_dict()
        save_as_external_data = True
    ctx = _Ctx(path, global_dst_rank, save_as_external_data)
    buf = io.BytesIO()
    writer = global_dst_rank is None or global_dst_rank == _rank()
    if save_as_external_data and writer:
        path.mkdir(parents=True, exist_ok=True)
    _Pickler(buf, ctx).dump({"protocol_version": PROTOCOL_VERSION, "__oneflow__": None, "data": obj})
    if not writer:
        return
    if stream is not None:
        stream.write(buf.getvalue())
        return
    if save_as_external_data:
        (path / PICKLE_FILENAME).write_bytes(buf.getvalue())
    else:
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_bytes(buf.getvalue())


def _is_legacy_dir(path: Path):
    return path.is_dir() and not (path / PICKLE_FILENAME).exists()


def _load_legacy_dir(path: Path, ctx):
    if (path / META_FILENAME).is_file() and (path / DATA_FILENAME).is_file():
        return load_tensor_dir(path)          # the directory of one variable: the tensor itself
    if not (path / SNAPSHOT_DONE).exists() and not any((p / META_FILENAME).exists() for p in path.iterdir() if p.is_dir()):
        raise ValueError(f"{path} is not a valid checkpoint directory")
    out = {}
    for p in sorted(path.iterdir()):
        # missing pieces are tolerated (a variable directory without data is skipped)
        if p.is_dir() and (p / DATA_FILENAME).exists() and (p / META_FILENAME).exists():
            pend = _PendingTensor()
            pend.state = {"path": p.name}
            out[p.name] = _resolve_tensor(pend, ctx)
    return out


def _torch_load(src, map_location, support_pytorch_format, shown):
    """Last resort of ``load``: the file is not in this format; read it as a ``torch.save`` file when allowed."""
    cause = None
    if support_pytorch_format:
        try:
            return torch.load(src, map_location=map_location if isinstance(map_location, torch.device) else None,
                              weights_only=False)
        except Exception as e:
            cause = e
    raise ValueError(f"Cannot load file {shown}" + (f" ({type(cause).__name__}: {cause})" if cause else "")) from cause


def load(path, global_src_rank=None, map_location=None, *, support_pytorch_format=True):
    """Loads what ``save`` wrote (single file or directory), a legacy variable directory, or a ``torch.save``
    file. With ``global_src_rank`` only that rank reads; tensors come back as global broadcast tensors on
    ``cpu[src]``. ``map_location``: device / device string, or a placement (tensors become global).  ``path`` may
    also be a readable binary file object or the bytes themselves. A file in neither this nor (unless
    ``support_pytorch_format=False``) PyTorch's format raises ``ValueError("Cannot load file ...")``."""
    blob = path.read() if hasattr(path, "read") else (bytes(path) if isinstance(path, (bytes, bytearray)) else None)
    if isinstance(map_location, str):
        map_location = torch.device(map_location)
    if blob is not None:
        ctx = _Ctx(Path("."), global_src_rank, False, map_location)
        try:
            top = _Unpickler(io.BytesIO(blob)).load()
        except Exception:
            return _torch_load(io.BytesIO(blob), map_location, support_pytorch_format, "<stream>")
        if isinstance(top, dict) and "protocol_version" in top and "data" in top:
            top = top["data"]
        return _resolve(top, ctx, {})
    path = Path(path)
    rank = _rank()
    reader = global_src_rank is None or global_src_rank == rank
    ctx = _Ctx(path, global_src_rank, False, map_location)
    if _is_legacy_dir(path):
        return _load_legacy_dir(path, ctx)
    if path.is_dir():
        ctx.external = True
        file = path / PICKLE_FILENAME
    else:
        file = path
    raw = None
    if reader:
        raw = file.read_bytes()
    if global_src_rank is not None and dist.is_initialized():
        box = [raw]
        dist.broadcast_object_list(box, src=global_src_rank)
        raw = box[0]
    try:
        top = _Unpickler(io.BytesIO(raw)).load()
    except Exception:
        if path.is_dir():
            raise
        return _torch_load(str(path), map_location, support_pytorch_format, path)
    if not (isinstance(top, dict) and "protocol_version" in top and "data" in top):
        return _resolve(top, ctx, {})
    if top["protocol_version"] != PROTOCOL_VERSION:
        raise ValueError(f"unsupported checkpoint protocol {top['protocol_version']}")
    return _resolve(top["data"], ctx, {})
