"""The dual-object machinery: ``DualObject`` carries a PyTorch object and this framework's object through the same
program; ``autotest`` runs a test body several times on fresh random inputs and compares every pair."""
from __future__ import annotations

import collections.abc
import contextlib
import functools
import inspect
import operator
import os
import typing
import warnings

import numpy as np
import torch as torch_original

from . import generators as G
from .generators import Nothing, generator, rng

_GLOBAL_ONLY = ("to_global", "to_local", "to_consistent", "local_to_global", "global_to_global")


class PyTorchDoesNotSupportError(Exception):
    """PyTorch rejected the drawn arguments: the iteration does not count and is drawn again."""


class BothDoNotSupportError(Exception):
    """Both sides rejected the drawn arguments: the iteration does not count and is drawn again."""


class _Trace:
    def __init__(self):
        self.inputs, self.modules, self.results = [], [], []

    def clear(self):
        self.inputs.clear()
        self.modules.clear()
        self.results.clear()


_trace = _Trace()


def _flow():
    import oneflow_b200
    return oneflow_b200


# ------------------------------------------------------------------------------------------------ argument handling
def _annotations(fn):
    """(annotations of the positional parameters in order, annotations by name) of a callable; for a class, of its
    ``__init__``.  Callables without Python-level signatures (builtins) give nothing."""
    try:
        spec = inspect.getfullargspec(fn)
    except TypeError:
        return [], {}
    names = list(spec.args)
    if names and names[0] in ("self", "cls"):
        names = names[1:]
    ann = dict(spec.annotations)
    target = fn.__init__ if inspect.isclass(fn) else fn
    try:
        ann.update({k: v for k, v in typing.get_type_hints(target).items() if k in ann or k in names})
    except Exception:                                                    # noqa: BLE001  unresolved forward references
        pass
    return [ann.get(n) for n in names], ann


def _draw(x, ann=None):
    """Replace generators by their values (the same on both sides), inside containers too."""
    if isinstance(x, generator):
        if ann is not None:
            x.to(ann)
        return _draw(x.value())
    if isinstance(x, (list, tuple)) and not isinstance(x, torch_original.Size):
        return type(x)(_draw(v) for v in x)
    if isinstance(x, dict):
        return {k: _draw(v) for k, v in x.items()}
    return x


def _side(x, which):
    if isinstance(x, DualObject):
        return x.pytorch if which == 0 else x.oneflow
    if isinstance(x, (list, tuple)) and not isinstance(x, torch_original.Size):
        return type(x)(_side(v, which) for v in x)
    if isinstance(x, dict):
        return {k: _side(v, which) for k, v in x.items()}
    if isinstance(x, slice):
        return slice(_side(x.start, which), _side(x.stop, which), _side(x.step, which))
    return x


def _prepare(fn, args, kwargs):
    pos, kw = _annotations(fn)
    a = [_draw(v, pos[i] if i < len(pos) else None) for i, v in enumerate(args)]
    k = {name: _draw(v, kw.get(name)) for name, v in kwargs.items()}
    a = [v for v in a if not isinstance(v, Nothing)]
    k = {n: v for n, v in k.items() if not isinstance(v, Nothing)}
    return a, k


def _gather(t):
    """A flow tensor as a plain local tensor holding the logical value."""
    flow = _flow()
    if getattr(t, "is_global", False):
        t = t.to_global(sbp=[flow.sbp.broadcast] * len(t.sbp)).to_local()
    return t


# ------------------------------------------------------------------------------------------------ the dual object
class DualObject:
    def __init__(self, name, pytorch, oneflow):
        self.__dict__["name"] = name
        self.__dict__["pytorch"] = pytorch
        self.__dict__["oneflow"] = oneflow
        if isinstance(pytorch, torch_original.nn.Module) and isinstance(oneflow, torch_original.nn.Module) and pytorch is not oneflow:
            if not any(m.pytorch is pytorch for m in _trace.modules):
                self._sync_module()
                _trace.modules.append(self)

    def _sync_module(self):
        """Both modules start from the PyTorch one's parameters and buffers."""
        with torch_original.no_grad():
            state = {k: v.detach().clone() for k, v in self.pytorch.state_dict().items()}
            own = self.oneflow.state_dict()
            missing = [k for k in state if k not in own]
            if missing:
                warnings.warn(f"the oneflow module has no {missing}")
            self.oneflow.load_state_dict({k: v for k, v in state.items() if k in own}, strict=False)

    def __repr__(self):
        return f"DualObject({self.name}: pytorch={self.pytorch!r}, oneflow={self.oneflow!r})"

    # attribute access walks both objects
    def __getattr__(self, key):
        if key.startswith("__") and key.endswith("__"):
            raise AttributeError(key)
        p, o = self.pytorch, self.oneflow
        if key in _GLOBAL_ONLY and isinstance(p, (torch_original.Tensor, torch_original.nn.Module)):
            p_attr = lambda *a, **k: p                                   # noqa: E731  PyTorch has no global tensors
        else:
            try:
                p_attr = getattr(p, key)
            except AttributeError as e:
                raise PyTorchDoesNotSupportError(str(e)) from None
        o_attr = getattr(o, key)
        return _wrap(f"{self.name}.{key}", p_attr, o_attr)

    def __setattr__(self, key, value):
        setattr(self.pytorch, key, _side(value, 0))
        setattr(self.oneflow, key, _side(value, 1))

    def __call__(self, *args, **kwargs):
        args, kwargs = _prepare(self.pytorch, args, kwargs)
        out = _both(self.name, lambda: self.pytorch(*_side(args, 0), **_side(kwargs, 0)),
                    lambda: self.oneflow(*_side(args, 1), **_side(kwargs, 1)))
        if _profile["op"] is not None and self.pytorch is _profile["op"]:
            _profile["rows"].append(_time_both(self, args, kwargs))
        return out

    # containers
    def __iter__(self):
        return iter([_wrap(f"{self.name}[{i}]", p, o) for i, (p, o) in enumerate(zip(self.pytorch, self.oneflow))])

    def __len__(self):
        return len(self.pytorch)

    def __getitem__(self, idx):
        idx = _draw(idx)
        return _both(f"{self.name}[...]", lambda: self.pytorch[_side(idx, 0)], lambda: self.oneflow[_side(idx, 1)])

    def __setitem__(self, idx, value):
        idx, value = _draw(idx), _draw(value)
        self.pytorch[_side(idx, 0)] = _side(value, 0)
        self.oneflow[_side(idx, 1)] = _side(value, 1)

    def __enter__(self):
        return _wrap(self.name, self.pytorch.__enter__(), self.oneflow.__enter__())

    def __exit__(self, *exc):
        a = self.pytorch.__exit__(*exc)
        b = self.oneflow.__exit__(*exc)
        return bool(a and b)

    def __bool__(self):
        return bool(self.pytorch)

    def __array__(self, dtype=None, copy=None):
        """numpy sees the PyTorch side (``np.allclose(flow_result.numpy(), dual.numpy())`` in hand-written checks)."""
        p = self.pytorch
        a = p.detach().cpu().numpy() if isinstance(p, torch_original.Tensor) else np.asarray(p)
        return a.astype(dtype) if dtype is not None else a

    def __index__(self):
        return operator.index(self.pytorch)

    def __int__(self):
        return int(self.pytorch)

    def __float__(self):
        return float(self.pytorch)

    def __hash__(self):
        return id(self)


def _both(name, p_thunk, o_thunk):
    """Run one step on both sides.  PyTorch refusing it invalidates the drawn arguments (the iteration is repeated);
    only this framework refusing it is a failure."""
    p_err = o_err = None
    try:
        p_res = p_thunk()
    except Exception as e:                                               # noqa: BLE001
        p_err = e
    try:
        o_res = o_thunk()
    except Exception as e:                                               # noqa: BLE001
        o_err = e
    if p_err is not None and o_err is not None:
        raise BothDoNotSupportError(f"{name}: pytorch: {p_err!r}; oneflow: {o_err!r}")
    if p_err is not None:
        raise PyTorchDoesNotSupportError(f"{name}: {p_err!r}")
    if o_err is not None:
        raise o_err
    return _wrap(f"{name}()", p_res, o_res, record=True)


def _binop(fn, reflected=False):
    def method(self, other):
        other = _draw(other)
        if reflected:
            return _both(fn.__name__, lambda: fn(_side(other, 0), self.pytorch), lambda: fn(_side(other, 1), self.oneflow))
        return _both(fn.__name__, lambda: fn(self.pytorch, _side(other, 0)), lambda: fn(self.oneflow, _side(other, 1)))
    return method


def _unop(fn):
    def method(self):
        return _both(fn.__name__, lambda: fn(self.pytorch), lambda: fn(self.oneflow))
    return method


for _name, _fn in (("add", operator.add), ("sub", operator.sub), ("mul", operator.mul), ("truediv", operator.truediv),
                   ("floordiv", operator.floordiv), ("mod", operator.mod), ("pow", operator.pow), ("matmul", operator.matmul),
                   ("and", operator.and_), ("or", operator.or_), ("xor", operator.xor), ("lshift", operator.lshift),
                   ("rshift", operator.rshift)):
    setattr(DualObject, f"__{_name}__", _binop(_fn))
    setattr(DualObject, f"__r{_name}__", _binop(_fn, reflected=True))
for _name, _fn in (("lt", operator.lt), ("le", operator.le), ("gt", operator.gt), ("ge", operator.ge), ("eq", operator.eq),
                   ("ne", operator.ne), ("iadd", operator.iadd), ("isub", operator.isub), ("imul", operator.imul),
                   ("itruediv", operator.itruediv)):
    setattr(DualObject, f"__{_name}__", _binop(_fn))
for _name, _fn in (("neg", operator.neg), ("pos", operator.pos), ("abs", operator.abs), ("invert", operator.invert)):
    setattr(DualObject, f"__{_name}__", _unop(_fn))


_PLAIN = (bool, int, float, complex, str, bytes, type(None), torch_original.dtype, torch_original.device)


def _wrap(name, p, o, record=False):
    if isinstance(p, DualObject):
        return p
    d = DualObject(name, p, o)
    if record and isinstance(p, torch_original.Tensor):
        _trace.results.append(d)
    return d


def GetDualObject(name, pytorch, oneflow):
    return DualObject(name, pytorch, oneflow)


# ------------------------------------------------------------------------------------------------ comparison
def _np(t):
    t = t.detach()
    if t.dtype == torch_original.bfloat16:
        t = t.float()
    return t.cpu().numpy()


def check_tensor_equality(p, o, rtol=1e-4, atol=1e-5, check_dtype=False):
    o = _gather(o)
    if tuple(p.shape) != tuple(o.shape):
        return False, f"shape {tuple(p.shape)} vs {tuple(o.shape)}"
    if check_dtype and p.dtype != o.dtype:
        return False, f"dtype {p.dtype} vs {o.dtype}"
    a, b = _np(p), _np(o)
    if a.dtype == np.bool_ or b.dtype == np.bool_:
        ok = np.array_equal(a.astype(np.bool_), b.astype(np.bool_))
    else:
        ok = np.allclose(a, b, rtol=rtol, atol=atol, equal_nan=True)
    if ok:
        return True, ""
    with np.errstate(all="ignore"):
        diff = np.abs(a.astype(np.float64) - b.astype(np.float64)) if a.dtype.kind != "c" else np.abs(a - b)
    return False, f"max abs difference {np.nanmax(diff) if diff.size else 0} over shape {a.shape}"


def check_equality(d, rtol=1e-4, atol=1e-5, check_dtype=False):
    """(ok, message) for one dual pair, whatever it holds."""
    p, o = (d.pytorch, d.oneflow) if isinstance(d, DualObject) else d
    if isinstance(p, torch_original.Tensor):
        if not isinstance(o, torch_original.Tensor):
            return False, f"tensor vs {type(o).__name__}"
        return check_tensor_equality(p, o, rtol, atol, check_dtype)
    if p is None or o is None:
        return (p is None and o is None), f"{p!r} vs {o!r}"
    if isinstance(p, (torch_original.nn.Module, torch_original.optim.Optimizer)) or callable(p):
        return True, ""
    if isinstance(p, (str, bytes, torch_original.dtype, torch_original.device)):
        return (p == o or str(p) == str(o)), f"{p!r} vs {o!r}"
    if isinstance(p, (bool, int, float, complex, np.generic)):
        ok = bool(np.allclose(p, o, rtol=rtol, atol=atol, equal_nan=True))
        return ok, f"{p!r} vs {o!r}"
    if isinstance(p, np.ndarray):
        return bool(np.allclose(p, np.asarray(o), rtol=rtol, atol=atol, equal_nan=True)), "arrays differ"
    if isinstance(p, collections.abc.Mapping):
        for k in p:
            ok, msg = check_equality((p[k], o[k]), rtol, atol, check_dtype)
            if not ok:
                return False, f"[{k!r}]: {msg}"
        return True, ""
    if isinstance(p, collections.abc.Sequence):
        if len(p) != len(o):
            return False, f"length {len(p)} vs {len(o)}"
        for i, (a, b) in enumerate(zip(p, o)):
            ok, msg = check_equality((a, b), rtol, atol, check_dtype)
            if not ok:
                return False, f"[{i}]: {msg}"
        return True, ""
    return True, ""


# ------------------------------------------------------------------------------------------------ timing both sides
_profile = {"op": None, "rows": []}


def _time_both(d, args, kwargs, warmup=3, runs=20):
    import time

    def one(fn, a, k):
        for _ in range(warmup):
            fn(*a, **k)
        if torch_original.cuda.is_available():
            torch_original.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(runs):
            fn(*a, **k)
        if torch_original.cuda.is_available():
            torch_original.cuda.synchronize()
        return (time.perf_counter() - t0) / runs * 1e3

    with torch_original.no_grad():
        tp = one(d.pytorch, _side(args, 0), _side(kwargs, 0))
        to = one(d.oneflow, _side(args, 1), _side(kwargs, 1))
    shapes = [tuple(a.pytorch.shape) for a in args if isinstance(a, DualObject) and isinstance(a.pytorch, torch_original.Tensor)]
    return {"op": d.name, "args": shapes, "pytorch_ms": tp, "oneflow_ms": to}


def profile(op):
    """Decorator for ``profile_*`` methods: every call of ``op`` (a dual callable such as ``torch.nn.functional.relu``)
    inside the body is also timed on both sides; the method returns the rows (op, argument shapes, ms per call)."""
    def deco(f):
        @functools.wraps(f)
        def run(*a, **k):
            _profile["op"], _profile["rows"] = (op.pytorch if isinstance(op, DualObject) else op), []
            try:
                f(*a, **k)
                return list(_profile["rows"])
            finally:
                _profile["op"] = None
        return run
    return deco


# ------------------------------------------------------------------------------------------------ decorators
def _backward(d, random_grad):
    p, o = d.pytorch, d.oneflow
    flow = _flow()
    if random_grad:
        g = rng.uniform(0, 1, size=tuple(p.shape))
        if G.is_global():
            g = G._broadcast_obj(g)
        gp = torch_original.tensor(g, dtype=p.dtype, device=p.device)
        if getattr(o, "is_global", False):
            go = flow.tensor(g, dtype=o.dtype).to_global(o.placement, [flow.sbp.broadcast] * len(o.sbp))
        else:
            go = torch_original.tensor(g.reshape(tuple(o.shape)), dtype=o.dtype, device=o.device)
        p.backward(gp, retain_graph=True)
        o.backward(go, retain_graph=True)
    else:
        p.sum().backward(retain_graph=True)
        o.sum().backward(retain_graph=True)


def autotest(n=20, auto_backward: typing.Union[bool, str] = True, rtol=1e-4, atol=1e-5, check_graph=True, check_allclose=True,
             check_dtype=False, check_grad_use_random_data=True, include_complex=False):
    """Runs the test body ``n`` times.  The body builds its program on the dual ``torch`` namespace and returns the
    dual result(s); those, every intermediate tensor, the gradients of all random input tensors and the parameters and
    parameter gradients of all modules must agree between the two sides.  Iterations whose drawn arguments PyTorch
    rejects are drawn again."""
    verbose = os.getenv("ONEFLOW_TEST_VERBOSE") is not None

    def deco(f):
        @functools.wraps(f)
        def run(test_case, *args, **kwargs):
            todo, tries = n, 0
            while todo > 0:
                tries += 1
                if tries > n * 20:
                    raise ValueError("autotest: PyTorch rejected the drawn arguments too often — the test body is invalid")
                _trace.clear()
                try:
                    res = f(test_case, *args, **kwargs)
                except (PyTorchDoesNotSupportError, BothDoNotSupportError) as e:
                    if verbose:
                        print(f"{f.__name__}: drawn again: {e}")
                    continue
                pairs = []
                if res is not None:
                    items = list(res) if isinstance(res, (list, tuple)) or (
                        isinstance(res, DualObject) and isinstance(res.pytorch, (list, tuple))) else [res]
                    for x in items:
                        if x is None:
                            continue
                        if not isinstance(x, DualObject):
                            continue
                        p = x.pytorch
                        if auto_backward and isinstance(p, torch_original.Tensor) and p.requires_grad and x.oneflow.requires_grad \
                                and (p.is_floating_point() or p.is_complex()):
                            _backward(x, check_grad_use_random_data)
                        elif auto_backward is True and isinstance(p, torch_original.Tensor) and p.requires_grad != x.oneflow.requires_grad:
                            test_case.fail(f"{f.__name__}: requires_grad differs: pytorch {p.requires_grad}, oneflow {x.oneflow.requires_grad}")
                        pairs.append(("result", x))
                pairs += [("intermediate", d) for d in _trace.results]
                for d in _trace.inputs:
                    pairs.append(("input gradient", (d.pytorch.grad, d.oneflow.grad)))
                for m in _trace.modules:
                    own = dict(m.oneflow.named_parameters())
                    for key, pp in m.pytorch.named_parameters():
                        if key in own:
                            pairs.append((f"parameter {key}", (pp, own[key])))
                            pairs.append((f"gradient of {key}", (pp.grad, own[key].grad)))
                if check_allclose:
                    for what, d in pairs:
                        ok, msg = check_equality(d, rtol=rtol, atol=atol, check_dtype=check_dtype)
                        test_case.assertTrue(ok, f"{f.__name__}: {what} differs: {msg}")
                todo -= 1
            _trace.clear()
        return run
    return deco


@contextlib.contextmanager
def GlobalScope():
    old = G._state["global"]
    G._state["global"] = True
    try:
        yield
    finally:
        G._state["global"] = old


def globaltest(f):
    """Marks a test as working on global tensors: random inputs are created broadcast over all ranks."""
    @functools.wraps(f)
    def run(*args, **kwargs):
        with GlobalScope():
            return f(*args, **kwargs)
    return run


# ------------------------------------------------------------------------------------------------ dual data
def _dual_tensor(p, requires_grad, pin_memory=False):
    flow = _flow()
    p = p.requires_grad_(bool(requires_grad) and (p.is_floating_point() or p.is_complex()))
    o = p.detach().clone()
    if G.is_global():
        o = o.to_global(flow.placement.all("cpu"), flow.sbp.broadcast)
    elif pin_memory and torch_original.cuda.is_available():
        o = o.pin_memory()
    o.requires_grad_(p.requires_grad)
    d = DualObject("tensor", p, o)
    _trace.inputs.append(d)
    return d


def random_tensor(ndim=None, dim0=1, dim1=None, dim2=None, dim3=None, dim4=None, low=None, high=None, dtype=float,
                  requires_grad=True, pin_memory=False):
    """A random tensor present on both sides with equal values; ``dim*`` / ``ndim`` / ``low`` / ``high`` take numbers or
    generators; unspecified extents are drawn from [1, 8).  A generator object keeps the value it drew, so tensors built
    from the same generator objects get the same extents."""
    if isinstance(requires_grad, generator):
        requires_grad = requires_grad.value()
    t = G.random_pytorch_tensor(ndim, dim0, dim1, dim2, dim3, dim4, low, high, dtype, pin_memory).value()
    return _dual_tensor(t, requires_grad and dtype is not int, pin_memory)


def choice_tensor(a, size=None, replace=True, p=None, dtype=int, requires_grad=False):
    if isinstance(requires_grad, generator):
        requires_grad = requires_grad.value()
    t = G.choice_pytorch_tensor(a, size, replace, p, dtype).value()
    return _dual_tensor(t, requires_grad and dtype is not int)


def random_dtype(seq_names):
    dt = G.random_pytorch_dtype(seq_names).value()
    return DualObject("dtype", dt, dt)


torch = DualObject("torch", torch_original, _flow())

__all__ = ["autotest", "globaltest", "profile", "random_tensor", "random_dtype", "choice_tensor", "DualObject", "GetDualObject",
           "check_equality", "check_tensor_equality", "PyTorchDoesNotSupportError", "BothDoNotSupportError"]
