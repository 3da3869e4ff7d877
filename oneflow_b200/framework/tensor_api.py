"""Tensor construction and the methods the flow API adds to tensors.

Local tensors ARE ``torch.Tensor`` objects (``flow.Tensor`` answers ``isinstance`` for them and builds them);
global tensors are ``GlobalTensor`` wrappers. ``to_global`` / ``to_local`` / ``is_global`` / ``placement`` /
``sbp`` are attached to ``torch.Tensor`` so that both kinds share one surface
(reference: python/oneflow/framework/tensor.py, nn/modules/global_cast.py:40-95)."""
from __future__ import annotations

import numpy as np
import torch

from .. import sbp as S
from . import global_tensor as GT
from .placement import placement as Placement


class _MockDevice:
    """The reference's pseudo device for tests (``DeviceType::kMockDevice``, oneflow/core/common/device_type.proto):
    it names a device kind without memory of its own; host memory stands behind it."""
    type = "mock"

    def __init__(self, index=0):
        self.index = index

    def __eq__(self, other):
        return isinstance(other, _MockDevice) and other.index == self.index

    def __hash__(self):
        return hash(("mock", self.index))

    def __repr__(self):
        return f"device(type='mock', index={self.index})"


class _DeviceMeta(type):
    def __instancecheck__(cls, obj):
        return isinstance(obj, (torch.device, _MockDevice))

    def __call__(cls, *args, **kwargs):
        """``flow.device("cuda")`` names the current CUDA device (``cuda:0`` unless changed), so it compares equal to the
        ``.device`` of tensors placed there; everything else is ``torch.device``."""
        if args and isinstance(args[0], str) and args[0].partition(":")[0] == "mock":
            return _MockDevice(int(args[0].partition(":")[2] or (args[1] if len(args) > 1 else 0)))
        d = torch.device(*args, **kwargs)
        if d.type == "cuda" and d.index is None:
            return torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
        return d


class device(metaclass=_DeviceMeta):
    """``flow.device``: constructor and ``isinstance`` target for device objects (which are ``torch.device``)."""


class _TensorMeta(type):
    def __instancecheck__(cls, obj):
        return isinstance(obj, torch.Tensor)

    def __call__(cls, *args, **kwargs):
        """``flow.Tensor(2, 3)`` allocates; ``flow.Tensor(data)`` copies ``data`` (array, list, tensor) into a new
        float32 tensor — never aliasing the caller's numpy memory — on ``device`` when given."""
        if len(args) == 1 and not isinstance(args[0], (int, torch.Size)):
            data = args[0]
            dev = kwargs.get("device")
            if isinstance(data, torch.Tensor):
                return data.detach().clone().to(device=dev if dev is not None else data.device)
            return torch.tensor(np.asarray(data), dtype=kwargs.get("dtype", torch.get_default_dtype()), device=dev)
        dev = kwargs.pop("device", None)
        t = torch.Tensor(*args, **kwargs)
        return t.to(dev) if dev is not None else t

    def __getattr__(cls, name):
        """``flow.Tensor.add`` and the like: the unbound tensor methods."""
        if name.startswith("__"):
            raise AttributeError(name)
        return getattr(torch.Tensor, name)

    def __subclasscheck__(cls, sub):
        return issubclass(sub, torch.Tensor) or type.__subclasscheck__(cls, sub)


class Tensor(metaclass=_TensorMeta):
    """``flow.Tensor``: ``isinstance(x, flow.Tensor)`` holds for every local and global tensor and
    ``flow.Tensor(2, 3)`` builds a local tensor. Instances of this class itself only exist inside
    checkpoints being written, where they carry the tensor state under the class path ``oneflow.Tensor``."""
    _pickle_state = None

    def __getstate__(self):
        return self._pickle_state


Tensor.__module__ = "oneflow"


def _globalize(t, placement, sbp, requires_grad=False):
    if placement is None:
        return t.requires_grad_(requires_grad) if requires_grad else t
    nd = S.normalize(sbp if sbp is not None else S.broadcast, placement.ndim)
    allb = (S.broadcast,) * placement.ndim
    g = GT.to_global(t, placement, allb)
    g = GT.to_global(g, placement, nd)
    if requires_grad:
        g.requires_grad_(True)
    return g


def tensor(data, dtype=None, device=None, placement=None, sbp=None, requires_grad=False, pin_memory=False):
    if isinstance(data, GT.GlobalTensor):
        out = data.detach().clone()
        if dtype is not None:
            out = out.to(dtype)
        return out.requires_grad_(requires_grad) if requires_grad else out
    if isinstance(data, torch.Tensor):
        t = data.detach().clone()
        if dtype is not None:
            t = t.to(dtype)
    else:
        if isinstance(data, (list, tuple)) and data and all(isinstance(d, torch.Tensor) for d in data):
            t = torch.stack([d.detach() for d in data])       # a sequence of tensors stacks along a new first axis
            t = t.to(dtype) if dtype is not None else t
        else:
            t = torch.tensor(data, dtype=dtype)
    if placement is not None:
        return _globalize(t, placement, sbp, requires_grad)
    if device is not None:
        t = t.to(device)
    if pin_memory:
        t = t.pin_memory()
    return t.requires_grad_(requires_grad) if requires_grad else t


def _resolve_gen(generator, device):
    from .generator import resolve
    return resolve(generator, device)


def _factory(torch_fn):
    def fn(*args, placement=None, sbp=None, device=None, requires_grad=False, **kwargs):
        if placement is None:
            if device is not None:
                kwargs["device"] = device
            if kwargs.get("generator") is not None:
                kwargs["generator"] = _resolve_gen(kwargs["generator"], device or "cpu")
            t = torch_fn(*args, **kwargs)
            return t.requires_grad_(requires_grad) if requires_grad else t
        # global: every rank draws the logical tensor (first rank's values win along broadcast axes)
        kwargs["device"] = placement.device() if placement.contains(GT._rank()) else "cpu"
        if kwargs.get("generator") is not None:
            kwargs["generator"] = _resolve_gen(kwargs["generator"], kwargs["device"])
        t = torch_fn(*args, **kwargs)
        return _globalize(t, placement, sbp, requires_grad)
    fn.__name__ = torch_fn.__name__
    fn.__doc__ = f"flow.{torch_fn.__name__}: torch.{torch_fn.__name__} plus ``placement=`` / ``sbp=`` for global tensors."
    return fn


zeros, ones, empty, full = (_factory(f) for f in (torch.zeros, torch.ones, torch.empty, torch.full))
randn, rand, randint, randperm = (_factory(f) for f in (torch.randn, torch.rand, torch.randint, torch.randperm))
arange, eye, linspace = (_factory(f) for f in (torch.arange, torch.eye, torch.linspace))


logspace, hann_window, normal = (_factory(f) for f in (torch.logspace, torch.hann_window, torch.normal))


def _like_factory(torch_fn):
    def fn(input, *args, placement=None, sbp=None, device=None, requires_grad=False, **kwargs):
        if placement is None:
            if device is not None:
                kwargs["device"] = device
            if kwargs.get("generator") is not None:
                kwargs["generator"] = _resolve_gen(kwargs["generator"], device or input.device)
            t = torch_fn(input, *args, **kwargs)       # a global input gives a global result through the dispatch
            return t.requires_grad_(requires_grad) if requires_grad else t
        dev = placement.device() if placement.contains(GT._rank()) else "cpu"
        proto = torch.empty(tuple(input.shape), dtype=kwargs.pop("dtype", None) or input.dtype, device=dev)
        return _globalize(torch_fn(proto, *args, **kwargs), placement, sbp, requires_grad)
    fn.__name__ = torch_fn.__name__
    fn.__doc__ = f"flow.{torch_fn.__name__}: torch.{torch_fn.__name__} plus ``placement=`` / ``sbp=`` for global results."
    return fn


zeros_like, ones_like, full_like, empty_like = (_like_factory(f) for f in (torch.zeros_like, torch.ones_like, torch.full_like,
                                                                          torch.empty_like))
rand_like, randn_like, randint_like = (_like_factory(f) for f in (torch.rand_like, torch.randn_like, torch.randint_like))
for _f in (zeros_like, ones_like, full_like, empty_like, rand_like, randn_like, randint_like):
    _f.__name__ = _f.__name__ + "_op"        # the names the reference's functions carry


def from_numpy(a):
    return torch.from_numpy(a)


def install_tensor_methods():
    T = torch.Tensor
    if getattr(T, "_ofb_patched", False):
        return
    T.to_global = lambda self, placement=None, sbp=None, **kw: GT.to_global(self, placement, sbp, **kw)
    T.to_local = lambda self, copy=False: GT.to_local(self, copy=copy)
    T.is_global = property(lambda self: isinstance(self, GT.GlobalTensor))
    T.is_local = property(lambda self: not isinstance(self, GT.GlobalTensor))

    def _placement(self):
        raise RuntimeError("local tensor has no placement; call to_global first")

    def _sbp(self):
        raise RuntimeError("local tensor has no sbp; call to_global first")
    T.placement = property(_placement)
    T.sbp = property(_sbp)
    T.global_id = lambda self: id(self)
    _install_reference_methods(T)
    T._ofb_patched = True


def _install_reference_methods(T):
    """Tensor methods of the reference that torch.Tensor lacks (reference: python/oneflow/framework/tensor.py
    RegisterMethods, python/oneflow/framework/docstr/tensor.py)."""
    import warnings

    import torch.nn.functional as F

    def _top(name):
        def method(self, *a, **k):
            import oneflow_b200 as flow
            return getattr(flow, name)(self, *a, **k)
        method.__name__ = name
        return method

    T.cast = lambda self, dtype: self.to(dtype)

    class _CallableTensor(torch.Tensor):
        """What ``x.real`` / ``x.imag`` give: the tensor itself, which may also be called (``x.real()``) since
        the reference spells these as methods. Results of operations on it are plain tensors."""
        __torch_function__ = torch._C._disabled_torch_function_impl

        def __call__(self):
            return self.as_subclass(torch.Tensor)

    for _name in ("real", "imag"):
        _desc = getattr(T, _name)

        def _get(self, _desc=_desc):
            out = _desc.__get__(self)
            return out.as_subclass(_CallableTensor) if type(out) is torch.Tensor else out
        setattr(T, _name, property(_get, _desc.__set__, doc=_desc.__doc__))

    class _SliceError(RuntimeError, IndexError, ValueError, TypeError):
        """A bad slice (zero or negative step, float bounds) is a ``RuntimeError`` or ``IndexError`` in the reference
        and a ``ValueError`` / ``TypeError`` in Python: every one of them catches it."""

    _getitem = T.__getitem__

    def __getitem__(self, index):
        try:
            return _getitem(self, index)
        except (ValueError, TypeError) as e:
            raise _SliceError(str(e)) from None
        except IndexError as e:
            if "out of bounds" in str(e):
                raise IndexError(f"{e} (index out of range)") from None
            raise
    T.__getitem__ = __getitem__

    _backward = T.backward

    def backward(self, gradient=None, retain_graph=None, create_graph=False, inputs=None):
        """``backward`` that also starts from a complex scalar (the seed gradient is one, as for real scalars)."""
        if gradient is None and self.is_complex() and self.numel() == 1:
            gradient = torch.ones_like(self)
        return _backward(self, gradient, retain_graph, create_graph, inputs)
    backward.__doc__ = _backward.__doc__
    T.backward = backward
    def _register_post_grad_accumulation_hook(self, hook):
        """``hook(grad)`` runs after a gradient was accumulated into ``.grad``; a returned tensor replaces it, None
        keeps what the hook changed in place (reference: Tensor._register_post_grad_accumulation_hook)."""
        def run(param):
            res = hook(param.grad)
            if res is not None:
                param.grad = res
        return self.register_post_accumulate_grad_hook(run)
    T._register_post_grad_accumulation_hook = _register_post_grad_accumulation_hook

    def _no_buffer(self):
        raise RuntimeError("_tensor_buffer_shapes_and_dtypes is only available for tensors of dtype tensor_buffer")
    T._tensor_buffer_shapes_and_dtypes = property(_no_buffer)

    def global_id(self):
        if not isinstance(self, GT.GlobalTensor):
            raise RuntimeError("global_id is only available for global tensors")
        return id(self)
    T.global_id = global_id

    def _where(self, x=None, y=None):
        from .compat_ops import where
        return where(self, x, y)
    T.where = _where
    _type_as = T.type_as

    def type_as(self, other):
        """``type_as`` that follows a global target onto its placement and sbp."""
        if isinstance(other, GT.GlobalTensor) and not isinstance(self, GT.GlobalTensor):
            return _globalize(self.to(other.dtype), other.placement, other.sbp, False)
        return _type_as(self, other)
    T.type_as = type_as
    T.gelu = lambda self, approximate="none": F.gelu(self, approximate=approximate)
    T.mish = lambda self: F.mish(self)
    T.selu = lambda self: F.selu(self)
    T.silu = lambda self: F.silu(self)
    T.softplus = lambda self, beta=1, threshold=20: F.softplus(self, beta, threshold)
    T.softsign = _top("softsign")
    T.in_top_k = lambda self, predictions, k: _top("in_top_k")(self, predictions, k)
    T.nms = lambda self, scores, iou_threshold: _top("nms")(self, scores, iou_threshold)
    T.is_lazy = property(lambda self: False)
    T.is_consistent = property(lambda self: isinstance(self, GT.GlobalTensor))
    T.to_consistent = lambda self, *a, **k: self.to_global(*a, **k)

    def local_to_global(self, placement=None, sbp=None, *, check_meta=True, copy=False):
        if isinstance(self, GT.GlobalTensor):
            raise RuntimeError("local_to_global: the tensor is already global")
        if placement is None or sbp is None:
            raise ValueError("local_to_global needs both placement and sbp")
        return GT.to_global(self, placement, sbp, check_meta=check_meta, copy=copy)

    def global_to_global(self, placement=None, sbp=None, *, grad_sbp=None, check_meta=False, copy=False):
        if not isinstance(self, GT.GlobalTensor):
            raise RuntimeError("global_to_global: the tensor is local")
        if placement is None and sbp is None:
            raise ValueError("global_to_global needs placement or sbp")
        return GT.to_global(self, placement, sbp, grad_sbp=grad_sbp, check_meta=check_meta, copy=copy)
    T.local_to_global, T.global_to_global = local_to_global, global_to_global

    # offload / load: the storage moves between device and pinned host memory, the tensor object stays the same
    def offload(self):
        t = self._local if isinstance(self, GT.GlobalTensor) else self
        if not t.is_cuda:
            warnings.warn("offload: the tensor is already in host memory")
            return
        dev = t.device
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        host.copy_(t.data)
        t.data = host
        t._ofb_offloaded_from = dev

    def load(self):
        t = self._local if isinstance(self, GT.GlobalTensor) else self
        dev = getattr(t, "_ofb_offloaded_from", None)
        if dev is None:
            warnings.warn("load: the tensor is not offloaded")
            return
        t.data = t.data.to(dev, non_blocking=True)
        t._ofb_offloaded_from = None

    def is_offloaded(self):
        t = self._local if isinstance(self, GT.GlobalTensor) else self
        return getattr(t, "_ofb_offloaded_from", None) is not None
    T.offload, T.load, T.is_offloaded = offload, load, is_offloaded

    def _init_method(fn):
        def method(self, *a, **k):
            with torch.no_grad():
                fn(self, *a, **k)
            return self
        return method
    I = torch.nn.init
    T.kaiming_normal_ = _init_method(lambda self, a=0, mode="fan_in", nonlinearity="leaky_relu": I.kaiming_normal_(self, a, mode, nonlinearity))
    T.kaiming_uniform_ = _init_method(lambda self, a=0, mode="fan_in", nonlinearity="leaky_relu": I.kaiming_uniform_(self, a, mode, nonlinearity))
    T.xavier_normal_ = _init_method(lambda self, gain=1.0: I.xavier_normal_(self, gain))
    T.xavier_uniform_ = _init_method(lambda self, gain=1.0: I.xavier_uniform_(self, gain))
    T.orthogonal_ = _init_method(lambda self, gain=1.0: I.orthogonal_(self, gain))
    T.trunc_normal_ = _init_method(lambda self, mean=0.0, std=1.0, a=-2.0, b=2.0: I.trunc_normal_(self, mean, std, a, b))
    def _new_method(name, factory):
        orig = getattr(T, name)

        def method(self, *args, placement=None, sbp=None, **kw):
            if placement is None and sbp is None and not isinstance(self, GT.GlobalTensor):
                return orig(self, *args, **kw)
            if placement is None:
                placement = self.placement
            if sbp is None:
                sbp = self.sbp if isinstance(self, GT.GlobalTensor) else S.broadcast
            if kw.get("dtype") is None:
                kw["dtype"] = self.dtype
            kw.pop("device", None)
            if "size" in kw:
                args = (kw.pop("size"),) + args
            return factory(*args, placement=placement, sbp=sbp, **kw)
        method.__name__ = name
        setattr(T, name, method)
    for _n, _f in (("new_zeros", zeros), ("new_ones", ones), ("new_empty", empty), ("new_full", full)):
        _new_method(_n, _f)

    _to = T.to

    def to(self, *args, **kwargs):
        """``tensor.to(flow.Tensor)`` — the spelling that turns a graph-side proxy back into its tensor — is the
        identity on a tensor; everything else is torch's ``to``."""
        if args and (args[0] is Tensor or args[0] is torch.Tensor):
            return self
        return _to(self, *args, **kwargs)
    T.to = to
    _numpy = T.numpy

    def numpy(self, *args, **kwargs):
        """The values as a numpy array: detaches, and copies device tensors to the host first (the reference's
        ``Tensor.numpy`` does both implicitly)."""
        t = self.detach()
        if t.is_cuda:
            t = t.cpu()
        if t.is_conj():
            t = t.resolve_conj()
        if t._is_zerotensor():
            t = torch.zeros(t.shape, dtype=t.dtype)          # the symbolic all-zero gradient of autograd, made real
        if t.dtype == torch.bfloat16:
            t = t.float()                                    # numpy has no bfloat16: float32, as in the reference
        return _numpy(t, *args, **kwargs)
    T.numpy = numpy
    T.is_view = lambda self: self._is_view()
    T._meta_repr = lambda self: f"tensor(..., size={tuple(self.shape)}, dtype={self.dtype}, device={self.device})"
