"""Functions whose reference signature differs from the torch function of the same name (extra positional
arguments, scalar operands where torch wants tensors, looser index dtypes, ``generator`` / ``addend`` / ``dtype``
keywords).  Installed over the top-level namespace, ``flow.nn.functional`` and ``flow._C``
(signatures: oneflow/core/functional/functional_api.yaml; python/oneflow/nn/modules/*.py)."""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


def addmm(input, mat1, mat2, alpha=1, beta=1):
    """``beta * input + alpha * (mat1 @ mat2)`` with ``alpha`` / ``beta`` also accepted positionally
    (reference: python/oneflow/nn/modules/math_ops.py:195-250)."""
    return torch.addmm(input, mat1, mat2, beta=beta, alpha=alpha)


def matmul(input, other, transpose_a=False, transpose_b=False, alpha=1.0):
    """MatMul with optional transposes of the two innermost axes and a scale."""
    a = input.transpose(-1, -2) if transpose_a else input
    b = other.transpose(-1, -2) if transpose_b else other
    from .global_tensor import matmul_any
    out = matmul_any(a, b)
    return out if alpha == 1.0 else out * alpha


def _gen(generator, device):
    from .generator import resolve
    return resolve(generator, device)


def bernoulli(input, p=None, *, dtype=None, generator=None, inplace=False, out=None):
    """Bernoulli draws with probabilities ``input`` (or one probability ``p``), in ``dtype`` (default: float32 for
    integer inputs' sake as well), optionally written back into ``input``."""
    generator = _gen(generator, input.device)
    if p is None:
        res = torch.bernoulli(input.float() if not input.is_floating_point() else input, generator=generator)
    else:
        res = torch.empty_like(input, dtype=torch.float32).bernoulli_(float(p), generator=generator)
    if inplace:
        return input.copy_(res.to(input.dtype))
    return res.to(dtype if dtype is not None else (input.dtype if input.is_floating_point() else torch.float32))


def one_hot(input, num_classes=-1, on_value=1, off_value=0):
    """One-hot of any integer index dtype, with selectable on / off values; the result is int64 unless a value is a
    float."""
    oh = F.one_hot(input.long(), num_classes)
    if on_value == 1 and off_value == 0:
        return oh
    dt = torch.float32 if isinstance(on_value, float) or isinstance(off_value, float) else torch.int64
    return torch.where(oh.bool(), torch.tensor(on_value, dtype=dt, device=input.device),
                       torch.tensor(off_value, dtype=dt, device=input.device))


def dropout(input, p=0.5, training=True, inplace=False, generator=None, *, addend=None):
    """Dropout with an optional generator for the mask and an ``addend`` added to the result (the fused residual)."""
    if training and p > 0:
        generator = _gen(generator, input.device)
        if generator is None:
            out = F.dropout(input, p, True, inplace)
        else:
            keep = (torch.rand(input.shape, generator=generator, device=generator.device) >= p).to(input.device)
            out = input.mul_(keep / (1 - p)) if inplace else input * (keep / (1 - p))
    else:
        out = input
    return out if addend is None else out + addend


class Dropout(torch.nn.Dropout):
    """``nn.Dropout(p, inplace, generator)`` whose ``forward(x, addend=None)`` adds ``addend`` after dropping
    (reference: python/oneflow/nn/modules/dropout.py:43-57)."""

    def __init__(self, p=0.5, inplace=False, generator=None):
        super().__init__(p, inplace)
        self.generator = generator

    def forward(self, x, addend=None):
        return dropout(x, self.p, self.training, self.inplace, self.generator, addend=addend)


def _scalar_ok(fn):
    def f(input, other):
        if not isinstance(other, torch.Tensor):
            other = torch.as_tensor(other, device=input.device)
        if not isinstance(input, torch.Tensor):
            input = torch.as_tensor(input, device=other.device)
        return fn(input, other)
    f.__name__ = fn.__name__
    f.__doc__ = f"torch.{fn.__name__} that also takes a Python scalar on either side."
    return f


logical_and, logical_or, logical_xor = _scalar_ok(torch.logical_and), _scalar_ok(torch.logical_or), _scalar_ok(torch.logical_xor)


def where(condition, x=None, y=None):
    """``where`` whose condition may be any dtype (non-zero is true) and whose branches may be Python scalars."""
    if condition.dtype != torch.bool:
        condition = condition != 0
    if x is None and y is None:
        return torch.where(condition)
    return torch.where(condition, x, y)


def masked_select(input, mask):
    return torch.masked_select(input, mask if mask.dtype == torch.bool else mask != 0)


def masked_fill(input, mask, value):
    return torch.masked_fill(input, mask if mask.dtype == torch.bool else mask != 0, value)


def nonzero(input, as_tuple=False):
    return torch.nonzero(input, as_tuple=as_tuple)


def empty_strided(size, stride, dtype=None, device=None, requires_grad=False, pin_memory=False, **kw):
    t = torch.empty_strided(tuple(size), tuple(stride), dtype=dtype, device=device, pin_memory=pin_memory)
    return t.requires_grad_(True) if requires_grad and (t.is_floating_point() or t.is_complex()) else t


class PixelShuffle(torch.nn.Module):
    """Pixel shuffle with separate height and width factors: ``[N, C*h*w, H, W] -> [N, C, H*h, W*w]``
    (reference: python/oneflow/nn/modules/pixelshuffle.py)."""

    def __init__(self, upscale_factor=None, h_upscale_factor=None, w_upscale_factor=None):
        super().__init__()
        if upscale_factor is not None:
            if h_upscale_factor is not None or w_upscale_factor is not None:
                raise ValueError("give either upscale_factor or h_upscale_factor and w_upscale_factor")
            h_upscale_factor = w_upscale_factor = upscale_factor
        if h_upscale_factor is None or w_upscale_factor is None:
            raise ValueError("h_upscale_factor and w_upscale_factor are both required")
        if h_upscale_factor <= 0 or w_upscale_factor <= 0:
            raise ValueError("The scale factor of height and width must larger than zero")
        self.h_upscale_factor, self.w_upscale_factor = int(h_upscale_factor), int(w_upscale_factor)

    def forward(self, input):
        n, c, h, w = input.shape
        hf, wf = self.h_upscale_factor, self.w_upscale_factor
        if c % (hf * wf):
            raise ValueError("The channels of input tensor must be divisible by (h_upscale_factor * w_upscale_factor)")
        out = input.reshape(n, c // (hf * wf), hf, wf, h, w).permute(0, 1, 4, 2, 5, 3)
        return out.reshape(n, c // (hf * wf), h * hf, w * wf)

    def extra_repr(self):
        return f"w_upscale_factor={self.w_upscale_factor}, h_upscale_factor={self.h_upscale_factor}"


def _C_slice(x, start, stop, step):
    """``_C.slice(x, start, stop, step)``: one entry per leading axis."""
    return x[tuple(slice(a, b, c) for a, b, c in zip(start, stop, step))]


def _C_slice_update(x, update, start, stop, step, inplace=False):
    """``_C.slice_update(ref, value, start, stop, step)``: writes ``value`` into the slice; differentiable in both."""
    out = x if inplace else x.clone()
    out[tuple(slice(a, b, c) for a, b, c in zip(start, stop, step))] = update
    return out


_TYPE_NAMES = {torch.float32: "FloatTensor", torch.float64: "DoubleTensor", torch.float16: "HalfTensor",
               torch.bfloat16: "BFloat16Tensor", torch.uint8: "ByteTensor", torch.int8: "CharTensor", torch.int16: "ShortTensor",
               torch.int32: "IntTensor", torch.int64: "LongTensor", torch.bool: "BoolTensor",
               torch.complex64: "ComplexFloatTensor", torch.complex128: "ComplexDoubleTensor"}


def _tensor_type(self, dtype=None, non_blocking=False, **kw):
    """``Tensor.type()`` names the type as ``oneflow.FloatTensor`` / ``oneflow.cuda.FloatTensor``; with an argument
    (a dtype, a type name or a typed-tensor class) it converts."""
    if dtype is None:
        return ("oneflow.cuda." if self.is_cuda else "oneflow.") + _TYPE_NAMES[self.dtype]
    if isinstance(dtype, torch.dtype):
        return self.to(dtype)
    name = dtype if isinstance(dtype, str) else getattr(dtype, "__name__", str(dtype))
    cuda = ".cuda." in "." + name or getattr(dtype, "is_cuda", False) is True
    short = name.split(".")[-1]
    if short == "Tensor":
        short = "FloatTensor"               # ``flow.Tensor`` is the float32 host tensor type
    for dt, n in _TYPE_NAMES.items():
        if n == short:
            out = self.to(dt)
            if cuda and not out.is_cuda:
                out = out.cuda()
            elif not cuda and out.is_cuda and (not isinstance(dtype, str) or name.startswith(("oneflow.", "torch."))):
                out = out.cpu()             # a host tensor type (class or qualified name) names the host as well
            return out
    raise ValueError(f"invalid type: '{name}'")


def sort(input, dim=-1, descending=False, stable=True):
    """Sort with ties kept in index order (the reference's sort is stable; results match numpy's on small inputs)."""
    return torch.sort(input, dim=dim, descending=descending, stable=stable)


def argsort(input, dim=-1, descending=False, stable=True):
    return torch.argsort(input, dim=dim, descending=descending, stable=stable)


def _C_group_norm(x, gamma=None, beta=None, affine=False, num_groups=1, epsilon=1e-5, data_format="channels_first",
                  activation="none"):
    """``_C.group_norm``: group normalisation over channels-first or channels-last data with an optional fused
    activation (``"none"`` or ``"silu"``)."""
    if data_format == "channels_last":
        x = x.movedim(-1, 1)
    y = F.group_norm(x, num_groups, gamma if affine else None, beta if affine else None, epsilon)
    if activation == "silu":
        y = F.silu(y)
    elif activation not in (None, "none"):
        raise ValueError(f"group_norm: unsupported activation {activation!r}")
    return y.movedim(1, -1) if data_format == "channels_last" else y


def _C_roi_align(x, rois, spatial_scale, pooled_h, pooled_w, sampling_ratio, aligned):
    """``_C.roi_align(x, rois, spatial_scale, pooled_h, pooled_w, sampling_ratio, aligned)``."""
    from .toplevel_extra import roi_align
    return roi_align(x, rois, spatial_scale, pooled_h, pooled_w, sampling_ratio, aligned)


def _long_target(t):
    return t.long() if isinstance(t, torch.Tensor) and t.dtype in (torch.int32, torch.int16, torch.int8, torch.uint8) else t


def cross_entropy(input, target, weight=None, size_average=None, ignore_index=-100, reduce=None, reduction="mean",
                  label_smoothing=0.0):
    """``cross_entropy`` whose class-index targets may be any integer dtype (the reference takes int32 labels)."""
    return F.cross_entropy(input, _long_target(target), weight, ignore_index=ignore_index, reduction=reduction,
                           label_smoothing=label_smoothing)


def nll_loss(input, target, weight=None, size_average=None, ignore_index=-100, reduce=None, reduction="mean"):
    return F.nll_loss(input, _long_target(target), weight, ignore_index=ignore_index, reduction=reduction)


class CrossEntropyLoss(torch.nn.CrossEntropyLoss):
    def forward(self, input, target):
        return super().forward(input, _long_target(target))


class NLLLoss(torch.nn.NLLLoss):
    def forward(self, input, target):
        return super().forward(input, _long_target(target))


_LOW = (torch.bfloat16, torch.float16)


def softsign(input):
    """``x / (1 + |x|)``; 16-bit inputs are evaluated in float32 and rounded once (the reference's kernels do the
    arithmetic in float: oneflow/core/ep/common/primitive/unary_functor.h)."""
    if input.dtype in _LOW:
        return F.softsign(input.float()).to(input.dtype)
    return F.softsign(input)


def rsqrt(input):
    """``1 / sqrt(x)``, rounded once for 16-bit host tensors as well."""
    if input.dtype in _LOW and not input.is_cuda:
        return torch.rsqrt(input.float()).to(input.dtype)
    return torch.rsqrt(input)


def install():
    """Put the functions above where the reference has them."""
    import oneflow_b200 as flow
    from .. import _C
    from ..nn import functional as NF
    top = dict(addmm=addmm, matmul=matmul, bernoulli=bernoulli, logical_and=logical_and, logical_or=logical_or,
               logical_xor=logical_xor, where=where, masked_select=masked_select, masked_fill=masked_fill, nonzero=nonzero,
               empty_strided=empty_strided, sort=sort, argsort=argsort)
    for k, v in top.items():
        setattr(flow, k, v)
        setattr(_C, k, v)
    flow.nn.CrossEntropyLoss, flow.nn.NLLLoss = CrossEntropyLoss, NLLLoss
    flow.softsign = _C.softsign = NF.softsign = softsign
    flow.rsqrt = _C.rsqrt = rsqrt
    for k, v in dict(one_hot=one_hot, dropout=dropout, cross_entropy=cross_entropy, nll_loss=nll_loss).items():
        setattr(NF, k, v)
        setattr(_C, k, v)
    flow.nn.Dropout = Dropout
    flow.nn.PixelShuffle = PixelShuffle
    _C.slice = _C_slice
    _C.group_norm = _C_group_norm
    _C.roi_align = _C_roi_align
    _C.slice_update = _C_slice_update
    torch.Tensor.type = _tensor_type

    T = torch.Tensor
    T.contiguous_ = lambda self: _C.contiguous_(self)
    T.sort = lambda self, dim=-1, descending=False, stable=True: sort(self, dim, descending, stable)
    T.argsort = lambda self, dim=-1, descending=False, stable=True: argsort(self, dim, descending, stable)
    T.addmm = lambda self, mat1, mat2, alpha=1, beta=1: addmm(self, mat1, mat2, alpha, beta)
    T.logical_and = lambda self, other: logical_and(self, other)
    T.logical_or = lambda self, other: logical_or(self, other)
    T.logical_xor = lambda self, other: logical_xor(self, other)
    _copy = T.copy_

    def copy_(self, other, non_blocking=False):
        """``copy_`` that also takes a numpy array (the reference's ``Tensor.copy_`` does)."""
        if isinstance(other, np.ndarray):
            other = torch.from_numpy(other)
        if self.is_leaf and self.requires_grad and torch.is_grad_enabled():
            with torch.no_grad():                   # overwriting a parameter's value is not a differentiable step
                return _copy(self, other, non_blocking)
        return _copy(self, other, non_blocking)
    T.copy_ = copy_
