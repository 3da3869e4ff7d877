"""More of ``flow._C``: the functional ops of the reference (oneflow/core/functional/functional_api.yaml) that neither
``_C.py`` / ``_C_extra.py`` define nor torch offers under the same name and argument order.  Every function names
the functor it stands for.  Backward-only functors (``*_grad``) are not part of the public surface: autograd derives
them."""
from __future__ import annotations

import math

import torch

from .framework.generator import resolve as _resolve_gen
import torch.nn.functional as F


def _list(v):
    if v is None:
        return None
    return [int(v)] if isinstance(v, int) else [int(x) for x in v]


# ------------------------------------------------------------------------------------------------ in-place arithmetic
def mul_(input, other):
    """InplaceMul / InplaceScalarMul"""
    return input.mul_(other)


def addcmul_(input, tensor1, tensor2, *, value=1):
    """InplaceAddcmul"""
    return input.addcmul_(tensor1, tensor2, value=value)


def addcdiv_(input, tensor1, tensor2, *, value=1):
    """InplaceAddCDiv"""
    return input.addcdiv_(tensor1, tensor2, value=value)


def greater_(input, other):
    """InplaceBroadcastGreater: the comparison result is written into ``input`` in its own dtype."""
    return input.copy_(torch.gt(input, other).to(input.dtype))


def host_scalar_add_by_tensor(x, scalar):
    """HostScalarAddByTensor: adds a one-element host tensor to every element."""
    return x + scalar.reshape(()).to(x.device)


def broadcast_equal(input, other):
    """BroadcastEqual / ScalarLogicalEqual"""
    return torch.eq(torch.as_tensor(input) if not isinstance(input, torch.Tensor) else input, other)


def broadcast_pow(x, y):
    """BroadcastPow"""
    return torch.pow(x, y)


def trunc_divide(input, other, *, inplace=False):
    """TruncDiv / ScalarTruncDiv"""
    return input.div_(other, rounding_mode="trunc") if inplace else torch.div(input, other, rounding_mode="trunc")


def not_equal_zero(x):
    """NotEqualZero"""
    return (x != 0).to(x.dtype)


def reciprocal_no_nan(x):
    """ReciprocalNoNan: 1/x with 0 where x is 0."""
    return torch.where(x == 0, torch.zeros_like(x), 1.0 / x)


def rint(x):
    """Rint: round half to even."""
    return torch.round(x)


def trigamma(x):
    """Trigamma"""
    return torch.polygamma(1, x)


def zeta(x, other):
    """BroadcastZeta / ZetaScalarTensor / ZetaTensorScalar (Hurwitz zeta)."""
    return torch.special.zeta(x, other)


def fast_gelu(x):
    """FastGelu: the tanh approximation."""
    return F.gelu(x, approximate="tanh")


def gelu_with_approximate(x, approximate="none"):
    """GeluWithApproximate"""
    return F.gelu(x, approximate=approximate)


def sqrt_square_sum(x):
    """SqrtSquareSum: the 2-norm of all elements."""
    return torch.linalg.vector_norm(x.float()).to(x.dtype)


def l2_normalize(input, axis=0, epsilon=1e-12):
    """L2Normalize: x / sqrt(max(sum(x^2, axis), epsilon))."""
    sq = input.float().pow(2).sum(axis, keepdim=True).clamp_min(epsilon)
    return (input.float() * torch.rsqrt(sq)).to(input.dtype)


def T(input):
    """TransposeAllDimProperty"""
    return input.permute(*reversed(range(input.dim())))


# ------------------------------------------------------------------------------------------------ reductions
def _reduce(fn, x, dim, keepdim, dtype=None):
    if dtype is not None:
        x = x.to(dtype)
    if dim is None:
        return fn(x)
    dims = _list(dim)
    return fn(x, dim=dims, keepdim=keepdim) if dims else (fn(x) if not keepdim else fn(x).reshape([1] * x.dim()))


def reduce_sum(x, dim=None, keepdim=False, *, dtype=None):
    """ReduceSum / ReduceSumWhole"""
    return _reduce(torch.sum, x, dim, keepdim, dtype)


def reduce_nansum(input, dim=None, keepdim=False, *, dtype=None):
    """ReduceNanSum / ReduceNanSumWhole"""
    return _reduce(torch.nansum, input, dim, keepdim, dtype)


def reduce_mean(x, dim=None, keepdim=False):
    """ReduceMean / ReduceMeanWhole"""
    return _reduce(torch.mean, x, dim, keepdim)


def reduce_prod(x, dim=None, keepdim=False, *, dtype=None):
    """ReduceProd / ReduceProdWhole (several axes: one after the other)."""
    if dtype is not None:
        x = x.to(dtype)
    if dim is None:
        return torch.prod(x)
    for d in sorted((d % x.dim() for d in _list(dim)), reverse=True):
        x = torch.prod(x, dim=d, keepdim=keepdim)
    return x


def reduce_all(x, dim=None, keepdim=False):
    """ReduceAll / ReduceAllWhole"""
    return torch.all(x) if dim is None else torch.all(x, dim=_list(dim), keepdim=keepdim)


def reduce_any(x, dim=None, keepdim=False):
    """ReduceAny / ReduceAnyWhole"""
    return torch.any(x) if dim is None else torch.any(x, dim=_list(dim), keepdim=keepdim)


def reduce_max(x, axis, keepdim=False):
    """ReduceMax"""
    return torch.amax(x, dim=_list(axis), keepdim=keepdim)


def reduce_min(x, axis, keepdim=False):
    """ReduceMin"""
    return torch.amin(x, dim=_list(axis), keepdim=keepdim)


def _device_stage(x, axis, fn):
    """First stage of a two-stage max / min over a split tensor: the local extreme (kept dims), a 0/1 mask of where
    it is attained and how many elements attain it — what the gradient needs to split ties evenly."""
    dims = _list(axis)
    out = fn(x, dim=dims, keepdim=True)
    mask = (x == out).to(torch.int32)
    count = mask.sum(dim=dims, keepdim=True).to(torch.int32)
    return out, mask, count


def reduce_max_device_stage(input, axis):
    """ReduceMaxDeviceStage -> (out, mask, count)"""
    return _device_stage(input, axis, torch.amax)


def reduce_min_device_stage(input, axis):
    """ReduceMinDeviceStage -> (out, mask, count)"""
    return _device_stage(input, axis, torch.amin)


def _global_stage(x, device_count, axis, keepdims, fn):
    dims = _list(axis)
    out = fn(x, dim=dims, keepdim=True)
    mask = (x == out).to(torch.int32) * device_count.to(torch.int32)
    return (out if keepdims else out.squeeze(dims)), mask


def reduce_max_global_stage(input, device_count, axis, keepdims=False):
    """ReduceMaxGlobalStage: second stage over the gathered per-device extremes -> (out, mask weighted by count)."""
    return _global_stage(input, device_count, axis, keepdims, torch.amax)


def reduce_min_global_stage(input, device_count, axis, keepdims=False):
    """ReduceMinGlobalStage"""
    return _global_stage(input, device_count, axis, keepdims, torch.amin)


def reduce_sum_like(input, like, axis):
    """ReduceSumLike: sum over ``axis`` and take ``like``'s shape."""
    dims = _list(axis)
    return (input.sum(dim=dims) if dims else input).reshape(like.shape)


def broadcast_reduce_sum_like(input, like):
    """BroadcastReduceSumLike: undo a broadcast — sum the axes that ``like`` does not have or has with extent 1."""
    return input.sum_to_size(like.shape) if tuple(input.shape) != tuple(like.shape) else input


# ------------------------------------------------------------------------------------------------ shapes and copies
def expand_dims(input, dim):
    """ExpandDims"""
    return input.unsqueeze(dim)


def unsqueeze_(input, dim):
    """InplaceUnsqueeze"""
    return input.unsqueeze_(dim)


def squeeze_(x, dim=None):
    """InplaceSqueeze"""
    if dim is None:
        return x.squeeze_()
    for d in sorted((d % max(x.dim(), 1) for d in _list(dim)), reverse=True):
        x.squeeze_(d)
    return x


def unsqueeze_multiple(input, dim, dims):
    """UnsqueezeMultiple: insert size-1 axes so that the kept axes land at positions ``dim`` of a ``dims``-D result."""
    keep = sorted(d % dims for d in _list(dim)) if dim is not None and len(_list(dim)) else []
    if not keep:
        keep = list(range(dims - input.dim(), dims))
    shape = [1] * dims
    for src, d in enumerate(keep):
        shape[d] = input.shape[src]
    return input.reshape(shape)


def reshape_like(input, like):
    """ReshapeLike"""
    return input.reshape(like.shape)


def cast_like(x, like):
    """CastLike"""
    return x.to(like.dtype)


def identity(input):
    """Identity: a new tensor object sharing the data (a graph node of its own for autograd)."""
    return input.view_as(input)


amp_white_identity = identity     # AmpWhiteIdentity: marks a point as safe for low precision; autocast decides here
amp_black_identity = identity     # AmpBlackIdentity


def contiguous_(input):
    """InplaceToContiguous"""
    if not input.is_contiguous():
        input.data = input.data.contiguous()
    return input


def slice_view_1d_contiguous(x, start, end):
    """SliceView1dContiguous: rows [start, end) of the leading axis as a view."""
    return x[start:end]


def copy(x, device_type=None, device_id=None, pin_memory=False):
    """Copy: to a device given as (type, id) or as a device object."""
    dev = torch.device(device_type, device_id) if isinstance(device_type, str) and device_id is not None and device_type != "cpu" \
        else torch.device(device_type)
    y = x.to(dev, copy=True)
    return y.pin_memory() if pin_memory and dev.type == "cpu" and torch.cuda.is_available() else y


def to(x, *args, **kwargs):
    """To"""
    return x.to(*args, **kwargs)


def pin_memory(input):
    """PinMemory"""
    return input.pin_memory() if torch.cuda.is_available() and not input.is_cuda else input


def unfold_tensor(x, dimension, size, step):
    """UnfoldTensor"""
    return x.unfold(dimension, size, step)


def split_like(x, like, axis):
    """SplitLike: split ``x`` along ``axis`` into pieces as long as the tensors of ``like``."""
    return tuple(torch.split(x, [t.shape[axis] for t in like], dim=axis))


def tensor_getitem(x, index):
    """TensorGetItem"""
    return x[index]


def tensor_setitem(x, index, value):
    """TensorSetItem"""
    x[index] = value


def repeat_interleave_index(input, cumsum, dim):
    """RepeatInterLeaveIndex: for repeat counts ``input`` with inclusive prefix sums ``cumsum``, the source index of
    every output position (``[0,0,1,2,2,2]`` for counts ``[2,1,3]``)."""
    total = int(cumsum[-1])
    return torch.searchsorted(cumsum, torch.arange(total, device=input.device, dtype=cumsum.dtype), right=True).to(torch.int32)


def select_top_n(inputs, n):
    """SelectTopN: the first ``n`` tensors of a tuple."""
    return tuple(inputs[:n])


def stream_touch(x):
    """StreamTouch: keeps the tensors alive until the current stream has passed this point."""
    if torch.cuda.is_available():
        s = torch.cuda.current_stream()
        for t in x:
            if t.is_cuda:
                t.record_stream(s)


def throw_error(input):
    """ThrowError: raises (used by tests of error propagation)."""
    raise RuntimeError("throw_error op was called")


# ------------------------------------------------------------------------------------------------ constants / random
def constant(shape, value, *, dtype, device=None):
    """Constant"""
    return torch.full(tuple(shape), value, dtype=dtype, device=device)


def tensor_constant(shape, value, *, dtype, device=None):
    """TensorConstant: fill with the value held by a one-element tensor, no host sync."""
    out = torch.empty(tuple(shape), dtype=dtype, device=device if device is not None else value.device)
    return out.copy_(value.reshape(()).to(out.device).expand(out.shape))


def global_constant(shape, value, *, dtype, placement, sbp):
    """GlobalConstant"""
    import oneflow_b200 as flow
    return flow.full(tuple(shape), value, dtype=dtype, placement=placement, sbp=sbp)


def global_tensor_constant(shape, value, *, dtype, placement, sbp):
    """GlobalTensorConstant"""
    import oneflow_b200 as flow
    v = value.to_local() if hasattr(value, "to_local") and getattr(value, "is_global", False) else value
    return flow.full(tuple(shape), v.reshape(()).item(), dtype=dtype, placement=placement, sbp=sbp)


def global_empty(shape, *, dtype, placement, sbp):
    """GlobalEmpty"""
    import oneflow_b200 as flow
    return flow.empty(tuple(shape), dtype=dtype, placement=placement, sbp=sbp)


def global_arange(*args, dtype=None, placement, sbp):
    """GlobalArange(start, end, step) / GlobalArange(end)"""
    import oneflow_b200 as flow
    return flow.arange(*args, dtype=dtype, placement=placement, sbp=sbp)


def bernoulli_(input, p=None, *, dtype=None, generator=None):
    """BernoulliInplace (probabilities taken from ``input``) / BernoulliProbInplace (one probability ``p``)."""
    generator = _resolve_gen(generator, input.device)
    if p is None:
        return input.copy_(torch.bernoulli(input, generator=generator))
    return input.bernoulli_(p, generator=generator)


def exponential_(x, lambd=1.0, generator=None):
    """Exponential"""
    return x.exponential_(lambd, generator=_resolve_gen(generator, x.device))


def uniform_(x, from_=0.0, to=1.0, **kw):
    """InplaceUniform"""
    return x.uniform_(kw.get("from", from_), to)


def eye_(x):
    """EyeInplace: ones on the main diagonal, zeros elsewhere."""
    x.zero_()
    x.diagonal().fill_(1)
    return x


def tril_(x, diagonal=0):
    """InplaceTril"""
    return x.tril_(diagonal)


def triu_(x, diagonal=0):
    """InplaceTriu"""
    return x.triu_(diagonal)


# ------------------------------------------------------------------------------------------------ gather / scatter
def dim_gather(input, dim, index, sparse_grad=False):
    """DimGather"""
    return torch.gather(input, dim, index.long(), sparse_grad=sparse_grad)


def arg_sort(input, direction):
    """ArgSort over the last axis; ``direction`` is ``"ASCENDING"`` or ``"DESCENDING"``."""
    return torch.argsort(input, dim=-1, descending=direction.upper() == "DESCENDING", stable=True).to(torch.int32)


def _nd_index(indices):
    idx = indices.long()
    return tuple(idx[..., i] for i in range(idx.shape[-1]))


def scatternd(indices, updates, shape):
    """ScatterNd: zeros of ``shape`` with ``updates`` added at the n-d ``indices`` (duplicates accumulate)."""
    out = torch.zeros(tuple(shape), dtype=updates.dtype, device=updates.device)
    return out.index_put_(_nd_index(indices), updates, accumulate=True)


def scatterndlike(like, updates, indices):
    """ScatterNdLike"""
    return scatternd(indices, updates, like.shape).to(like.dtype)


def tensor_scatter_nd_update(tensor, indices, updates, inplace=False):
    """TensorScatterNdUpdate: overwrite the addressed slices."""
    out = tensor if inplace else tensor.clone()
    return out.index_put_(_nd_index(indices), updates.to(out.dtype))


def scatter_update(input, dim, index, src, *, inplace=False):
    """DimScatterUpdate / DimScatterUpdateScalar"""
    out = input if inplace else input.clone()
    return out.scatter_(dim, index.long(), src)


def scatter_mul(input, dim, index, src, *, inplace=False):
    """DimScatterMul / DimScatterMulScalar"""
    out = input if inplace else input.clone()
    if not isinstance(src, torch.Tensor):
        src = torch.full_like(index, src, dtype=out.dtype)
    return out.scatter_reduce_(dim, index.long(), src, reduce="prod", include_self=True)


def scatter_add_like(like, dim, index, src):
    """DimScatterAddLike"""
    return torch.zeros_like(like).scatter_add_(dim, index.long(), src.to(like.dtype))


def unsorted_segment_sum(x, segment_ids, axis, num_segments):
    """UnsortedSegmentSum: out[..., s, ...] = sum of the slices of ``x`` along ``axis`` whose id is ``s``."""
    shape = list(x.shape)
    shape[axis] = num_segments
    out = torch.zeros(shape, dtype=x.dtype, device=x.device)
    return out.index_add_(axis, segment_ids.long().reshape(-1), x)


def unsorted_segment_sum_like(x, segment_ids, like, axis):
    """UnsortedSegmentSumLike"""
    return unsorted_segment_sum(x, segment_ids, axis, like.shape[axis]).to(like.dtype)


def unsorted_batch_segment_sum(data, segment_ids, num_segments):
    """UnsortedBatchSegmentSum: per batch row, ``out[b, s] = sum over j with segment_ids[b, j] == s of data[b, j]``."""
    lead = segment_ids.shape[:-1]
    out = torch.zeros(tuple(lead) + (num_segments,) + tuple(data.shape[segment_ids.dim():]), dtype=data.dtype, device=data.device)
    idx = segment_ids.long()
    while idx.dim() < data.dim():
        idx = idx.unsqueeze(-1)
    return out.scatter_add_(segment_ids.dim() - 1, idx.expand_as(data), data)


# ------------------------------------------------------------------------------------------------ linear algebra
def batch_matmul(a, b, transpose_a=False, transpose_b=False, alpha=1.0):
    """BatchMatMul"""
    out = torch.matmul(a.transpose(-1, -2) if transpose_a else a, b.transpose(-1, -2) if transpose_b else b)
    return out if alpha == 1.0 else out * alpha


def matrix_vector_product(input, vec):
    """MatrixVectorProduct"""
    return torch.mv(input, vec)


def vector_matrix_product(vec, input):
    """VectorMatrixProduct"""
    return torch.mv(input.t(), vec)


def vector_norm(input, ord=2, dim=None, keepdim=False, *, dtype=None):
    """VectorNorm"""
    return torch.linalg.vector_norm(input, ord=ord, dim=_list(dim) if dim is not None else None, keepdim=keepdim, dtype=dtype)


def matrix_norm(input, ord, dim, keepdim=False, *, dtype=None):
    """MatrixNorm"""
    return torch.linalg.matrix_norm(input, ord=ord, dim=tuple(_list(dim)), keepdim=keepdim, dtype=dtype)


def inv(x):
    """Inv"""
    return torch.linalg.inv(x)


def linalg_cross(input, other, dim=None):
    """LinalgCross"""
    return torch.linalg.cross(input, other, dim=-1 if dim is None else dim)


def bias_add(x, bias, axis=1):
    """BiasAdd: a 1-D bias along ``axis``."""
    shape = [1] * x.dim()
    shape[axis] = -1
    return x + bias.reshape(shape)


# ------------------------------------------------------------------------------------------------ fft
_NORM_MODES = {0: "backward", 1: "forward", 2: "ortho"}


def fft_c2c(input, n=None, dims=None, norm_mode=0, forward=True, normalized=False):
    """FftC2C"""
    fn = torch.fft.fftn if forward else torch.fft.ifftn
    norm = _NORM_MODES[norm_mode]
    if not forward:
        norm = {"backward": "backward", "forward": "forward", "ortho": "ortho"}[norm]
    return fn(input, s=_list(n), dim=_list(dims), norm=norm)


def fft_r2c(input, n=None, dims=None, norm_mode=0, onesided=False, forward=True, normalized=False):
    """FftR2C"""
    norm = _NORM_MODES[norm_mode]
    if onesided:
        out = torch.fft.rfftn(input, s=_list(n), dim=_list(dims), norm=norm)
    else:
        out = torch.fft.fftn(input, s=_list(n), dim=_list(dims), norm=norm)
    return out if forward else out.conj()


def fft_c2r(input, n=None, dims=None, norm_mode=0, forward=True, normalized=False):
    """FftC2R"""
    x = input.conj() if forward else input
    return torch.fft.irfftn(x, s=_list(n), dim=_list(dims), norm=_NORM_MODES[norm_mode])


def _fft1(fn):
    def f(input, n=-1, dim=-1, norm=None):
        return fn(input, n=None if n is None or n < 0 else n, dim=dim, norm=norm)
    return f


def _fftn(fn, default_dim):
    def f(input, s=None, dim=default_dim, norm=None):
        return fn(input, s=_list(s), dim=_list(dim) if dim is not None else None, norm=norm)
    return f


ifft, rfft, irfft, hfft, ihfft = (_fft1(f) for f in (torch.fft.ifft, torch.fft.rfft, torch.fft.irfft, torch.fft.hfft, torch.fft.ihfft))
fft2, ifft2, rfft2, irfft2, hfft2, ihfft2 = (_fftn(f, (-2, -1)) for f in (torch.fft.fft2, torch.fft.ifft2, torch.fft.rfft2,
                                                                         torch.fft.irfft2, torch.fft.hfft2, torch.fft.ihfft2))
fftn, ifftn, rfftn, irfftn, hfftn, ihfftn = (_fftn(f, None) for f in (torch.fft.fftn, torch.fft.ifftn, torch.fft.rfftn,
                                                                      torch.fft.irfftn, torch.fft.hfftn, torch.fft.ihfftn))


# ------------------------------------------------------------------------------------------------ nn: norms, pools, pads, resampling
def normalization(x, moving_mean=None, moving_variance=None, gamma=None, beta=None, axis=1, epsilon=1e-5, momentum=0.9,
                  is_training=False):
    """Normalization: batch norm over every axis but ``axis``.  ``momentum`` is the weight of the OLD running value
    (the reference's convention), i.e. ``1 - momentum`` in torch's."""
    if axis != 1:
        x = x.movedim(axis, 1)
    y = F.batch_norm(x, moving_mean, moving_variance, gamma, beta, is_training or moving_mean is None, 1.0 - momentum, epsilon)
    return y.movedim(1, axis) if axis != 1 else y


def normalization_add_relu(x, addend=None, moving_mean=None, moving_variance=None, gamma=None, beta=None, axis=1,
                           epsilon=1e-5, momentum=0.9, is_training=False):
    """NormalizationAddRelu: relu(batch_norm(x) + addend)."""
    y = normalization(x, moving_mean, moving_variance, gamma, beta, axis, epsilon, momentum, is_training)
    if addend is not None:
        y = y + addend
    return torch.relu(y)


def layer_norm_affine(x, gamma, beta, begin_norm_axis, begin_params_axis, epsilon):
    """LayerNormAffine: normalise over the axes from ``begin_norm_axis``; gamma / beta cover those from
    ``begin_params_axis``."""
    norm_shape = tuple(x.shape[begin_norm_axis:])
    y = F.layer_norm(x, norm_shape, None, None, epsilon)
    pshape = tuple(x.shape[begin_params_axis:])
    return y * gamma.reshape(pshape) + beta.reshape(pshape)


def _deconv(nd):
    fn = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[nd - 1]

    def f(input, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1, data_format="channels_first"):
        if data_format != "channels_first":
            input = input.movedim(-1, 1)
        y = fn(input, weight, bias, stride, padding, output_padding, groups, dilation)
        return y if data_format == "channels_first" else y.movedim(1, -1)
    f.__doc__ = f"Deconv{nd}d"
    return f


deconv1d, deconv2d, deconv3d = _deconv(1), _deconv(2), _deconv(3)


def avg_pool2d_nhwc(x, kernel_size, stride, padding, padding_before, padding_after, data_format="channels_first", ceil_mode=False):
    """TFAvgPool2D: TensorFlow-style average pooling with explicit before / after padding, padded cells excluded."""
    nhwc = data_format != "channels_first"
    if nhwc:
        x = x.permute(0, 3, 1, 2)
    pb, pa = _list(padding_before), _list(padding_after)
    xp = F.pad(x, (pb[1], pa[1], pb[0], pa[0]))
    ones = F.pad(torch.ones_like(x[:1, :1]), (pb[1], pa[1], pb[0], pa[0]))
    s = F.avg_pool2d(xp, kernel_size, stride, 0, ceil_mode, divisor_override=1)
    cnt = F.avg_pool2d(ones, kernel_size, stride, 0, ceil_mode, divisor_override=1)
    y = s / cnt
    return y.permute(0, 2, 3, 1) if nhwc else y


def constant_pad(x, pad, value=0):
    """ConstantPad"""
    return F.pad(x, _list(pad), mode="constant", value=value)


def reflection_pad(x, pad):
    """ReflectionPad"""
    return F.pad(x, _list(pad), mode="reflect")


def replication_pad(x, pad):
    """ReplicationPad"""
    return F.pad(x, _list(pad), mode="replicate")


def _upsample(mode, nd, has_align):
    def f(x, *args, **kw):
        names = {1: ["scale_factor"], 2: ["height_scale", "width_scale"], 3: ["depth_scale", "height_scale", "width_scale"]}[nd]
        names = names + (["align_corners"] if has_align else []) + ["output_size", "data_format"]
        vals = dict(zip(names, args))
        vals.update(kw)
        scales = [float(vals.get(n, 0.0)) for n in names[:nd]]
        size = vals.get("output_size")
        fmt = vals.get("data_format", "channels_first")
        if fmt != "channels_first":
            x = x.movedim(-1, 1)
        extra = {"align_corners": bool(vals.get("align_corners", False))} if has_align else {}
        if size is not None:
            y = F.interpolate(x, size=tuple(_list(size)), mode=mode, **extra)
        else:
            y = F.interpolate(x, scale_factor=scales if nd > 1 else scales[0], mode=mode, **extra)
        return y if fmt == "channels_first" else y.movedim(1, -1)
    return f


upsample_linear_1d = _upsample("linear", 1, True)
upsample_nearest_1d = _upsample("nearest", 1, False)
upsample_nearest_2d = _upsample("nearest", 2, False)
upsample_bilinear_2d = _upsample("bilinear", 2, True)
upsample_bicubic_2d = _upsample("bicubic", 2, True)
upsample_nearest_3d = _upsample("nearest", 3, False)
upsample_trilinear_3d = _upsample("trilinear", 3, True)


def image_flip(x, flip_code):
    """ImageFlip on a buffer of HWC images: code bit 0 flips horizontally, bit 1 vertically."""
    from .nn.modules.dataset import ImageFlip
    return ImageFlip()(x, flip_code)


def tensor_buffer_to_tensor(input, instance_shape, dtype):
    """TensorBufferToTensor: stack equally shaped buffer entries into ``[batch, *instance_shape]``."""
    return torch.stack([t.reshape(tuple(instance_shape)).to(dtype) for t in input.tensors])


# ------------------------------------------------------------------------------------------------ losses
def kl_div_loss(input, target, log_target=False, reduction="mean"):
    """KLDivLoss"""
    return F.kl_div(input, target, reduction=reduction, log_target=log_target)


def binary_cross_entropy_loss(input, target, weight=None, reduction="mean"):
    """BinaryCrossEntropyLoss"""
    return F.binary_cross_entropy(input, target, weight, reduction=reduction)


def binary_cross_entropy_with_logits_loss(input, target, weight=None, pos_weight=None, reduction="mean"):
    """BinaryCrossEntropyWithLogitsLoss"""
    return F.binary_cross_entropy_with_logits(input, target, weight, pos_weight=pos_weight, reduction=reduction)


def sparse_cross_entropy(prediction, label, depth=None):
    """SparseCrossEntropy: ``-log(prediction[label])`` for probabilities (not logits)."""
    p = torch.gather(prediction, -1, label.long().unsqueeze(-1)).squeeze(-1)
    return -torch.log(p)


def distributed_sparse_cross_entropy(prediction, label, depth=None):
    """SparseCrossEntropyMs: as above with the class axis split over ranks — labels outside the local range give 0
    and the partial results sum to the answer."""
    import oneflow_b200 as flow
    from .framework.global_tensor import GlobalTensor
    if isinstance(prediction, GlobalTensor):
        return sparse_cross_entropy(prediction.to_global(sbp=[flow.sbp.broadcast] * len(prediction.sbp)), label, depth)
    return sparse_cross_entropy(prediction, label, depth)


def softmax_cross_entropy(logits, label):
    """SoftmaxCrossEntropy with dense (probability) labels over the last axis, no reduction."""
    return -(label * F.log_softmax(logits.float(), dim=-1)).sum(-1).to(logits.dtype)


def cross_entropy_label_smoothing(input, target, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
    """CrossEntropyLabelSmoothing"""
    return F.cross_entropy(input, target, weight, ignore_index=ignore_index, reduction=reduction, label_smoothing=label_smoothing)


def cross_entropy_prob(input, target, weight=None, reduction="mean", label_smoothing=0.0):
    """CrossEntropyProb: class-probability targets."""
    return F.cross_entropy(input, target, weight, reduction=reduction, label_smoothing=label_smoothing)


def combined_margin_loss(x, label, m1, m2, m3):
    """CombinedMarginLoss: cos(m1 * theta + m2) - m3 on the label column."""
    from .nn.extra_modules import CombinedMarginLoss
    return CombinedMarginLoss(m1, m2, m3)(x, label)


# ------------------------------------------------------------------------------------------------ quantisation
def min_max_observer(input, quantization_formula, quantization_bit, quantization_scheme, per_layer_quantization):
    """MinMaxObserver -> (scale, zero_point)"""
    from .nn.extra_modules import MinMaxObserver
    return MinMaxObserver(quantization_formula, quantization_bit, quantization_scheme, per_layer_quantization)(input)


def moving_average_min_max_observer(input, current_train_step, moving_max, moving_min, training, stop_update_after_iters,
                                    quantization_formula, quantization_bit, quantization_scheme, momentum):
    """MovingAverageMinMaxObserver -> (scale, zero_point); ``moving_max`` / ``moving_min`` are updated in place."""
    from .nn.extra_modules import MovingAverageMinMaxObserver
    m = MovingAverageMinMaxObserver(stop_update_after_iters, quantization_formula, quantization_bit, quantization_scheme, momentum)
    m.moving_max, m.moving_min = moving_max, moving_min
    m.train(training)
    return m(input, current_train_step)


def fake_quantization(input, scale, zero_point, quantization_formula, quantization_bit, quantization_scheme):
    """FakeQuantization"""
    from .nn.extra_modules import FakeQuantization
    return FakeQuantization(quantization_formula, quantization_bit, quantization_scheme)(input, scale, zero_point)


def groupwise_dequantize(input, scale, *, zero=None, num_bits=8, symmetric=True, group_dim=-1, group_size=-1):
    """GroupwiseDequantize: ``(q - zero) * scale`` with one scale (and zero) per group of ``group_size`` consecutive
    elements along ``group_dim``; 4-bit values come packed two per byte along the last axis, high nibble first
    (reference: oneflow/user/kernels/groupwise_quantization_kernels.cu)."""
    q = input
    if num_bits == 4:
        hi, lo = (q >> 4) & 0xF, q & 0xF
        if symmetric:           # signed nibbles
            hi, lo = torch.where(hi > 7, hi - 16, hi), torch.where(lo > 7, lo - 16, lo)
        q = torch.stack([hi, lo], dim=-1).reshape(*q.shape[:-1], q.shape[-1] * 2)
    elif num_bits != 8:
        raise ValueError("num_bits must be 4 or 8")
    gd = group_dim % q.dim()
    gs = q.shape[gd] // scale.shape[gd] if group_size < 0 else group_size
    s = scale.repeat_interleave(gs, dim=gd)
    x = q.to(scale.dtype)
    if zero is not None:
        x = x - zero.repeat_interleave(gs, dim=gd).to(scale.dtype)
    return x * s


def fused_linear_with_groupwise_quantized_weight(x, w, w_scale, *, w_zero=None, b=None, num_bits=8, symmetric=True,
                                                 group_dim=-1, group_size=-1):
    """FusedLinearWithGroupwiseQuantizedWeight: ``x @ dequantize(w).T + b``."""
    wd = groupwise_dequantize(w, w_scale, zero=w_zero, num_bits=num_bits, symmetric=symmetric, group_dim=group_dim,
                              group_size=group_size)
    return F.linear(x, wd.to(x.dtype), b)


# ------------------------------------------------------------------------------------------------ rnn cells
def _fused_lstm_cell(igates, hgates, cx, b_ih=None, b_hh=None):
    """FusedLstmCell -> (hy, cy, workspace): gates ordered input, forget, cell, output."""
    g = igates + hgates
    if b_ih is not None:
        g = g + b_ih + b_hh
    i, f, c, o = g.chunk(4, dim=-1)
    i, f, c, o = torch.sigmoid(i), torch.sigmoid(f), torch.tanh(c), torch.sigmoid(o)
    cy = f * cx + i * c
    hy = o * torch.tanh(cy)
    return hy, cy, torch.cat([i, f, c, o], dim=-1)


def _fused_gru_cell(igates, hgates, hx, b_ih=None, b_hh=None):
    """FusedGruCell -> (hy, workspace): gates ordered reset, update, new."""
    if b_ih is not None:
        igates, hgates = igates + b_ih, hgates + b_hh
    ir, iz, in_ = igates.chunk(3, dim=-1)
    hr, hz, hn = hgates.chunk(3, dim=-1)
    r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
    n = torch.tanh(in_ + r * hn)
    hy = n + z * (hx - n)
    return hy, torch.cat([r, z, n, hx, hn], dim=-1)


def pack_padded_sequence(input, lengths, batch_first):
    """PackPaddedSequence -> (data, batch_sizes); sequences must be sorted by decreasing length."""
    packed = torch.nn.utils.rnn.pack_padded_sequence(input, lengths.cpu(), batch_first=batch_first, enforce_sorted=True)
    return packed.data, packed.batch_sizes


# ------------------------------------------------------------------------------------------------ multi-tensor optimizer updates
def multi_tensor_sgd_update(model, model_diff, scale, weight_decay, learning_rate_val):
    """MultiTensorSgdUpdate: one fused launch per 48 tensors on CUDA."""
    from .ops import kernels as K
    with torch.no_grad():
        K.multi_tensor_sgd(list(model_diff), list(model), None, None, lr=learning_rate_val, weight_decay=weight_decay, scale=scale)


def multi_tensor_momentum_update(model, model_diff, momentum_buf, scale, weight_decay, learning_rate_val, momentum, dampening,
                                 nesterov, maximize):
    """MultiTensorMomentumUpdate"""
    from .ops import kernels as K
    with torch.no_grad():
        K.multi_tensor_sgd(list(model_diff), list(model), None, list(momentum_buf), lr=learning_rate_val, momentum=momentum,
                           dampening=dampening, nesterov=nesterov, maximize=maximize, weight_decay=weight_decay, scale=scale)


def multi_tensor_adam_update(model, model_diff, m, v, learning_rate_val, l2, beta1, beta2, bias_correction1_val,
                             bias_correction2_val, do_bias_correction, scale, weight_decay, epsilon):
    """MultiTensorAdamUpdate: the caller passes the bias corrections ``1 - beta^t`` it computed."""
    with torch.no_grad():
        bc1 = bias_correction1_val if do_bias_correction else 1.0
        bc2 = bias_correction2_val if do_bias_correction else 1.0
        for w, g, mi, vi in zip(model, model_diff, m, v):
            gf = g.float() * scale + l2 * w
            mi.mul_(beta1).add_(gf, alpha=1 - beta1)
            vi.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
            denom = vi.sqrt() / math.sqrt(bc2) + epsilon
            w.sub_((learning_rate_val / bc1) * (mi / denom) + learning_rate_val * weight_decay * w)


def multi_tensor_yolov5_weight_update(model, model_update, d):
    """MultiTensorYoloV5WeightUpdate: the EMA step ``model = d * model + (1 - d) * model_update``, in place."""
    with torch.no_grad():
        torch._foreach_mul_(list(model), d)
        torch._foreach_add_(list(model), list(model_update), alpha=1 - d)


# ------------------------------------------------------------------------------------------------ gradient accumulation helpers
def grad_acc_repeat(input, repeat_num):
    """GradAccRepeat: the same tensor is served to every micro-step; eagerly that is the tensor itself."""
    return input


def grad_acc_collect(input, collect_num):
    """GradAccCollect: the sum over micro-steps arrives already accumulated in ``.grad`` here."""
    return input


def grad_acc_pack(input, pack_num):
    """GradAccPack: ``pack_num`` micro-batches stacked along dim 0 (a list or an already stacked tensor)."""
    return torch.cat(list(input), 0) if isinstance(input, (list, tuple)) else input


def grad_acc_unpack(input, unpack_num):
    """GradAccUnpack: split dim 0 into ``unpack_num`` micro-batches."""
    return input.chunk(unpack_num, 0)


# ------------------------------------------------------------------------------------------------ communication
def comm_broadcast(x, *, src_rank=0, inplace=True):
    """CommBroadcast / CommBroadcastTensors"""
    from . import comm
    if isinstance(x, (list, tuple)):
        return tuple(comm_broadcast(t, src_rank=src_rank, inplace=inplace) for t in x)
    t = x if inplace else x.clone()
    comm.broadcast(t, src_rank)
    return t


def local_all_gather(output, input):
    """LocalAllGather"""
    from . import comm
    comm.all_gather_into_tensor(output, input)
    return output


def local_reduce_scatter(output, input):
    """LocalReduceScatter"""
    from . import comm
    comm.reduce_scatter_tensor(output, input)
    return output


def local_reduce(x, *, dst=0, inplace=True):
    """LocalReduce"""
    from . import comm
    t = x if inplace else x.clone()
    comm.reduce(t, dst)
    return t


def send(input, dst, send_meta=True):
    """Send"""
    from . import comm
    comm.send(input, dst, send_meta)


def recv(src, shape=None, dtype=None, device=None, *, out=None):
    """Recv"""
    from . import comm
    return comm.recv(src, shape, dtype, device, out=out)


def _rebox(x, out_sbp, out_placement=None):
    return x.to_global(placement=out_placement if out_placement is not None else x.placement, sbp=out_sbp)


def eager_p_to_b(x, in_placement, out_placement, shape):
    """EagerPToB"""
    import oneflow_b200 as flow
    return _rebox(x, [flow.sbp.broadcast] * len(out_placement.hierarchy), out_placement)


def eager_b_to_s(x, in_placement, out_placement, out_sbp, shape):
    """EagerBToS"""
    return _rebox(x, out_sbp, out_placement)


def eager_s_to_b(x, in_placement, out_placement, in_sbp, shape):
    """EagerSToB"""
    import oneflow_b200 as flow
    return _rebox(x, [flow.sbp.broadcast] * len(out_placement.hierarchy), out_placement)


def eager_naive_s_to_s(x, in_placement, out_placement, in_sbp, out_sbp, shape):
    """EagerNaiveSToS"""
    return _rebox(x, out_sbp, out_placement)


def eager_p_to_s(x, in_placement, out_placement, out_sbp, shape):
    """EagerPToS"""
    return _rebox(x, out_sbp, out_placement)


def eager_s_to_p(x, in_placement, out_placement, out_sbp, shape):
    """EagerSToP"""
    return _rebox(x, out_sbp, out_placement)


def global_all_reduce(x):
    """GlobalAllReduce: partial-sum -> broadcast."""
    import oneflow_b200 as flow
    return _rebox(x, [flow.sbp.broadcast] * len(x.sbp))


def global_reduce_scatter(x, op_type="sum"):
    """GlobalReduceScatter: partial-sum -> split(0)."""
    import oneflow_b200 as flow
    return _rebox(x, [flow.sbp.split(0)] * len(x.sbp))


def global_all_gather(x):
    """GlobalAllGather: split -> broadcast."""
    import oneflow_b200 as flow
    return _rebox(x, [flow.sbp.broadcast] * len(x.sbp))


def global_s2s(x, out_sbp):
    """GlobalS2S: split(i) -> split(j) by all-to-all."""
    return _rebox(x, out_sbp)


def distributed_partial_fc_sample_disable_boxing(sampled_weight_diff, sampled_label):
    """DistributedPariticalFCSampleDisableBoxing: hands this rank's sampled gradient rows and labels on unchanged
    (no boxing is inserted between the sample op and the sparse update here)."""
    return sampled_weight_diff, sampled_label


# ------------------------------------------------------------------------------------------------ noncontiguous binary
def noncontiguous_binary_op(lhs, rhs, op="add", inplace=False):
    """NonContiguousBinaryOp: add / sub / mul / div on strided operands without materialising them."""
    fn = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[op]
    if inplace:
        return getattr(lhs, op + "_")(rhs)
    return fn(lhs, rhs)


# ------------------------------------------------------------------------------------------------ OneEmbedding stage ops
from .one_embedding.ops import (one_embedding_adagrad_update, one_embedding_adam_update,  # noqa: E402,F401
                                one_embedding_embedding_gradient_shuffle, one_embedding_embedding_put,
                                one_embedding_embedding_shuffle, one_embedding_ftrl_update, one_embedding_fused_lookup,
                                one_embedding_id_shuffle, one_embedding_lookup, one_embedding_sgd_update,
                                one_embedding_unique_key_value_pair)
