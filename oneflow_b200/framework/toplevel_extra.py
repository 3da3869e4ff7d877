"""Top-level ``flow.*`` names of the reference that PyTorch does not provide under the same name
(reference: python/oneflow/__init__.py and the functional definitions it re-exports)."""
from __future__ import annotations

import os
import types

import numpy as np
import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ shape / dtype sugar
def cast(x, dtype, pin_memory=False):
    return x.to(dtype)


def contiguous(x):
    return x.contiguous()


def expand(x, *sizes):
    return x.expand(*sizes)


def repeat(x, *sizes):
    return x.repeat(*sizes)


def view(x, *shape):
    return x.view(*shape)


def _new_kw(dtype, device, requires_grad, kw):
    out = {k: kw[k] for k in ("placement", "sbp") if kw.get(k) is not None}
    if dtype is not None:
        out["dtype"] = dtype
    if device is not None and "placement" not in out:
        out["device"] = device
    if requires_grad:
        out["requires_grad"] = True
    return out


def new_empty(x, size, dtype=None, device=None, requires_grad=False, **kw):
    return x.new_empty(size, **_new_kw(dtype, device, requires_grad, kw))


def new_full(x, size, fill_value, dtype=None, device=None, requires_grad=False, **kw):
    return x.new_full(size, fill_value, **_new_kw(dtype, device, requires_grad, kw))


def new_ones(x, size=None, dtype=None, device=None, requires_grad=False, **kw):
    return x.new_ones(size if size is not None else x.shape, **_new_kw(dtype, device, requires_grad, kw))


def new_zeros(x, size=None, dtype=None, device=None, requires_grad=False, **kw):
    return x.new_zeros(size if size is not None else x.shape, **_new_kw(dtype, device, requires_grad, kw))


for _f in (new_empty, new_full, new_ones, new_zeros):
    _f.__name__ = _f.__name__ + "_op"        # the names the reference's functions carry (its tests look at them)


def broadcast_like(x, like, broadcast_axes=None):
    if broadcast_axes:
        for a in sorted(broadcast_axes):
            if x.dim() < like.dim():
                x = x.unsqueeze(a)
    return x.expand_as(like)


def slice(x, slice_tup_list):
    """slice_tup_list: [(start, stop, step), ...] per leading dimension (None = full range)."""
    idx = tuple(builtins_slice(*(t if t is not None else (None, None, None))) for t in slice_tup_list)
    return x[idx]


def slice_update(x, update, slice_tup_list):
    idx = tuple(builtins_slice(*(t if t is not None else (None, None, None))) for t in slice_tup_list)
    x[idx] = update
    return x


import builtins as _b  # noqa: E402

builtins_slice = _b.slice


def batch_gather(x, indices):
    """out[b..., i, ...] = x[b..., indices[b..., i], ...]: gather along axis indices.ndim - 1 with leading batch dims."""
    axis = indices.dim() - 1
    idx = indices.long()
    for _ in range(x.dim() - indices.dim()):
        idx = idx.unsqueeze(-1)
    idx = idx.expand(*indices.shape, *x.shape[axis + 1:])
    return torch.gather(x, axis, idx)


def scatter_nd(index, update, shape):
    """Zeros of ``shape`` with ``update`` added at the n-d ``index`` positions."""
    from .._C_more import scatternd
    return scatternd(index, update, shape)


def tensor_scatter_nd_update(tensor, indices, updates):
    from .._C_more import tensor_scatter_nd_update as _f
    return _f(tensor, indices, updates)


def gather_nd(x, index):
    return x[tuple(index.long().unbind(-1))]


def in_top_k(targets, predictions, k):
    top = predictions.topk(min(int(k), predictions.shape[-1]), dim=-1).indices
    return (top == targets.long().unsqueeze(-1)).any(-1)


# ------------------------------------------------------------------------------------------------ activations
def gelu(x, approximate="none"):
    return F.gelu(x, approximate=approximate)


silu = F.silu
mish = F.mish
softplus = F.softplus
softshrink = F.softshrink
softsign = F.softsign
pad = F.pad


def quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


def square_relu(x):
    return torch.relu(x) ** 2


# ------------------------------------------------------------------------------------------------ in-place variants
def div_(x, other):
    return x.div_(other)


def erfinv_(x):
    return x.erfinv_()


def gt_(x, other):
    return x.copy_((x > other).to(x.dtype))


def index_add_(x, dim, index, source, alpha=1):
    return x.index_add_(dim, index, source, alpha=alpha)


def lerp_(x, end, weight):
    return x.lerp_(end, weight)


def masked_fill_(x, mask, value):
    return x.masked_fill_(mask, value)


def normal_(x, mean=0.0, std=1.0, generator=None):
    return x.normal_(mean, std, generator=generator)


# ------------------------------------------------------------------------------------------------ global tensor casts
def global_to_global(x, placement=None, sbp=None, grad_sbp=None, check_meta=True, copy=False):
    return x.to_global(placement=placement, sbp=sbp, grad_sbp=grad_sbp, check_meta=check_meta, copy=copy)


def local_to_global(x, placement=None, sbp=None, shape=None, dtype=None, sync_data=True, copy=False, check_meta=True):
    return x.to_global(placement=placement, sbp=sbp, check_meta=check_meta, copy=copy)


# ------------------------------------------------------------------------------------------------ vision / metrics
def nms(boxes, scores, iou_threshold):
    """Indices of the boxes kept by greedy non-maximum suppression, sorted by decreasing score."""
    order = scores.argsort(descending=True)
    x1, y1, x2, y2 = boxes.unbind(-1)
    areas = (x2 - x1) * (y2 - y1)
    keep = []
    while order.numel():
        i = order[0]
        keep.append(i)
        if order.numel() == 1:
            break
        rest = order[1:]
        w = (torch.min(x2[i], x2[rest]) - torch.max(x1[i], x1[rest])).clamp(min=0)
        h = (torch.min(y2[i], y2[rest]) - torch.max(y1[i], y1[rest])).clamp(min=0)
        inter = w * h
        iou = inter / (areas[i] + areas[rest] - inter)
        order = rest[iou <= iou_threshold]
    return torch.stack(keep) if keep else torch.empty(0, dtype=torch.long, device=boxes.device)


def roi_align(x, rois, spatial_scale, pooled_h, pooled_w, sampling_ratio=-1, aligned=False):
    """RoIAlign with the reference's argument order: ``x`` [N, C, H, W], ``rois`` [K, 5] = (batch index, x1, y1, x2, y2),
    output ``[K, C, pooled_h, pooled_w]`` (reference: functional_api.yaml ``roi_align``)."""
    try:
        from torchvision.ops import roi_align as _tv
    except ImportError:
        return _roi_align_impl(x, rois, (int(pooled_h), int(pooled_w)), float(spatial_scale), int(sampling_ratio), bool(aligned))
    return _tv(x, rois.to(x.dtype), (int(pooled_h), int(pooled_w)), float(spatial_scale), int(sampling_ratio), bool(aligned))


def _roi_align_impl(input, boxes, output_size, spatial_scale=1.0, sampling_ratio=-1, aligned=False):
    """input [N, C, H, W]; boxes [K, 5] = (batch index, x1, y1, x2, y2). Bilinear RoIAlign (average of the samples)."""
    oh, ow = (output_size, output_size) if isinstance(output_size, int) else output_size
    N, C, H, W = input.shape
    out = input.new_zeros((boxes.shape[0], C, oh, ow))
    off = 0.5 if aligned else 0.0
    for k in range(boxes.shape[0]):
        b = int(boxes[k, 0])
        x1, y1, x2, y2 = (boxes[k, 1:] * spatial_scale - off).tolist()
        rw, rh = x2 - x1, y2 - y1
        if not aligned:
            rw, rh = max(rw, 1.0), max(rh, 1.0)
        sr_h = sampling_ratio if sampling_ratio > 0 else max(int(np.ceil(rh / oh)), 1)
        sr_w = sampling_ratio if sampling_ratio > 0 else max(int(np.ceil(rw / ow)), 1)
        ys = y1 + (torch.arange(oh * sr_h, device=input.device, dtype=torch.float32) + 0.5) * rh / (oh * sr_h)
        xs = x1 + (torch.arange(ow * sr_w, device=input.device, dtype=torch.float32) + 0.5) * rw / (ow * sr_w)
        # samples up to one pixel outside the map read the edge value, farther out they count as zero
        vy, vx = ((ys >= -1) & (ys <= H)).float(), ((xs >= -1) & (xs <= W)).float()
        gy = (ys.clamp(0, H - 1) / max(H - 1, 1)) * 2 - 1
        gx = (xs.clamp(0, W - 1) / max(W - 1, 1)) * 2 - 1
        grid = torch.stack(torch.meshgrid(gy, gx, indexing="ij")[::-1], -1).unsqueeze(0)
        samp = F.grid_sample(input[b:b + 1].float(), grid, mode="bilinear", padding_mode="zeros", align_corners=True)
        samp = samp * (vy[:, None] * vx[None, :])
        out[k] = samp.view(C, oh, sr_h, ow, sr_w).mean((2, 4)).to(input.dtype)
    return out


def deform_conv2d(input, offset, weight, bias=None, stride=1, padding=0, dilation=1, mask=None):
    try:
        from torchvision.ops import deform_conv2d as _dc
    except Exception as e:  # pragma: no cover - depends on the image
        raise NotImplementedError("deform_conv2d needs torchvision.ops in this environment") from e
    return _dc(input, offset, weight, bias, stride, padding, dilation, mask)


def roc_auc_score(label, pred):
    """Area under the ROC curve of scores ``pred`` for binary ``label`` (ties get the average rank)."""
    y = label.reshape(-1).float().cpu()
    p = pred.reshape(-1).float().cpu()
    order = p.argsort()
    ranks = torch.empty_like(p)
    sp = p[order]
    n = p.numel()
    r = torch.arange(1, n + 1, dtype=torch.float32)
    # average ranks over ties
    uniq, inv, cnt = torch.unique_consecutive(sp, return_inverse=True, return_counts=True)
    csum = torch.zeros(uniq.numel()).index_add_(0, inv, r)
    ranks[order] = (csum / cnt)[inv]
    pos = y > 0.5
    n_pos, n_neg = int(pos.sum()), int((~pos).sum())
    if n_pos == 0 or n_neg == 0:
        return torch.tensor([float("nan")])
    return ((ranks[pos].sum() - n_pos * (n_pos + 1) / 2) / (n_pos * n_neg)).reshape(1)


# ------------------------------------------------------------------------------------------------ tensor buffers (ragged lists)
class _TensorBufferDType:
    """``flow.tensor_buffer``: the element type of a ragged batch (the reference's ``DataType::kTensorBuffer``)."""

    def __repr__(self):
        return "oneflow.tensor_buffer"


tensor_buffer = _TensorBufferDType()


class TensorBuffer:
    """A batch of variable-shaped tensors (what data-loading ops of the reference pass around)."""
    dtype = tensor_buffer

    def __init__(self, tensors):
        self.tensors = list(tensors)

    @property
    def _tensor_buffer_shapes_and_dtypes(self):
        return [(tuple(t.shape), t.dtype) for t in self.tensors]

    def __len__(self):
        return len(self.tensors)


def tensor_to_tensor_buffer(x, instance_dims):
    lead = x.shape[:x.dim() - instance_dims]
    flat = x.reshape((-1,) + tuple(x.shape[x.dim() - instance_dims:]))
    buf = TensorBuffer(list(flat.unbind(0)))
    buf.batch_shape = tuple(lead)
    return buf


def tensor_buffer_to_list_of_tensors(buf, out_shapes=None, out_dtypes=None, dynamic_out=False):
    out = []
    for i, t in enumerate(buf.tensors):
        if out_dtypes:
            t = t.to(out_dtypes[i] if i < len(out_dtypes) else out_dtypes[-1])
        out.append(t)
    return out


def tensor_buffer_to_tensor(buf, dtype, instance_shape):
    """Stack equally shaped buffer entries into one ``[*batch, *instance_shape]`` tensor."""
    out = torch.stack([t.reshape(tuple(instance_shape)).to(dtype) for t in buf.tensors])
    lead = getattr(buf, "batch_shape", None)
    return out.reshape(tuple(lead) + tuple(instance_shape)) if lead else out


def gen_tensor_buffer(shape, shape_list, value_list, data_type=torch.float32, dynamic_out=False):
    return TensorBuffer([torch.full(tuple(s), v, dtype=data_type) for s, v in zip(shape_list, value_list)])


# ------------------------------------------------------------------------------------------------ dtype helpers / legacy config
def dtypes():
    return [torch.bool, torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64, torch.float16, torch.bfloat16, torch.float32,
            torch.float64, torch.complex64, torch.complex128]


def convert_oneflow_dtype_to_numpy_dtype(dtype):
    return torch.empty((), dtype=dtype if dtype != torch.bfloat16 else torch.float32).numpy().dtype if dtype != torch.bfloat16 else np.dtype("float32")


class FunctionConfig:
    """Legacy job-function configuration object: an attribute bag whose setters are callables (config.foo(value))."""

    def __init__(self):
        object.__setattr__(self, "_values", {})

    def __getattr__(self, name):
        def setter(value=True):
            self._values[name] = value
        return setter


function_config = FunctionConfig
oneflow_python_base_dir = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stub_module(name, doc, **attrs):
    m = types.ModuleType("oneflow." + name, doc)
    for k, v in attrs.items():
        setattr(m, k, v)
    return m


# Internal helper modules of the reference that user code occasionally imports by name.
from .. import asyncs, hub, multiprocessing  # noqa: E402,F401
hook = _stub_module("hook", "Tensor hook helpers.", register_hook=lambda t, fn: t.register_hook(fn))
docstr = _stub_module("docstr", "Docstrings are attached in place in this implementation.")
env_util = _stub_module("env_util", "Environment helpers (see oneflow.env).")
scope_util = _stub_module("scope_util", "Scope helpers of the lazy runtime (not needed here: no scope symbols).")
session_ctx = _stub_module("session_ctx", "Session context (single implicit session).")
register_class_method_util = _stub_module("register_class_method_util", "Tensor methods are registered by framework.tensor_api.")
stateful_op = _stub_module("stateful_op", "Stateful op holder of the reference's eager kernels (kernels here are stateless C entry points).")


from .. import remat  # noqa: E402,F401


from .generator import Generator, default_generator, get_rng_state, set_rng_state  # noqa: E402,F401


def set_default_tensor_type(t):
    """Default floating-point dtype from a typed tensor class or its name (``flow.DoubleTensor``,
    ``"oneflow.FloatTensor"``; reference: python/oneflow/framework/dtype.py)."""
    from .compat_ops import _TYPE_NAMES
    name = t if isinstance(t, str) else getattr(t, "__name__", str(t))
    short = name.split(".")[-1]
    for dt, n in _TYPE_NAMES.items():
        if n == short:
            if not dt.is_floating_point:
                raise TypeError("only floating-point types are supported as the default type")
            return torch.set_default_dtype(dt)
    raise TypeError(f"invalid type object: {name}")


def distributed_partial_fc_sample(weight, label, num_sample):
    """Deprecated function form of ``nn.DistributedPariticalFCSample``."""
    from ..nn.modules.partial_fc import distributed_partial_fc_sample as _f
    return _f(weight, label, num_sample)
