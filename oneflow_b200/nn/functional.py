"""``flow.nn.functional``: torch.nn.functional plus the fused ops of ``flow._C``."""
from torch.nn.functional import *  # noqa: F401,F403
import torch.nn.functional as _F

from .._C import (fused_bias_add_dropout, fused_bias_add_gelu, fused_scale_mask_softmax,  # noqa: F401
                  fused_scale_mask_softmax_dropout, fused_scale_tril_softmax_mask_scale)


def __getattr__(name):
    return getattr(_F, name)


def linear(input, weight, bias=None):
    """``input @ weight^T + bias``: the tcgen05 GEMM for bf16 CUDA tensors, SBP-aware (fused tensor-parallel products)
    for global tensors, torch's op otherwise."""
    from ..framework import fused_ops
    return fused_ops.linear(input, weight, bias)


def mlp(input, weight1, bias1, weight2, bias2, act="gelu", residual=None):
    """``linear(act(linear(input, weight1, bias1)), weight2, bias2) + residual`` as one unit (the hidden activation is
    private to the call, so its gradient is folded into a GEMM epilogue in backward); SBP-aware like ``linear``."""
    from ..framework import fused_ops
    return fused_ops.mlp(input, weight1, bias1, weight2, bias2, act=act, residual=residual)


def layer_norm(input, normalized_shape, weight=None, bias=None, eps=1e-5):
    from ..framework import fused_ops
    return fused_ops.layer_norm(input, normalized_shape, weight, bias, eps)


def embedding(input, weight, padding_idx=None, max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False):
    if padding_idx is not None or max_norm is not None or scale_grad_by_freq or sparse:
        return _F.embedding(input, weight, padding_idx, max_norm, norm_type, scale_grad_by_freq, sparse)
    from ..framework import fused_ops
    return fused_ops.embedding(input, weight)


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, generator=None):
    """Fused attention (tcgen05 kernels for bf16 CUDA inputs: grouped-query heads, Sq != Sk, Philox dropout), torch's op
    otherwise. Global tensors go through torch's op and its SBP rule."""
    from ..framework import global_tensor as _GT
    if any(isinstance(t, _GT.GlobalTensor) for t in (query, key, value)):
        return _F.scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal, scale=scale)
    from .. import _C
    return _C.scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal, scale, generator)


def conv2d(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """torch's conv2d, or the implicit-GEMM tcgen05 kernels for bf16 channels-last stride-1 "same" convolutions."""
    from .modules.conv import conv2d as _conv2d
    return _conv2d(input, weight, bias, stride, padding, dilation, groups)


# ------------------------------------------------------------------------------------------------ reference-only functions
import torch as _torch  # noqa: E402


def quick_gelu(x):
    """``x * sigmoid(1.702 * x)`` (reference: oneflow/core/functional/impl/activation_functor.cpp, QuickGelu)."""
    return x * _torch.sigmoid(1.702 * x)


def square_relu(x):
    """``relu(x) ** 2`` (reference: oneflow/core/functional/impl/activation_functor.cpp, SquareReLU)."""
    return _torch.square(_torch.relu(x))


def sparse_softmax_cross_entropy(labels, logits):
    """Per-element cross entropy of integer ``labels`` against ``logits`` over the last axis, no reduction
    (reference: python/oneflow/nn/modules/sparse_softmax_cross_entropy.py:19-70). 2-D bf16 CUDA logits and global
    logits (the class axis may be split: vocabulary parallel) run the fused kernels and return fp32."""
    from ..framework import fused_ops, global_tensor as _GT
    if logits.dim() == 2 and (isinstance(logits, _GT.GlobalTensor) or (logits.is_cuda and logits.dtype == _torch.bfloat16)):
        return fused_ops.sparse_softmax_cross_entropy(logits, labels)
    nc = logits.shape[-1]
    loss = _F.cross_entropy(logits.reshape(-1, nc).float(), labels.reshape(-1).long(), reduction="none")
    return loss.reshape(labels.shape).to(logits.dtype)


def depend(input, depend):
    """Identity on ``input`` that also depends on ``depend`` (one tensor or a list): anything that produced ``depend``
    is ordered before the consumers of the result and receives a zero gradient through it
    (reference: python/oneflow/nn/functional/depend.py:22-78)."""
    deps = [depend] if isinstance(depend, _torch.Tensor) else list(depend)
    return _Depend.apply(input, *deps)


class _Depend(_torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, *deps):
        ctx.meta = [(d.shape, d.dtype, d.device) if d.requires_grad else None for d in deps]
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return (g,) + tuple(None if m is None else _torch.zeros(m[0], dtype=m[1], device=m[2]) for m in ctx.meta)


def interpolate_like(input, like, mode="nearest", align_corners=None):
    """``interpolate`` to the spatial size of ``like`` (reference: python/oneflow/nn/modules/interpolate.py:313-370)."""
    return _F.interpolate(input, size=tuple(like.shape[2:]), mode=mode, align_corners=align_corners)


def ctc_greedy_decoder(log_probs, input_lengths, merge_repeated=True):
    """Best-path CTC decoding.  ``log_probs`` [T, B, C] with the blank as class C-1, ``input_lengths`` [B].
    Returns ``decoded`` int64 [B, T] (left-packed, zero padded) and ``neg_sum_logits`` [B, 1], minus the sum of the
    largest log-probability of every valid frame (reference: oneflow/user/kernels/ctc_greedy_decoder.cpp:27-52).
    Vectorised: an emit mask, then a stable left-pack by cumulative count."""
    T, B, C = log_probs.shape
    best, idx = log_probs.max(dim=2)                                   # [T, B]
    t = _torch.arange(T, device=log_probs.device)[:, None]
    valid = t < input_lengths.to(log_probs.device)[None, :]
    neg_sum = -(best * valid).sum(0).reshape(B, 1)
    prev = _torch.cat([_torch.full_like(idx[:1], -1), idx[:-1]], 0)
    emit = valid & (idx != C - 1)
    if merge_repeated:
        emit = emit & (idx != prev)
    pos = emit.long().cumsum(0) - 1                                    # slot of every emitted frame
    decoded = _torch.zeros((B, T + 1), dtype=_torch.int64, device=log_probs.device)
    slot = _torch.where(emit, pos, _torch.full_like(pos, T))          # non-emitted frames go to a spill column
    decoded.scatter_(1, slot.t(), (idx * emit).t())
    return decoded[:, :T].contiguous(), neg_sum


def deform_conv2d(input, offset, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), mask=None):
    """Deformable convolution v1 (``mask is None``) / v2.  ``offset`` [N, 2*G*kh*kw, Ho, Wo] holds (dy, dx) per
    offset group and kernel tap, ``mask`` [N, G*kh*kw, Ho, Wo] the modulation
    (reference: python/oneflow/nn/functional/deform_conv.py:22-122, user/kernels/deform_conv_kernel.cu).
    Sampling is bilinear with zeros outside the image; the sampled columns then meet the weights in one batched GEMM."""
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)  # noqa: E731
    (sh, sw), (ph, pw), (dh, dw) = pair(stride), pair(padding), pair(dilation)
    if input.dim() != 4 or weight.dim() != 4 or offset.dim() != 4 or (mask is not None and mask.dim() != 4):
        raise RuntimeError("deform_conv2d expects 4-D input, weight, offset and mask")
    N, Cin, H, W = input.shape
    Cout, Cg, kh, kw = weight.shape
    K = kh * kw
    og = offset.shape[1] // (2 * K)
    if og == 0 or offset.shape[1] != 2 * og * K:
        raise RuntimeError(f"offset.shape[1]={offset.shape[1]} is not a multiple of 2 * kh * kw = {2 * K}")
    groups = Cin // Cg
    Ho = (H + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    Wo = (W + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    dev, ft = input.device, _torch.float32
    base_y = (_torch.arange(Ho, device=dev, dtype=ft) * sh - ph)[None, :, None] + \
        (_torch.arange(kh, device=dev, dtype=ft) * dh).repeat_interleave(kw)[:, None, None]          # [K, Ho, 1]
    base_x = (_torch.arange(Wo, device=dev, dtype=ft) * sw - pw)[None, None, :] + \
        (_torch.arange(kw, device=dev, dtype=ft) * dw).repeat(kh)[:, None, None]                     # [K, 1, Wo]
    off = offset.float().reshape(N, og, K, 2, Ho, Wo)
    y = off[:, :, :, 0] + base_y                                                                      # [N, og, K, Ho, Wo]
    x = off[:, :, :, 1] + base_x
    grid = _torch.stack([2 * x / max(W - 1, 1) - 1, 2 * y / max(H - 1, 1) - 1], -1).reshape(N * og, K * Ho, Wo, 2)
    cols = _F.grid_sample(input.float().reshape(N * og, Cin // og, H, W), grid, mode="bilinear", padding_mode="zeros",
                          align_corners=True).reshape(N, og, Cin // og, K, Ho, Wo)
    if mask is not None:
        cols = cols * mask.float().reshape(N, og, 1, K, Ho, Wo)
    cols = cols.reshape(N, groups, Cg * K, Ho * Wo)
    w = weight.float().reshape(groups, Cout // groups, Cg * K)
    out = _torch.einsum("gok,ngkl->ngol", w, cols).reshape(N, Cout, Ho, Wo)
    if bias is not None:
        out = out + bias.float().reshape(1, -1, 1, 1)
    return out.to(input.dtype)


def batch_norm(input, running_mean, running_var, weight=None, bias=None, training=False, momentum=0.1, eps=1e-5):
    """``batch_norm``; 4-D inputs are read as [N, H, W, C] while ``ONEFLOW_ENABLE_NHWC=1``
    (reference: python/oneflow/nn/functional/batch_norm.py:38-45)."""
    import os
    if input.dim() == 4 and os.getenv("ONEFLOW_ENABLE_NHWC") == "1":
        return _F.batch_norm(input.permute(0, 3, 1, 2), running_mean, running_var, weight, bias, training, momentum,
                             eps).permute(0, 2, 3, 1)
    return _F.batch_norm(input, running_mean, running_var, weight, bias, training, momentum, eps)
