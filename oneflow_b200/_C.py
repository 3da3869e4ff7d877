"""``flow._C``: the functional ops of the reference that have no torch spelling — the fused ops named in
oneflow/core/functional/functional_api.yaml (:1254 fused_bias_add_gelu, :1549 fused_scale_tril_softmax_mask_scale,
:2651-2703 attention, :2815 fused_dot_feature_interaction, fused_mlp) — with autograd. bf16 CUDA tensors
run the hand-written sm_100a kernels; other inputs take the PyTorch statement of the same maths. Anything
else resolves to the torch function of the same name."""
from __future__ import annotations

import math

import torch

from .framework.generator import resolve as _resolve_gen

from .framework.global_tensor import to_global, to_local  # noqa: F401
from .ops import gemm as G
from .ops import kernels as K


def _native_ok(*ts):
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts) and ts[0].shape[-1] % 8 == 0


class _BiasAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act):
        ctx.save_for_backward(x, bias)
        ctx.act = act
        return K.bias_act_fwd(x.contiguous(), bias, act)

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        dx = K.bias_act_bwd(x.contiguous(), bias, dy.contiguous(), ctx.act)
        db = K.column_sum(dx.reshape(-1, dx.shape[-1])).to(bias.dtype) if bias is not None else None
        return dx, db, None


def fused_bias_add_gelu(x, bias, *, axis=-1):
    """gelu(x + bias) with bias broadcast along ``axis`` (last axis for the kernel path)."""
    if _native_ok(x, bias) and (axis in (-1, x.dim() - 1)):
        return _BiasAct.apply(x, bias, G.ACT_GELU)
    shape = [1] * x.dim()
    shape[axis] = -1
    return torch.nn.functional.gelu(x + bias.reshape(shape))


def fused_bias_add_dropout(x, bias, *, p=0.5, axis=-1, generator=None, training=True):
    """dropout(x + bias, p)."""
    shape = [1] * x.dim()
    shape[axis] = -1
    return torch.nn.functional.dropout(x + bias.reshape(shape), p, training)


def fused_bias_add_mask_scale(x, bias, mask, scale, addend=None, *, axis=-1):
    return K.bias_mask_scale(x.contiguous(), bias, mask, scale, addend) if _native_ok(x, bias) and not x.requires_grad \
        else ((x + bias) * mask.to(x.dtype) * scale + (addend if addend is not None else 0))


class _TrilSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, diagonal, tril_scale, mask_scale):
        y, sm = K.softmax_fwd(x.contiguous(), scale=tril_scale, tril=True, diagonal=diagonal, dropout_mask=mask,
                              dropout_scale=mask_scale, want_softmax=True)
        ctx.save_for_backward(sm, mask)
        ctx.args = (diagonal, tril_scale, mask_scale)
        return y, sm

    @staticmethod
    def backward(ctx, dy, _dsm):
        sm, mask = ctx.saved_tensors
        diagonal, tril_scale, mask_scale = ctx.args
        dx = K.softmax_bwd(sm, dy.contiguous(), scale=tril_scale, tril=True, diagonal=diagonal, dropout_mask=mask,
                           dropout_scale=mask_scale)
        return dx, None, None, None, None


def fused_scale_tril_softmax_mask_scale(x, mask=None, *, p=None, diagonal=0, tril_scale_value=1.0, mask_scale_value=None,
                                        tril_fill_value=0.0, generator=None):
    """``(dropout_mask * softmax(tril(x * tril_scale)) * mask_scale, softmax_y)`` over ``[.., s_q, s_k]`` scores.
    Either a ready ``mask`` with its ``mask_scale_value`` is given, or a dropout probability ``p`` from which the mask
    is drawn and the scale ``1 / (1 - p)`` follows (the reference's signature). Scores above the diagonal are set to
    ``tril_fill_value`` before the softmax (0 by default, as in the reference; language models pass -10000 or -inf)."""
    if mask is None and p is not None and p >= 1:
        mask, mask_scale_value = torch.zeros(x.shape, dtype=torch.bool, device=x.device), 0.0
    elif mask is None and p is not None and p > 0:
        generator = _resolve_gen(generator, x.device)
        gen_dev = generator.device if generator is not None else x.device
        mask = (torch.rand(x.shape, device=gen_dev, generator=generator) >= p).to(x.device)
        mask_scale_value = 1.0 / (1.0 - p)
    if mask_scale_value is None:
        mask_scale_value = 1.0
    if mask is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 2048 \
            and tril_fill_value <= -1e4:           # the kernel drops the masked scores outright
        return _TrilSoftmax.apply(x, mask, diagonal, tril_scale_value, mask_scale_value)
    s_q, s_k = x.shape[-2:]
    keep = torch.ones(s_q, s_k, dtype=torch.bool, device=x.device).tril(diagonal)
    sm = torch.softmax((x * tril_scale_value).masked_fill(~keep, tril_fill_value), -1)
    y = sm * (mask.to(x.dtype) if mask is not None else 1.0) * mask_scale_value
    return y, sm


def fused_scale_mask_softmax(x, mask, fill_value=-10000.0, scale=1.0):
    """softmax(masked_fill(x * scale, mask == 0, fill_value))."""
    if x.is_cuda and x.dtype == torch.bfloat16 and not x.requires_grad and x.shape[-1] % 8 == 0 and x.shape[-1] <= 2048 \
            and mask.numel() % x.shape[-1] == 0 and (x.numel() // x.shape[-1]) % (mask.numel() // x.shape[-1]) == 0:
        return K.softmax_fwd(x.contiguous(), scale=scale, attn_mask=mask, mask_fill=fill_value)
    return torch.softmax((x * scale).masked_fill(~mask.bool(), fill_value), -1)


def fused_scale_mask_softmax_dropout(x, mask, dropout_mask=None, *, fill_value=0.0, scale=1.0, p=0.5, training=True, generator=None):
    """``(dropout(softmax(masked_fill(x * scale, mask == 0, fill_value))), softmax_y)``.  The dropout mask is drawn here
    (``p``, ``training``, ``generator``) unless a ready ``dropout_mask`` is passed."""
    sm = fused_scale_mask_softmax(x, mask, fill_value, scale)
    if dropout_mask is None:
        if not training or p == 0:
            return sm, sm
        if p >= 1:
            return sm * 0.0, sm                    # everything is dropped; no 1 / (1 - p) to form
        generator = _resolve_gen(generator, x.device)
        gen_dev = generator.device if generator is not None else x.device
        dropout_mask = (torch.rand(sm.shape, device=gen_dev, generator=generator) >= p).to(x.device)
    return sm * dropout_mask.to(x.dtype) * (1.0 / (1.0 - p)), sm


class _Fmha(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, dropout_p=0.0, seed=0, offset=0):
        out, lse = K.fmha_fwd(q, k, v, causal=causal, scale=scale, dropout_p=dropout_p, seed=seed, offset=offset)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale, ctx.drop = causal, scale, (dropout_p, seed, offset)
        return out

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, out, lse = ctx.saved_tensors
        p, seed, offset = ctx.drop
        dq, dk, dv = K.fmha_bwd(q, k, v, out, d_o.contiguous(), lse, causal=ctx.causal, scale=ctx.scale, dropout_p=p, seed=seed,
                                offset=offset)
        return dq, dk, dv, None, None, None, None, None


def _bshd_ok(t):
    B, S, H, D = t.shape
    return t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == S * t.stride(1) and t.data_ptr() % 16 == 0


_DROPOUT_CALLS = [0]


def _dropout_stream(generator, device):
    """(seed, offset) of the next attention dropout: the seed of the generator in charge, and a call counter so that two
    calls never share a mask."""
    generator = _resolve_gen(generator, device)
    seed = generator.initial_seed() if generator is not None else torch.initial_seed()
    _DROPOUT_CALLS[0] += 1
    return seed, _DROPOUT_CALLS[0]


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, generator=None):
    """query: [B, H, Sq, D], key / value: [B, Hk, Sk, D] (torch convention; Hk divides H for grouped-query attention).
    With ``is_causal`` and Sq != Sk the diagonal is aligned to the bottom-right corner, as in the flash-attention
    library the reference calls (oneflow/user/kernels/scaled_dot_product_attention_kernel.cu:54-138). The fused tcgen05
    kernel serves bf16 CUDA inputs with head dim 64/128 and no explicit mask, dropout (Philox, regenerated in backward)
    included."""
    D = query.shape[-1]
    H, Hk = query.shape[1], key.shape[1]
    Sq, Sk = query.shape[-2], key.shape[-2]
    if (query.is_cuda and query.dtype == torch.bfloat16 and D in (64, 128) and attn_mask is None and 0.0 <= dropout_p < 1.0
            and key.shape == value.shape and key.dtype == value.dtype == torch.bfloat16 and H % Hk == 0 and query.shape[0] == key.shape[0]):
        q, k, v = (t.transpose(1, 2) for t in (query, key, value))  # [B, S, H, D] views
        if not all(_bshd_ok(t) for t in (q, k, v)) or k.stride(1) != v.stride(1):
            q, k, v = (t.contiguous() for t in (q, k, v))
        sc = scale if scale is not None else 1.0 / math.sqrt(D)
        seed, offset = _dropout_stream(generator, query.device) if dropout_p > 0.0 else (0, 0)
        return _Fmha.apply(q, k, v, bool(is_causal), sc, float(dropout_p), seed, offset).transpose(1, 2)
    if Hk != H and H % Hk == 0:
        key, value = (t.repeat_interleave(H // Hk, dim=1) for t in (key, value))
    if is_causal and Sq != Sk and attn_mask is None:
        attn_mask = torch.ones(Sq, Sk, dtype=torch.bool, device=query.device).tril(Sk - Sq)
        is_causal = False
    return torch.nn.functional.scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal, scale=scale)


def fused_multi_head_attention_inference(query, key, value, num_heads, causal=False, query_hidden_slice_start=0,
                                         query_hidden_slice_end=-1, key_hidden_slice_start=0, key_hidden_slice_end=-1,
                                         value_hidden_slice_start=0, value_hidden_slice_end=-1, attn_bias=None,
                                         causal_diagonal_offset=0):
    """query/key/value: [B, S, hidden(_slices)] packed layouts (BM(HK)); returns [B, S, H*D]."""
    def sl(t, a, b):
        return t[..., a:(t.shape[-1] if b == -1 else b)]
    q = sl(query, query_hidden_slice_start, query_hidden_slice_end)
    k = sl(key, key_hidden_slice_start, key_hidden_slice_end)
    v = sl(value, value_hidden_slice_start, value_hidden_slice_end)
    B, S, HD = q.shape
    D = HD // num_heads
    q4, k4, v4 = (t.reshape(B, t.shape[1], num_heads, D) for t in (q, k, v))
    if (q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and attn_bias is None and causal_diagonal_offset == 0
            and (k.shape[1] == S or not causal) and k4.stride(1) == v4.stride(1) and all(_bshd_ok(t) for t in (q4, k4, v4))):
        with torch.no_grad():
            out, _ = K.fmha_fwd(q4, k4, v4, causal=causal)
        return out.reshape(B, S, HD)
    o = torch.nn.functional.scaled_dot_product_attention(q4.transpose(1, 2), k4.transpose(1, 2), v4.transpose(1, 2),
                                                         attn_mask=attn_bias, is_causal=causal and attn_bias is None)
    return o.transpose(1, 2).reshape(B, S, HD)


def fused_multi_head_attention_inference_v2(*, query, query_layout="BM(HK)", query_head_size=None, key=None,
                                            key_layout=None, value=None, value_layout=None, attn_bias=None,
                                            output_layout="BM(HK)", causal=False, scale=None, **unused):
    H = query.shape[-1] // query_head_size
    return fused_multi_head_attention_inference(query, key, value, H, causal=causal, attn_bias=attn_bias)


def fused_mlp(x, weights, biases, skip_final_activation=False):
    """Linear + ReLU layers as fused GEMMs (bias and ReLU in the epilogue; in backward every layer folds the previous
    layer's ReLU gradient into its data-gradient GEMM); local and global tensors (framework/fused_ops.mlp_chain)."""
    from .framework import fused_ops
    return fused_ops.mlp_chain(x, list(weights), list(biases), act="relu", skip_final_activation=skip_final_activation)


def fused_matmul_bias(x, weight, bias, _add_to_output=None, alpha=1.0, beta=1.0):
    """``alpha * (x @ weight^T + bias) + beta * _add_to_output``: one GEMM with the bias and the addend in its epilogue
    (for alpha = beta = 1), global tensors included (framework/fused_ops.linear)."""
    from .framework import fused_ops
    if alpha == 1.0 and beta == 1.0:
        return fused_ops.linear(x, weight, bias, residual=_add_to_output)
    y = fused_ops.linear(x, weight, bias)
    return y * alpha if _add_to_output is None else y * alpha + _add_to_output * beta


def fused_attention_qkv_packed(qkv, *, seq_len, head_size, causal=True, scale=None):
    from .framework import fused_ops
    return fused_ops.fused_attention_qkv_packed(qkv, seq_len=seq_len, head_size=head_size, causal=causal, scale=scale)


def fused_dot_feature_interaction(features, output_concat=None, self_interaction=False, output_padding=0, pooling="none"):
    from .ops.interaction import dot_feature_interaction
    return dot_feature_interaction(features, output_concat, self_interaction, output_padding, pooling)


def layer_norm(x, normalized_shape=None, weight=None, bias=None, eps=1e-5, *, begin_norm_axis=None, begin_params_axis=None,
               epsilon=None):
    """Layer norm, either torch-style (``normalized_shape``) or with the reference's ``begin_norm_axis`` /
    ``begin_params_axis`` / ``epsilon`` (normalise over the axes from ``begin_norm_axis`` on, no affine)."""
    if begin_norm_axis is not None or isinstance(normalized_shape, int):
        axis = begin_norm_axis if begin_norm_axis is not None else normalized_shape
        e = epsilon if epsilon is not None else (weight if isinstance(weight, float) else eps)
        return torch.nn.functional.layer_norm(x, tuple(x.shape[axis:]), None, None, e)
    return torch.nn.functional.layer_norm(x, normalized_shape, weight, bias, epsilon if epsilon is not None else eps)


def local_all_reduce(x, inplace=False):
    from . import comm
    t = x if inplace else x.clone()
    return comm.all_reduce(t)


from ._C_extra import *  # noqa: F401,F403,E402  (the long tail of fused functions)
from ._C_more import *  # noqa: F401,F403,E402
from ._C_more import T, _fused_gru_cell, _fused_lstm_cell  # noqa: F401,E402


def __getattr__(name):
    """Ops not defined here: the function of that name of the top-level package, of ``flow.nn.functional``, of torch."""
    import sys
    if name.startswith("__"):
        raise AttributeError(name)
    top = sys.modules.get("oneflow_b200")
    if top is not None and name in top.__dict__ and callable(top.__dict__[name]):
        return top.__dict__[name]
    fn = sys.modules.get("oneflow_b200.nn.functional")
    if fn is not None and name in fn.__dict__:
        return fn.__dict__[name]
    if hasattr(torch, name):
        return getattr(torch, name)
    if hasattr(torch.nn.functional, name):
        return getattr(torch.nn.functional, name)
    raise AttributeError(f"flow._C has no op {name!r}")
