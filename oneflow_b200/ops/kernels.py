"""Python faces of the hand-written CUDA kernels (LayerNorm, fused bias/activation/dropout,
softmax family, cross-entropy, attention, optimizer updates).

Each function has two bodies: the native sm_100a kernel for CUDA tensors and a plain PyTorch
fp32 statement of the same maths for CPU tensors (which is also what the tests compare the
kernels against). A CUDA tensor never falls back to PyTorch ops: if the kernel library is
missing the call raises.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from . import _native
from ._native import check, ptr, stream_ptr

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
launch_count = 0  # number of native kernel-launching calls issued through this module (bench bookkeeping)


def _lib():
    return _native.kernels()


def _count(n=1):
    global launch_count
    launch_count += n


def _need_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"expected bfloat16, got {t.dtype}")
        if t is not None and not t.is_contiguous():
            raise ValueError("expected a contiguous tensor")
        if t is not None and t.data_ptr() % 16:
            raise ValueError("expected a 16-byte aligned tensor")


# ------------------------------------------------------------------------------------------------
# LayerNorm
# ------------------------------------------------------------------------------------------------
def layer_norm_fwd(x, gamma, beta, eps=1e-5):
    """x [rows, cols] bf16 -> (y bf16, mean fp32 [rows], rstd fp32 [rows])."""
    rows, cols = x.shape
    if not x.is_cuda:
        xf = x.float()
        mean = xf.mean(-1)
        var = xf.var(-1, unbiased=False)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean[:, None]) * rstd[:, None]
        if gamma is not None:
            y = y * gamma.float()
        if beta is not None:
            y = y + beta.float()
        return y.to(x.dtype), mean, rstd
    _need_bf16(x, gamma, beta)
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(_lib().ofb_layer_norm_fwd(ptr(x), ptr(gamma), ptr(beta), ptr(y), ptr(mean), ptr(rstd), c_int(rows), c_int(cols),
                                    c_float(eps), stream_ptr()), "layer_norm_fwd")
    _count()
    return y, mean, rstd


def layer_norm_bwd(dy, x, gamma, mean, rstd, add_to_dx=None, dgamma=None, dbeta=None, want_param_grads=True):
    """Returns (dx bf16, dgamma fp32, dbeta fp32). When dgamma/dbeta buffers are given the parameter
    gradients are accumulated into them."""
    rows, cols = x.shape
    if (dgamma is None) != (dbeta is None):
        raise ValueError("layer_norm_bwd: dgamma and dbeta must be given together or not at all")
    if not x.is_cuda:
        xf, dyf = x.float(), dy.float()
        xh = (xf - mean[:, None]) * rstd[:, None]
        g = dyf * (gamma.float() if gamma is not None else 1.0)
        dx = rstd[:, None] * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True))
        if add_to_dx is not None:
            dx = dx + add_to_dx.float()
        dg = (dyf * xh).sum(0)
        db = dyf.sum(0)
        if dgamma is not None:
            dgamma += dg
            dbeta += db
            dg, db = dgamma, dbeta
        return dx.to(x.dtype), dg, db
    _need_bf16(dy, x, gamma, add_to_dx)
    dx = torch.empty_like(x)
    accumulate = dgamma is not None
    scratch = None
    if want_param_grads:
        if dgamma is None:
            dgamma = torch.empty(cols, dtype=torch.float32, device=x.device)
            dbeta = torch.empty(cols, dtype=torch.float32, device=x.device)
        parts = _lib().ofb_layer_norm_bwd_parts(c_int(rows))
        scratch = torch.empty(2 * parts * cols, dtype=torch.float32, device=x.device)
    check(_lib().ofb_layer_norm_bwd(ptr(dy), ptr(x), ptr(gamma), ptr(mean), ptr(rstd), ptr(add_to_dx), ptr(dx),
                                    ptr(dgamma if want_param_grads else None), ptr(dbeta if want_param_grads else None),
                                    ptr(scratch), c_int(int(accumulate)), c_int(rows), c_int(cols), stream_ptr()),
          "layer_norm_bwd")
    _count(2 if want_param_grads else 1)
    return dx, dgamma, dbeta


# ------------------------------------------------------------------------------------------------
# bias + activation, bias + dropout
# ------------------------------------------------------------------------------------------------
def _act_ref(v, act):
    from .gemm import _act_ref as f
    return f(v, act)


def bias_act_fwd(x, bias, act):
    """act(x + bias) with act in {0 none, 1 gelu, 2 gelu_tanh, 3 relu}; bias broadcast over the last dim."""
    if not x.is_cuda:
        v = x.float() + (bias.float() if bias is not None else 0.0)
        return _act_ref(v, act).to(x.dtype)
    _need_bf16(x, bias)
    y = torch.empty_like(x)
    check(_lib().ofb_bias_act_fwd(ptr(x), ptr(bias), ptr(y), c_longlong(x.numel()), c_int(x.shape[-1]), c_int(act),
                                  stream_ptr()), "bias_act_fwd")
    _count()
    return y


def bias_act_bwd(x, bias, dy, act):
    """dy * act'(x + bias)."""
    if not x.is_cuda:
        from .gemm import _act_grad_ref
        v = x.float() + (bias.float() if bias is not None else 0.0)
        return (dy.float() * _act_grad_ref(v, act)).to(x.dtype)
    _need_bf16(x, bias, dy)
    dx = torch.empty_like(x)
    check(_lib().ofb_bias_act_bwd(ptr(x), ptr(bias), ptr(dy), ptr(dx), c_longlong(x.numel()), c_int(x.shape[-1]),
                                  c_int(act), stream_ptr()), "bias_act_bwd")
    _count()
    return dx


def bias_mask_scale(x, bias, mask, scale, addend=None):
    """mask * (x + bias) * scale (+ addend); mask is a uint8/bool keep-mask or None."""
    if not x.is_cuda:
        v = x.float() + (bias.float() if bias is not None else 0.0)
        if mask is not None:
            v = v * mask.float()
        v = v * scale
        if addend is not None:
            v = v + addend.float()
        return v.to(x.dtype)
    _need_bf16(x, bias, addend)
    if mask is not None:
        mask = mask.view(torch.uint8) if mask.dtype == torch.bool else mask
        if mask.dtype != torch.uint8 or not mask.is_contiguous():
            raise TypeError("mask must be a contiguous uint8/bool tensor")
    y = torch.empty_like(x)
    check(_lib().ofb_bias_mask_scale(ptr(x), ptr(bias), ptr(mask), ptr(addend), ptr(y), c_longlong(x.numel()),
                                     c_int(x.shape[-1]), c_float(scale), stream_ptr()), "bias_mask_scale")
    _count()
    return y


def dropout_mask(shape, p, seed, offset=0, device="cuda"):
    """uint8 keep-mask with P(keep) = 1 - p from a counter-based generator (deterministic in seed/offset)."""
    n = int(math.prod(shape))
    if torch.device(device).type != "cuda":
        g = torch.Generator().manual_seed(int(seed) + int(offset))
        return (torch.rand(shape, generator=g) >= p).to(torch.uint8)
    mask = torch.empty(shape, dtype=torch.uint8, device=device)
    check(_lib().ofb_dropout_mask(ptr(mask), c_longlong(n), c_ulonglong(seed), c_ulonglong(offset), c_float(p),
                                  stream_ptr()), "dropout_mask")
    _count()
    return mask


def cast_scale(x, scale=1.0, out_dtype=torch.float32, scale_by_tensor=None, out=None):
    """cast(x) * scale * scale_by_tensor (fused_cast_scale)."""
    if not x.is_cuda:
        v = x.float() * scale
        if scale_by_tensor is not None:
            v = v * scale_by_tensor.float()
        r = v.to(out_dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    x = x.contiguous()
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(_lib().ofb_cast_scale(ptr(x), c_int(_DT[x.dtype]), ptr(out), c_int(_DT[out.dtype]), c_longlong(x.numel()),
                                c_float(scale), ptr(scale_by_tensor), stream_ptr()), "cast_scale")
    _count()
    return out


def column_sum(x, out=None):
    """fp32 sum over rows of a bf16 [rows, cols] matrix (bias gradient); accumulates into `out` if given."""
    rows, cols = x.shape
    if not x.is_cuda:
        r = x.float().sum(0)
        if out is not None:
            out += r
            return out
        return r
    _need_bf16(x)
    if out is None:
        out = torch.zeros(cols, dtype=torch.float32, device=x.device)
    check(_lib().ofb_column_sum(ptr(x), ptr(out), c_int(rows), c_int(cols), stream_ptr()), "column_sum")
    _count()
    return out


# ------------------------------------------------------------------------------------------------
# softmax family
# ------------------------------------------------------------------------------------------------
def softmax_fwd(x, *, scale=1.0, tril=False, diagonal=0, attn_mask=None, mask_fill=-10000.0, dropout_mask=None,
                dropout_scale=1.0, want_softmax=False):
    """y = dropout_mask * softmax(mask(x * scale)) * dropout_scale over the last dim.

    tril: rows are laid out [..., s_q, s_k]; row r keeps columns <= r + diagonal.
    attn_mask: uint8 [mask_rows, cols], 0 = masked (filled with mask_fill), broadcast by row % mask_rows.
    Returns y or (y, softmax_y).
    """
    cols = x.shape[-1]
    rows = x.numel() // cols
    tril_rows = x.shape[-2] if x.dim() >= 2 else 1
    if not x.is_cuda:
        v = x.float() * scale
        if attn_mask is not None:
            am = attn_mask.reshape(-1, cols).bool()
            idx = torch.arange(rows) % am.shape[0]
            v = v.reshape(rows, cols).masked_fill(~am[idx], mask_fill).reshape(x.shape)
        if tril:
            r = torch.arange(tril_rows)[:, None]
            c = torch.arange(cols)[None, :]
            v = v.masked_fill(c > r + diagonal, float("-inf"))
        sm = torch.softmax(v, -1)
        y = sm
        if dropout_mask is not None:
            y = y * dropout_mask.float()
        y = (y * dropout_scale).to(x.dtype)
        return (y, sm.to(x.dtype)) if want_softmax else y
    _need_bf16(x)
    y = torch.empty_like(x)
    sm = torch.empty_like(x) if want_softmax else None
    if dropout_mask is not None and dropout_mask.dtype == torch.bool:
        dropout_mask = dropout_mask.view(torch.uint8)
    am_rows = 0
    if attn_mask is not None:
        attn_mask = attn_mask.view(torch.uint8) if attn_mask.dtype == torch.bool else attn_mask
        attn_mask = attn_mask.reshape(-1, cols).contiguous()
        am_rows = attn_mask.shape[0]
    check(_lib().ofb_softmax_fwd(ptr(x), ptr(dropout_mask), ptr(attn_mask), c_longlong(am_rows), ptr(y), ptr(sm),
                                 c_longlong(rows), c_int(cols), c_int(int(tril)), c_int(tril_rows), c_int(diagonal),
                                 c_float(scale), c_float(mask_fill), c_float(dropout_scale), stream_ptr()),
          "softmax_fwd")
    _count()
    return (y, sm) if want_softmax else y


def softmax_bwd(softmax_y, dy, *, scale=1.0, tril=False, diagonal=0, dropout_mask=None, dropout_scale=1.0):
    cols = dy.shape[-1]
    rows = dy.numel() // cols
    tril_rows = dy.shape[-2] if dy.dim() >= 2 else 1
    if not dy.is_cuda:
        y = softmax_y.float()
        g = dy.float()
        if dropout_mask is not None:
            g = g * dropout_mask.float()
        g = g * dropout_scale
        dx = scale * y * (g - (g * y).sum(-1, keepdim=True))
        if tril:
            r = torch.arange(tril_rows)[:, None]
            c = torch.arange(cols)[None, :]
            dx = dx.masked_fill(c > r + diagonal, 0.0)
        return dx.to(dy.dtype)
    _need_bf16(softmax_y, dy)
    if dropout_mask is not None and dropout_mask.dtype == torch.bool:
        dropout_mask = dropout_mask.view(torch.uint8)
    dx = torch.empty_like(dy)
    check(_lib().ofb_softmax_bwd(ptr(softmax_y), ptr(dy), ptr(dropout_mask), ptr(dx), c_longlong(rows), c_int(cols),
                                 c_int(int(tril)), c_int(tril_rows), c_int(diagonal), c_float(scale),
                                 c_float(dropout_scale), stream_ptr()), "softmax_bwd")
    _count()
    return dx


# ------------------------------------------------------------------------------------------------
# sparse softmax cross-entropy (vocabulary-shardable)
# ------------------------------------------------------------------------------------------------
def xent_stats(logits, labels, vocab_start=0):
    """Per-row (max, sum exp(x - max), logit at the label if it lies in this shard): fp32 [rows, 3]."""
    rows, cols = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        mx = lf.max(-1).values
        s = torch.exp(lf - mx[:, None]).sum(-1)
        lab = labels - vocab_start
        inside = (lab >= 0) & (lab < cols)
        tgt = torch.where(inside, lf.gather(1, lab.clamp(0, cols - 1)[:, None])[:, 0], torch.zeros_like(mx))
        return torch.stack([mx, s, tgt], 1)
    stats = torch.empty(rows, 3, dtype=torch.float32, device=logits.device)
    check(_lib().ofb_xent_stats(ptr(logits), ptr(labels), ptr(stats), c_int(rows), c_int(cols),
                                c_longlong(logits.stride(0)), c_int(vocab_start), stream_ptr()), "xent_stats")
    _count()
    return stats


def xent_merge(parts):
    """Merges [nshards, rows, 3] statistics into [rows, 3]."""
    n, rows, _ = parts.shape
    if not parts.is_cuda:
        gm = parts[:, :, 0].max(0).values
        s = (parts[:, :, 1] * torch.exp(parts[:, :, 0] - gm[None])).sum(0)
        return torch.stack([gm, s, parts[:, :, 2].sum(0)], 1)
    parts = parts.contiguous()
    merged = torch.empty(rows, 3, dtype=torch.float32, device=parts.device)
    check(_lib().ofb_xent_merge(ptr(parts), ptr(merged), c_int(n), c_int(rows), stream_ptr()), "xent_merge")
    _count()
    return merged


def xent_grad(logits, labels, merged, grad_scale=1.0, vocab_start=0, ignore_index=-100, want_grad=True, inplace=False):
    """loss[row] = log(sum) + max - target ; dlogits = (softmax - onehot) * grad_scale. Returns (loss, dlogits)."""
    rows, cols = logits.shape
    if not logits.is_cuda:
        gm, s, tgt = merged[:, 0], merged[:, 1], merged[:, 2]
        ign = labels == ignore_index
        loss = torch.where(ign, torch.zeros_like(gm), torch.log(s) + gm - tgt)
        d = None
        if want_grad:
            d = torch.exp(logits.float() - gm[:, None]) / s[:, None]
            lab = labels - vocab_start
            inside = (lab >= 0) & (lab < cols) & ~ign
            idx = torch.nonzero(inside)[:, 0]
            d[idx, lab[idx]] -= 1.0
            d = d * grad_scale
            d[ign] = 0
            d = d.to(logits.dtype)
        return loss, d
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    d = (logits if inplace else torch.empty_like(logits)) if want_grad else None
    check(_lib().ofb_xent_grad(ptr(logits), ptr(labels), ptr(merged), ptr(loss), ptr(d), c_int(rows), c_int(cols),
                               c_longlong(logits.stride(0)), c_int(vocab_start), c_float(grad_scale),
                               c_longlong(ignore_index), stream_ptr()), "xent_grad")
    _count()
    return loss, d


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
def _bshd_stride(t, name):
    B, S, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D or t.stride(0) != S * t.stride(1):
        raise ValueError(f"fmha: {name} must be a [B,S,H,D] view with contiguous heads inside a token row")
    return t.stride(1)


def fmha_dropout_mask(B, H, Sq, Sk, p, seed, offset, device):
    """bool [B, H, Sq, Sk]: the keep mask the fused attention kernels regenerate from (seed, offset) (Philox4x32-10 indexed by
    batch*heads + head, query row and group of four key columns). CUDA only: the CPU fallback draws its own mask."""
    mask = torch.empty((B * H, Sq, Sk), dtype=torch.uint8, device=device)
    check(_lib().ofb_fmha_dropout_mask(ptr(mask), c_int(B * H), c_int(Sq), c_int(Sk), c_float(p), c_ulonglong(int(seed) & (2 ** 64 - 1)),
                                       c_uint(int(offset) & 0xFFFFFFFF), stream_ptr()), "fmha_dropout_mask")
    _count()
    return mask.view(B, H, Sq, Sk).bool()


def fmha_reference(q, k, v, causal, scale, kv_len=None, dropout_p=0.0, keep_mask=None):
    """fp32 PyTorch attention: q [B,Sq,H,D], k / v [B,Sk,Hk,D] (H a multiple of Hk) -> (out [B,Sq,H,D], lse [B,H,Sq]).
    Causal: query row r sees key columns <= r + (Sk - Sq). ``keep_mask`` (bool [B,H,Sq,Sk]) with ``dropout_p`` drops
    probabilities after the softmax; without a mask one is drawn from torch's generator."""
    B, Sq, H, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    if Hk != H:
        kf, vf = (t.repeat_interleave(H // Hk, dim=1) for t in (kf, vf))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        m = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(Sk - Sq)
        s = s.masked_fill(~m, float("-inf"))
    if kv_len is not None:
        cols = torch.arange(Sk, device=q.device)[None, None, None, :]
        s = s.masked_fill(cols >= kv_len.to(q.device)[:, None, None, None], float("-inf"))
    lse = torch.logsumexp(s, -1)
    dead = torch.isinf(lse)[..., None]          # rows that see no key at all: zero output, zero gradient
    p = torch.softmax(s.masked_fill(dead, 0.0), -1) * (~dead)
    if dropout_p > 0.0:
        if keep_mask is None:
            keep_mask = torch.rand(p.shape, device=p.device) >= dropout_p
        p = p * keep_mask.to(p.dtype) / (1.0 - dropout_p)
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).contiguous()
    return o.to(q.dtype), lse


def fmha_fwd(q, k, v, causal=False, scale=None, kv_len=None, dropout_p=0.0, seed=0, offset=0):
    """Fused attention forward. q: bf16 [B,Sq,H,D] view, k / v: [B,Sk,Hk,D] views (all may alias one packed QKV buffer;
    Hk divides H: grouped-query attention). ``dropout_p`` > 0 drops probabilities by the Philox stream (seed, offset);
    the same pair must be given to ``fmha_bwd``. Returns (out [B,Sq,H,D] contiguous, lse fp32 [B,H,Sq])."""
    B, Sq, H, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        return fmha_reference(q, k, v, causal, scale, kv_len, dropout_p)
    if k.shape != v.shape or k.shape[0] != B or k.shape[3] != D or H % Hk:
        raise ValueError(f"fmha: incompatible shapes q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    qs, ks, vs = _bshd_stride(q, "q"), _bshd_stride(k, "k"), _bshd_stride(v, "v")
    if ks != vs:
        raise ValueError("fmha: k and v must share their token stride")
    out = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    if kv_len is not None:
        kv_len = kv_len.to(device=q.device, dtype=torch.int32).contiguous()
    check(_lib().ofb_fmha_fwd_ex(ptr(q), ptr(k), ptr(v), c_longlong(qs), c_longlong(ks), ptr(out), ptr(lse), ptr(kv_len),
                                 c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(Hk), c_int(D), c_int(int(causal)), c_float(scale),
                                 c_float(dropout_p), c_ulonglong(int(seed) & (2 ** 64 - 1)), c_uint(int(offset) & 0xFFFFFFFF),
                                 stream_ptr()), "fmha_fwd")
    _count()
    return out, lse


# ------------------------------------------------------------------------------------------------
# optimizer kernels
# ------------------------------------------------------------------------------------------------
def _ptr_array(tensors):
    arr = (c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if t is not None else None
    return arr


def _size_array(tensors):
    arr = (c_longlong * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.numel()
    return arr


_MAX_TENSORS = 48


def multi_tensor_adamw(grads, masters, copies, ms, vs, *, lr, beta1, beta2, eps, weight_decay, l2=0.0, scale=1.0,
                       step=1, bias_correction=True, lr_tensor=None, scale_tensor=None, skip_if=None):
    """One fused AdamW step over lists of tensors (fp32 masters/moments, bf16 or fp32 grads, optional bf16 copies)."""
    bc1 = 1.0 - beta1 ** step if bias_correction else 1.0
    bc2 = 1.0 - beta2 ** step if bias_correction else 1.0
    if not masters[0].is_cuda:
        for i, w in enumerate(masters):
            if skip_if is not None and int(skip_if.item()) != 0:
                break
            s = scale * (float(scale_tensor.item()) if scale_tensor is not None else 1.0)
            cur_lr = float(lr_tensor.item()) if lr_tensor is not None else lr
            g = grads[i].float() * s + l2 * w
            ms[i].mul_(beta1).add_(g, alpha=1 - beta1)
            vs[i].mul_(beta2).addcmul_(g, g, value=1 - beta2)
            denom = vs[i].sqrt() / math.sqrt(bc2) + eps
            w.sub_((cur_lr / bc1) * (ms[i] / denom) + cur_lr * weight_decay * w)
            if copies is not None and copies[i] is not None:
                copies[i].copy_(w)
        return
    grad_is_bf16 = int(grads[0].dtype == torch.bfloat16)
    for s0 in range(0, len(masters), _MAX_TENSORS):
        sl = slice(s0, s0 + _MAX_TENSORS)
        g, w, m, v = grads[sl], masters[sl], ms[sl], vs[sl]
        c = copies[sl] if copies is not None else [None] * len(w)
        check(_lib().ofb_multi_tensor_adamw(
            c_int(len(w)), _ptr_array(g), _ptr_array(w), _ptr_array(c), _ptr_array(m), _ptr_array(v), _size_array(w),
            c_int(grad_is_bf16), c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(weight_decay),
            c_float(l2), c_float(scale), c_float(bc1), c_float(bc2), ptr(lr_tensor), ptr(scale_tensor), ptr(skip_if),
            stream_ptr()), "multi_tensor_adamw")
        _count()


def multi_tensor_sgd(grads, masters, copies, ms, *, lr, momentum=0.0, dampening=0.0, nesterov=False, maximize=False,
                     weight_decay=0.0, l1=0.0, l2=0.0, scale=1.0, lr_tensor=None, scale_tensor=None, skip_if=None):
    """One fused SGD(+momentum) step over lists of tensors."""
    if not masters[0].is_cuda:
        for i, w in enumerate(masters):
            if skip_if is not None and int(skip_if.item()) != 0:
                break
            s = scale * (float(scale_tensor.item()) if scale_tensor is not None else 1.0)
            cur_lr = float(lr_tensor.item()) if lr_tensor is not None else lr
            g = grads[i].float() * s + l1 * torch.sign(w) + l2 * w
            if ms is not None and ms[i] is not None:
                ms[i].mul_(momentum).add_(g, alpha=1 - dampening)
                g = g + momentum * ms[i] if nesterov else ms[i]
            w.copy_((w + cur_lr * g if maximize else w - cur_lr * g) - cur_lr * weight_decay * w)
            if copies is not None and copies[i] is not None:
                copies[i].copy_(w)
        return
    grad_is_bf16 = int(grads[0].dtype == torch.bfloat16)
    for s0 in range(0, len(masters), _MAX_TENSORS):
        sl = slice(s0, s0 + _MAX_TENSORS)
        g, w = grads[sl], masters[sl]
        m = ms[sl] if ms is not None else [None] * len(w)
        c = copies[sl] if copies is not None else [None] * len(w)
        check(_lib().ofb_multi_tensor_sgd(
            c_int(len(w)), _ptr_array(g), _ptr_array(w), _ptr_array(c), _ptr_array(m), _size_array(w),
            c_int(grad_is_bf16), c_float(lr), c_float(momentum), c_float(dampening), c_int(int(nesterov)),
            c_int(int(maximize)), c_float(weight_decay), c_float(l1), c_float(l2), c_float(scale), ptr(lr_tensor),
            ptr(scale_tensor), ptr(skip_if), stream_ptr()), "multi_tensor_sgd")
        _count()


def multi_tensor_sqsum(grads, out=None):
    """out[0] = sum of squares of all finite gradient entries, out[1] = number of non-finite entries (fp32 [2])."""
    if not grads[0].is_cuda:
        s = sum(float(torch.where(torch.isfinite(g.float()), g.float(), torch.zeros(())).pow(2).sum()) for g in grads)
        bad = sum(int((~torch.isfinite(g.float())).sum()) for g in grads)
        r = torch.tensor([s, float(bad)], dtype=torch.float32)
        if out is not None:
            out.copy_(r)
            return out
        return r
    dev = grads[0].device
    if out is None:
        out = torch.empty(2, dtype=torch.float32, device=dev)
    scratch = torch.empty(_lib().ofb_sqsum_scratch_floats(), dtype=torch.float32, device=dev)
    grad_is_bf16 = int(grads[0].dtype == torch.bfloat16)
    for k, s0 in enumerate(range(0, len(grads), _MAX_TENSORS)):
        g = grads[s0:s0 + _MAX_TENSORS]
        check(_lib().ofb_multi_tensor_sqsum(c_int(len(g)), _ptr_array(g), _size_array(g), c_int(grad_is_bf16),
                                            ptr(scratch), ptr(out), c_int(int(k > 0)), stream_ptr()),
              "multi_tensor_sqsum")
        _count(2)
    return out


def clip_factor(sq_and_bad, max_norm):
    """From multi_tensor_sqsum's output: (clip factor fp32 [1], found_inf int64 [1], total_norm fp32 [1])."""
    if not sq_and_bad.is_cuda:
        norm = sq_and_bad[0].sqrt()
        f = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones(())
        return f.reshape(1), (sq_and_bad[1] > 0).long().reshape(1), norm.reshape(1)
    dev = sq_and_bad.device
    factor = torch.empty(1, dtype=torch.float32, device=dev)
    found = torch.empty(1, dtype=torch.int64, device=dev)
    norm = torch.empty(1, dtype=torch.float32, device=dev)
    check(_lib().ofb_clip_factor(ptr(sq_and_bad), c_float(max_norm), ptr(factor), ptr(found), ptr(norm), stream_ptr()),
          "clip_factor")
    _count()
    return factor, found, norm


def fmha_bwd_reference(q, k, v, o, d_o, lse, causal, scale, kv_len=None, dropout_p=0.0, keep_mask=None):
    """fp32 PyTorch attention backward (shapes as ``fmha_reference``) -> (dq, dk, dv)."""
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad():
        out, _ = fmha_reference(qf, kf, vf, causal, scale, kv_len, dropout_p, keep_mask)
        out.backward(d_o.float())
    return qf.grad.to(q.dtype), kf.grad.to(q.dtype), vf.grad.to(q.dtype)


def fmha_bwd(q, k, v, o, d_o, lse, causal=False, scale=None, kv_len=None, dqkv=None, dropout_p=0.0, seed=0, offset=0):
    """Fused attention backward. Self-attention with one head count (q, k, v of one shape): returns (dq, dk, dv) as
    [B,S,H,D] views of one packed [B,S,3,H,D] buffer (``dqkv`` if given), so that the QKV projection's backward consumes a
    single matrix. Otherwise (other key length, fewer key/value heads): three separate contiguous tensors."""
    B, Sq, H, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    packed = (Sk == Sq and Hk == H)
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        if dropout_p > 0.0:
            raise ValueError("fmha_bwd on CPU cannot regenerate the forward's dropout mask; differentiate fmha_reference instead")
        dq, dk, dv = fmha_bwd_reference(q, k, v, o, d_o, lse, causal, scale, kv_len)
        if not packed:
            return dq, dk, dv
        if dqkv is None:
            dqkv = torch.empty((B, Sq, 3, H, D), dtype=q.dtype)
        dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2] = dq, dk, dv
        return dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    qs, ks, vs = _bshd_stride(q, "q"), _bshd_stride(k, "k"), _bshd_stride(v, "v")
    if ks != vs:
        raise ValueError("fmha: k and v must share their token stride")
    _need_bf16(o, d_o)
    if packed:
        if dqkv is None:
            dqkv = torch.empty((B, Sq, 3, H, D), dtype=torch.bfloat16, device=q.device)
        dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
        dq_stride = dkv_stride = 3 * H * D
    else:
        dq = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q.device)
        dkv = torch.empty((B, Sk, 2, Hk, D), dtype=torch.bfloat16, device=q.device)
        dk, dv = dkv[:, :, 0], dkv[:, :, 1]
        dq_stride, dkv_stride = H * D, 2 * Hk * D
    _lib().ofb_fmha_bwd_scratch_floats.restype = c_longlong
    n = _lib().ofb_fmha_bwd_scratch_floats(c_int(B), c_int(Sq), c_int(H), c_int(D))
    scratch = torch.empty(n, dtype=torch.float32, device=q.device)
    if kv_len is not None:
        kv_len = kv_len.to(device=q.device, dtype=torch.int32).contiguous()
    check(_lib().ofb_fmha_bwd_ex(ptr(q), ptr(k), ptr(v), c_longlong(qs), c_longlong(ks), ptr(o), ptr(d_o), ptr(lse),
                                 ptr(dq), ptr(dk), ptr(dv), c_longlong(dq_stride), c_longlong(dkv_stride), ptr(scratch), ptr(kv_len),
                                 c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(Hk), c_int(D), c_int(int(causal)), c_float(scale),
                                 c_float(dropout_p), c_ulonglong(int(seed) & (2 ** 64 - 1)), c_uint(int(offset) & 0xFFFFFFFF),
                                 stream_ptr()), "fmha_bwd")
    _count(4)
    return dq, dk, dv


def bce_logits(logits, labels, loss_scale=1.0, grad_scale=1.0, loss_sum=None):
    """Binary cross entropy on ``logits[:, 0]`` against fp32 ``labels``: returns (loss_sum [1] fp32, dlogits like
    logits with the gradient in column 0 and zeros elsewhere). ``loss_sum`` accumulates when passed in."""
    rows, ld = logits.shape
    if not logits.is_cuda:
        x = logits[:, 0].float()
        loss = (torch.clamp(x, min=0) - x * labels + torch.log1p(torch.exp(-x.abs()))).sum() * loss_scale
        d = torch.zeros_like(logits)
        d[:, 0] = (grad_scale * (torch.sigmoid(x) - labels)).to(logits.dtype)
        out = loss.reshape(1) if loss_sum is None else loss_sum.add_(loss)
        return out, d
    _need_bf16(logits)
    if loss_sum is None:
        loss_sum = torch.zeros(1, dtype=torch.float32, device=logits.device)
    d = torch.empty_like(logits)
    check(_lib().ofb_bce_logits(ptr(logits), c_int(ld), ptr(labels), ptr(d), ptr(loss_sum), c_longlong(rows),
                                c_float(loss_scale), c_float(grad_scale), stream_ptr()), "bce_logits")
    _count()
    return loss_sum, d


def _interaction_on_tensor_cores(D, T, self_interaction, out_dim):
    """The tcgen05 kernels cover the DLRM shape class: dim 128, up to 31 sparse features, strict lower triangle."""
    import os
    return (D == 128 and 1 <= T <= 31 and not self_interaction and out_dim % 8 == 0 and out_dim - D <= 512
            and os.environ.get("OFB_INTERACTION_TC", "1") != "0")


def interaction_fwd(dense, sparse, self_interaction=False, out_dim=None):
    """[dense | lower triangle of X X^T | zero pad] with X = [dense; sparse] per sample (no autograd)."""
    B, D = dense.shape
    T = sparse.shape[1]
    F = T + 1
    npairs = F * (F + 1) // 2 if self_interaction else F * (F - 1) // 2
    out_dim = out_dim or (D + npairs + 7) // 8 * 8
    if not dense.is_cuda:
        from .interaction import dot_feature_interaction_reference
        return dot_feature_interaction_reference([dense, sparse], dense, self_interaction, out_dim - D - npairs)
    out = torch.empty((B, out_dim), dtype=dense.dtype, device=dense.device)
    if _interaction_on_tensor_cores(D, T, self_interaction, out_dim):
        check(_lib().ofb_interaction_tc_fwd(ptr(dense), ptr(sparse), ptr(out), c_longlong(B), c_int(T), c_int(D), c_int(out_dim),
                                            stream_ptr()), "interaction_tc_fwd")
        _count()
        return out
    check(_lib().ofb_interaction_fwd(ptr(dense), ptr(sparse), ptr(out), c_longlong(B), c_int(T), c_int(D), c_int(int(self_interaction)),
                                     c_int(out_dim), stream_ptr()), "interaction_fwd")
    _count()
    return out


def interaction_bwd(dense, sparse, dout, self_interaction=False):
    """Gradients of interaction_fwd wrt (dense, sparse)."""
    B, D = dense.shape
    T = sparse.shape[1]
    if not dense.is_cuda:
        from .interaction import dot_feature_interaction_reference
        d32, s32 = dense.float().requires_grad_(), sparse.float().requires_grad_()
        F = T + 1
        npairs = F * (F + 1) // 2 if self_interaction else F * (F - 1) // 2
        ref = dot_feature_interaction_reference([d32, s32], d32, self_interaction, dout.shape[1] - D - npairs)
        ref.backward(dout.float())
        return d32.grad.to(dense.dtype), s32.grad.to(sparse.dtype)
    dd, ds = torch.empty_like(dense), torch.empty_like(sparse)
    if _interaction_on_tensor_cores(D, T, self_interaction, dout.shape[1]):
        check(_lib().ofb_interaction_tc_bwd(ptr(dense), ptr(sparse), ptr(dout.contiguous()), ptr(dd), ptr(ds), c_longlong(B), c_int(T),
                                            c_int(D), c_int(dout.shape[1]), stream_ptr()), "interaction_tc_bwd")
        _count()
        return dd, ds
    check(_lib().ofb_interaction_bwd(ptr(dense), ptr(sparse), ptr(dout.contiguous()), ptr(dd), ptr(ds), c_longlong(B), c_int(T), c_int(D),
                                     c_int(int(self_interaction)), c_int(dout.shape[1]), stream_ptr()), "interaction_bwd")
    _count()
    return dd, ds
