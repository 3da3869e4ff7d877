"""The long tail of ``flow._C`` fused functions (reference: oneflow/core/functional/functional_api.yaml, the entries
named ``fused_*``, ``skip_*``, ``rms_*``, ``grouped_matmul*``): same signatures and maths, expressed with tensor ops
(autograd comes from PyTorch); the GEMM-shaped ones run on the tcgen05 GEMM with its fused epilogue for bf16 CUDA
tensors. Semantics follow the reference's own test oracles (python/oneflow/test/modules/test_fused_*.py)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _act(name, t):
    if name in (None, "none"):
        return t
    if name == "sigmoid":
        return torch.sigmoid(t)
    if name == "relu":
        return torch.relu(t)
    if name == "gelu":
        return F.gelu(t)
    if name == "fast_gelu":
        return F.gelu(t, approximate="tanh")
    if name == "silu":
        return F.silu(t)
    raise ValueError(f"unknown activation {name}")


def _linear(x, w, b=None):
    from ._C import fused_matmul_bias
    if b is not None:
        return fused_matmul_bias(x, w, b)
    return F.linear(x, w)


# ------------------------------------------------------------------------------------------------ normalisation
def rms_norm(x, weight=None, normalized_shape=None, epsilon=1e-6):
    dims = tuple(range(-len(normalized_shape), 0)) if normalized_shape is not None else (-1,)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dims, keepdim=True) + epsilon)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def rms_layer_norm(hidden_states, weight, variance_epsilon):
    return rms_norm(hidden_states, weight, (hidden_states.shape[-1],), variance_epsilon)


def skip_layer_norm(x, *, gamma=None, beta=None, bias=None, skip=None, epsilon=1e-5, alpha=1e1):
    """layer_norm(x + bias + alpha * skip) * gamma + beta over the last dimension."""
    t = x
    if bias is not None:
        t = t + bias
    if skip is not None:
        t = t + skip * alpha
    return F.layer_norm(t, (x.shape[-1],), gamma, beta, epsilon)


def skip_rms_norm(x, *, weight=None, bias=None, skip=None, epsilon=1e-5, alpha=1e1):
    t = x
    if bias is not None:
        t = t + bias
    if skip is not None:
        t = t + skip * alpha
    return rms_norm(t, weight, (x.shape[-1],), epsilon)


# ------------------------------------------------------------------------------------------------ GEMM family
def fused_glu(x, w, b=None, v=None, c=None, activation="none"):
    """hidden * act(gate): (hidden, gate) = chunk(x w^T + b, 2) or, with v / c, hidden = x w^T + b, gate = x v^T + c."""
    if v is not None:
        hidden, gate = _linear(x, w, b), _linear(x, v, c)
    else:
        hidden, gate = _linear(x, w, b).chunk(2, dim=-1)
    return hidden * _act(activation, gate)


def fused_matmul_bias_add_relu_dropout(x, weights, biases, skip_final_activation, dropout_rate_list, generator=None):
    n = len(weights)
    for i, (w, b) in enumerate(zip(weights, biases)):
        x = _linear(x, w, b)
        if not (skip_final_activation and i == n - 1):
            x = torch.relu(x)
        p = dropout_rate_list[i] if i < len(dropout_rate_list) else 0.0
        if p:
            x = F.dropout(x, p, True)
    return x


def grouped_matmul(xs, weights):
    return tuple(F.linear(x, w) for x, w in zip(xs, weights))


def grouped_matmul_bias(xs, weights, biases):
    return tuple(_linear(x, w, b) for x, w, b in zip(xs, weights, biases))


def fused_cross_feature_interaction(x, weight, x_0, bias, interaction_mode):
    """DCN-v2 cross layer: "vector": (x w^T) * x0 + bias + x ; "matrix": (x W^T + bias) * x0 + x."""
    if interaction_mode == "vector":
        return F.linear(x, weight) * x_0 + bias + x
    if interaction_mode == "matrix":
        return (F.linear(x, weight) + bias) * x_0 + x
    raise ValueError("interaction_mode must be 'vector' or 'matrix'")


def fused_fast_gelu_mul(x, multiplier):
    return F.gelu(x, approximate="tanh") * multiplier


def fused_weighted_sum(inputs, weights, alpha=1.0):
    out = inputs[0] * weights[0]
    for t, w in zip(inputs[1:], weights[1:]):
        out = out + t * w
    return out * alpha


def fused_clip_grad(model_diff, max_norm, norm_type):
    """Scales the gradients in place so that their joint norm is at most max_norm; returns the norm before clipping."""
    if norm_type == float("inf"):
        total = torch.stack([g.detach().abs().max().float() for g in model_diff]).max()
    elif norm_type == -float("inf"):
        total = torch.stack([g.detach().abs().min().float() for g in model_diff]).min()
    else:
        total = torch.stack([g.detach().float().norm(norm_type) for g in model_diff]).norm(norm_type)
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in model_diff:
        g.mul_(coef.to(g.dtype))
    return total


# ------------------------------------------------------------------------------------------------ attention helpers
def fused_scale_tril(x, diagonal=0, fill_value=0, scale=1):
    mask = torch.ones(x.shape[-2:], dtype=torch.bool, device=x.device).tril(diagonal)
    return torch.where(mask, x * scale, torch.full_like(x, fill_value))


def fused_scale_mask_bias_softmax(x, mask, bias=None, scale=0.35355, inplace=False):
    t = x * scale + mask
    if bias is not None:
        t = t + bias
    return torch.softmax(t, -1)


def fused_bias_add_scale_mask_softmax_dropout(x, bias, mask, *, fill_value=0.0, scale=1.0, p=0.5, training=True, generator=None):
    t = (x + bias) * scale
    t = torch.where(mask.bool(), t, torch.full_like(t, fill_value))
    sm = torch.softmax(t, -1)
    return F.dropout(sm, p, training), sm


def fused_self_attention(hidden_states, head_size=8, alpha=1.0):
    """hidden_states [seq, batch, 3 * heads * head_size] (q, k, v interleaved per head) -> (alpha * q k^T [b, h, s, s], v [s, b, h * d])."""
    s, b, three_h = hidden_states.shape
    heads = three_h // (3 * head_size)
    t = hidden_states.view(s, b, heads, 3, head_size)
    q, k, v = t[..., 0, :], t[..., 1, :], t[..., 2, :]
    qk = torch.einsum("sbhd,tbhd->bhst", q, k) * alpha
    return qk, v.reshape(s, b, heads * head_size)


def fused_codegeex_qkv_reshape(query, key, value, num_attention_heads):
    def r(t):
        return t.reshape(t.shape[0], t.shape[1], num_attention_heads, t.shape[2] // num_attention_heads).contiguous()
    return r(query), r(key), r(value)


def fused_attention_concat_past_key_value(*, past_key=None, past_key_layout="BHMK", past_value=None, past_value_layout="BHMK", key,
                                          key_layout="BHMK", value, value_layout="BHMK", key_head_size=None):
    """Appends this step's key / value to the cache along the sequence axis.  The new tensors may come in any layout
    (also packed ``H2K`` / ``H3K``: key is tensor 0 / 1, value tensor 1 / 2 of the packing); the results are laid out
    like the caches (``past_*_layout``)."""
    from .ops import attn_layout as L
    hs = key_head_size
    if hs is None:
        ref = key if key_layout in ("BHMK", "BMHK", "MBHK") else (past_key if past_key is not None and past_key.dim() == 4 else None)
        if ref is None:
            raise ValueError("key_head_size is required when no 4-D tensor gives the head size")
        hs = ref.shape[-1]
    k_index = {"H2K": 0, "H3K": 1}.get(key_layout[3:-1] if "(" in key_layout else "", 0)
    v_index = {"H2K": 1, "H3K": 2}.get(value_layout[3:-1] if "(" in value_layout else "", 0)
    k = L.unpack(key, key_layout, head_size=hs, index=k_index)
    v = L.unpack(value, value_layout, head_size=hs, index=v_index)
    if past_key is not None:
        k = torch.cat([L.unpack(past_key, past_key_layout, head_size=hs), k], 2)
        v = torch.cat([L.unpack(past_value, past_value_layout, head_size=hs), v], 2)
    return L.pack(k, past_key_layout).contiguous(), L.pack(v, past_value_layout).contiguous()


def fused_apply_rotary_emb(x, *, cos=None, sin=None, position_ids=None, x_layout="BHMK", output_layout=None, mode="plane",
                           tensor_index=None, k_size=None, base=1e4, rotary_size=None):
    """Rotary position embedding over the first ``rotary_size`` elements of every head.

    ``cos`` / ``sin``: tables ``[positions, rotary_size // n]``, column ``c`` used for element ``c`` of a block; computed
    from ``base`` when absent, the two elements of pair ``j`` then get the frequency ``base ** (-2j / (rotary_size // n))``.  ``position_ids``: ``[B, n, M]`` for
    ``n``-dimensional positions (the rotary part splits into ``n`` blocks, one per coordinate); positions ``0..M-1``
    when absent.  Element ``i`` of a block is paired in ``"plane"`` mode with the element half a block away
    (``(-x2, x1)``), in ``"interval"`` mode with its neighbour (``(-x[2j+1], x[2j])``).  ``x`` may be packed
    (``BM(H3K)``: ``tensor_index`` picks query / key / value); the result comes in ``output_layout``
    (reference: oneflow/user/kernels/fused_attention_kernels.cu, FusedApplyRotaryEmb)."""
    from .ops import attn_layout as L
    packed = x_layout.endswith(("(H2K)", "(H3K)"))
    if packed and (output_layout is None or output_layout == x_layout):
        # the packed tensors are all rotated and come back packed the same way
        n = 2 if x_layout.endswith("(H2K)") else 3
        parts = [fused_apply_rotary_emb(x, cos=cos, sin=sin, position_ids=position_ids, x_layout=x_layout, output_layout="BMHK",
                                        mode=mode, tensor_index=t, k_size=k_size, base=base, rotary_size=rotary_size)
                 for t in range(n)]
        y = torch.stack(parts, 3)                                                 # [B, M, H, n, K]
        y = y.reshape(y.shape[0], y.shape[1], -1)
        return (y if x_layout.startswith("BM") else y.transpose(0, 1)).contiguous()
    q = L.unpack(x, x_layout, head_size=k_size, index=tensor_index or 0)
    B, H, M, K = q.shape
    rs = int(rotary_size) if rotary_size else K
    nd = position_ids.shape[1] if position_ids is not None else 1
    act = rs // nd
    dev = x.device
    i = torch.arange(rs, device=dev)
    col, blk = i % act, i // act
    pos = position_ids.to(dev).long() if position_ids is not None else torch.arange(M, device=dev).expand(B, 1, M)
    p = pos[:, blk, :].permute(0, 2, 1)                                             # [B, M, rs]: position per element
    if cos is None or sin is None:
        # pair index of an element: its offset inside the half block ("plane") or half its offset ("interval")
        pair = col % max(act // 2, 1) if mode == "plane" else col // 2
        freq = float(base) ** (-2.0 * pair.float() / act)
        ang = p.float() * freq
        c, s = ang.cos(), ang.sin()
    else:
        c, s = cos.to(dev)[p, col], sin.to(dev)[p, col]
    c, s = c[:, None].to(q.dtype), s[:, None].to(q.dtype)                           # [B, 1, M, rs]
    xr = q[..., :rs]
    if mode == "plane":
        xb = xr.reshape(B, H, M, nd, act)
        rot = torch.cat([-xb[..., act // 2:], xb[..., :act // 2]], -1).reshape(B, H, M, rs)
    elif mode == "interval":
        rot = torch.stack([-xr[..., 1::2], xr[..., 0::2]], -1).flatten(-2)
    else:
        raise ValueError(f"fused_apply_rotary_emb: unknown mode {mode!r}")
    y = torch.cat([xr * c + rot * s, q[..., rs:]], -1)
    return L.pack(y, output_layout or x_layout).contiguous()


# ------------------------------------------------------------------------------------------------ box IoU family (YOLO CIoU loss)
def fused_get_boundding_boxes_coord(x1, y1, w1, h1, x2, y2, w2, h2):
    return (x1 - w1 / 2, x1 + w1 / 2, y1 - h1 / 2, y1 + h1 / 2, x2 - w2 / 2, x2 + w2 / 2, y2 - h2 / 2, y2 + h2 / 2)


def fused_get_intersection_area(b1_x1, b1_x2, b2_x1, b2_x2, b1_y1, b1_y2, b2_y1, b2_y2):
    return (torch.min(b1_x2, b2_x2) - torch.max(b1_x1, b2_x1)).clamp(0) * (torch.min(b1_y2, b2_y2) - torch.max(b1_y1, b2_y1)).clamp(0)


def fused_get_iou(w1, h1, w2, h2, inter, eps):
    return inter / (w1 * h1 + w2 * h2 - inter + eps)


def fused_get_center_dist(b1_x1, b1_x2, b2_x1, b2_x2, b1_y1, b1_y2, b2_y1, b2_y2):
    return ((b2_x1 + b2_x2 - b1_x1 - b1_x2) ** 2 + (b2_y1 + b2_y2 - b1_y1 - b1_y2) ** 2) / 4


def fused_get_convex_diagonal_squared(b1_x1, b1_x2, b2_x1, b2_x2, b1_y1, b1_y2, b2_y1, b2_y2, eps):
    cw = torch.max(b1_x2, b2_x2) - torch.min(b1_x1, b2_x1)
    ch = torch.max(b1_y2, b2_y2) - torch.min(b1_y1, b2_y1)
    return cw ** 2 + ch ** 2 + eps


def fused_get_ciou_diagonal_angle(w1, h1, w2, h2, eps):
    return (4 / math.pi ** 2) * torch.pow(torch.atan(w2 / (h2 + eps)) - torch.atan(w1 / (h1 + eps)), 2)


def fused_get_ciou_result(v, iou, rho2, c2, eps):
    with torch.no_grad():
        alpha = v / (v - iou + (1.0 + eps))
    return iou - (rho2 / c2 + v * alpha), alpha
