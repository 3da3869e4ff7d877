"""Attention tensor layouts of the fused attention / rotary / KV-cache ops: a string names the order of batch (B),
sequence (M), heads (H) and head size (K); parentheses merge axes; ``H2K`` / ``H3K`` pack key+value or
query+key+value per head (reference: oneflow/core/functional/impl/fused_attention_functor.cpp:39-200).
``unpack`` gives the canonical ``[B, H, M, K]`` view of one of the packed tensors, ``pack`` lays a canonical tensor
out again.  Views only: nothing is copied until a consumer needs contiguity."""
from __future__ import annotations

_PLAIN = {"BHMK": (0, 1, 2, 3), "BMHK": (0, 2, 1, 3), "MBHK": (1, 2, 0, 3)}     # permutation that yields B, H, M, K


def unpack(t, layout, head_size=None, num_heads=None, index=0):
    """``t`` in ``layout`` -> ``[B, H, M, K]``.  ``index`` picks the tensor inside an ``H2K`` (0 key, 1 value) or
    ``H3K`` (0 query, 1 key, 2 value) packing; merged layouts need ``head_size`` or ``num_heads``."""
    if layout in _PLAIN:
        if t.dim() != 4:
            raise ValueError(f"layout {layout} needs a 4-D tensor, got {t.dim()}-D")
        return t.permute(*_PLAIN[layout])
    if layout in ("BM(HK)", "MB(HK)", "BM(H2K)", "MB(H2K)", "BM(H3K)", "MB(H3K)"):
        if t.dim() != 3:
            raise ValueError(f"layout {layout} needs a 3-D tensor, got {t.dim()}-D")
        n = {"HK": 1, "H2K": 2, "H3K": 3}[layout[3:-1]]
        hidden = t.shape[2]
        if head_size is None and num_heads is None:
            raise ValueError(f"layout {layout} needs head_size or num_heads")
        K = head_size if head_size is not None else hidden // (n * num_heads)
        if hidden % (n * K):
            raise ValueError(f"the last dimension {hidden} is not a multiple of {n} x head size {K}")
        H = hidden // (n * K)
        if not 0 <= index < n:
            raise ValueError(f"tensor index {index} outside the {n} tensors packed in {layout}")
        u = t.reshape(t.shape[0], t.shape[1], H, n, K)[:, :, :, index, :]          # [B|M, M|B, H, K]
        return u.permute(0, 2, 1, 3) if layout.startswith("BM") else u.permute(1, 2, 0, 3)
    raise ValueError(f"unsupported layout {layout}")


def pack(t, layout):
    """``[B, H, M, K]`` -> ``layout`` (the unpacked layouts and their merged forms)."""
    if layout == "BHMK":
        return t
    if layout == "BMHK":
        return t.permute(0, 2, 1, 3)
    if layout == "MBHK":
        return t.permute(2, 0, 1, 3)
    B, H, M, K = t.shape
    if layout == "BM(HK)":
        return t.permute(0, 2, 1, 3).reshape(B, M, H * K)
    if layout == "MB(HK)":
        return t.permute(2, 0, 1, 3).reshape(M, B, H * K)
    raise ValueError(f"unsupported output layout {layout}")


def seq_axis(layout):
    """Axis of the tensor (as laid out) that carries the sequence."""
    flat = layout.replace("(HK)", "X").replace("(H2K)", "X").replace("(H3K)", "X")
    return flat.index("M")
