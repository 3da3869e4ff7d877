"""Native dot-feature-interaction (csrc/kernels/interaction.cu) with autograd."""
from __future__ import annotations

from ctypes import c_int, c_longlong

import torch

from . import _native
from . import kernels as _k
from ._native import check, ptr, stream_ptr


class _Interaction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dense, sparse, self_interaction, out_dim):
        B, D = dense.shape
        T = sparse.shape[1]
        out = _k.interaction_fwd(dense, sparse, self_interaction, out_dim)
        ctx.save_for_backward(dense, sparse)
        ctx.args = (self_interaction, out_dim)
        return out

    @staticmethod
    def backward(ctx, dout):
        dense, sparse = ctx.saved_tensors
        self_interaction, out_dim = ctx.args
        B, D = dense.shape
        T = sparse.shape[1]
        dd, ds = _k.interaction_bwd(dense, sparse, dout, self_interaction)
        return dd, ds, None, None


def dot_feature_interaction_native(features, output_concat, self_interaction, output_padding):
    """features: [dense [B, D], sparse [B, T, D]] with output_concat is dense (the DLRM layout)."""
    if len(features) != 2 or features[0].dim() != 2 or features[1].dim() != 3 or output_concat is not features[0]:
        from .interaction import dot_feature_interaction_reference
        return dot_feature_interaction_reference(features, output_concat, self_interaction, output_padding)
    dense, sparse = features[0].contiguous(), features[1].contiguous()
    F = sparse.shape[1] + 1
    D = dense.shape[1]
    if F > 32 or D > 128 or D % 8:
        from .interaction import dot_feature_interaction_reference
        return dot_feature_interaction_reference(features, output_concat, self_interaction, output_padding)
    npairs = F * (F + 1) // 2 if self_interaction else F * (F - 1) // 2
    return _Interaction.apply(dense, sparse, bool(self_interaction), D + npairs + output_padding)
