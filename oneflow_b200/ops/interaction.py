"""DLRM dot feature interaction: concatenate F feature vectors per sample, take all pairwise dot products
``Z = X X^T``, keep the (strict) lower triangle, prepend ``output_concat`` and zero-pad
(reference: oneflow/user/kernels/fused_dot_feature_interaction_kernel.cu :1141-1413).
bf16/fp16 CUDA inputs run the native kernel (csrc/kernels/interaction.cu) when it is available."""
from __future__ import annotations

import torch


def dot_feature_interaction_reference(features, output_concat=None, self_interaction=False, output_padding=0, pooling="none"):
    x = torch.cat([f if f.dim() == 3 else f.unsqueeze(1) for f in features], 1)  # [B, F, D]
    if pooling == "sum":
        # sum pooling variant: (sum_i x_i)^2 - sum_i x_i^2 per embedding element, halved
        s = x.sum(1)
        out = 0.5 * (s * s - (x * x).sum(1))
    else:
        z = torch.bmm(x, x.transpose(1, 2))
        F = x.shape[1]
        idx = torch.tril_indices(F, F, offset=0 if self_interaction else -1, device=x.device)
        out = z[:, idx[0], idx[1]]
    parts = ([output_concat] if output_concat is not None else []) + [out]
    if output_padding:
        parts.append(out.new_zeros(out.shape[0], output_padding))
    return torch.cat(parts, 1)


def dot_feature_interaction(features, output_concat=None, self_interaction=False, output_padding=0, pooling="none"):
    x0 = features[0]
    if x0.is_cuda and x0.dtype == torch.bfloat16 and pooling == "none":
        # CUDA bf16 inputs always take the native kernels: a missing kernel library raises instead of falling back
        from .interaction_native import dot_feature_interaction_native
        return dot_feature_interaction_native(features, output_concat, self_interaction, output_padding)
    return dot_feature_interaction_reference(features, output_concat, self_interaction, output_padding, pooling)
