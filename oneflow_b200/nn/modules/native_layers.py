"""``flow.nn.Linear`` / ``LayerNorm`` / ``Embedding``: torch's layers (same constructor, same parameters, same
state dict) whose forward goes through ``framework/fused_ops``: bf16 CUDA tensors run the hand-written GEMM /
LayerNorm / embedding kernels, global tensors additionally pick their SBP signature there (tensor-parallel weights
use the fused all-gather->GEMM and GEMM->reduce-scatter kernels). Other inputs take PyTorch's path unchanged.
Reference layers: python/oneflow/nn/modules/linear.py, normalization.py (LayerNorm), sparse.py (Embedding)."""
from __future__ import annotations

import torch

from ...framework import fused_ops as F


class Linear(torch.nn.Linear):
    def forward(self, input):
        return F.linear(input, self.weight, self.bias)


class LayerNorm(torch.nn.LayerNorm):
    def forward(self, input):
        if self.weight is None or self.bias is None:
            return super().forward(input)
        return F.layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps)


class Embedding(torch.nn.Embedding):
    def forward(self, input):
        if self.padding_idx is not None or self.max_norm is not None or self.scale_grad_by_freq or self.sparse:
            return super().forward(input)
        return F.embedding(input, self.weight)
