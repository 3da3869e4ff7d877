"""``nn.FusedMLP``: a stack of Linear(+ReLU)(+dropout) layers executed as fused GEMM+bias+activation
kernels (reference: python/oneflow/nn/modules/fused_mlp.py, cublas_fused_mlp_kernel.cu). bf16 CUDA inputs
run each layer as one tcgen05 GEMM whose epilogue adds the bias and applies ReLU; the backward reuses the
GEMM with the activation-gradient epilogue and MN-major operands. Other inputs use the PyTorch ops."""
from __future__ import annotations

import torch

from ...ops import gemm as G
from ...ops import kernels as K


class _FusedLinearAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        x2 = x.reshape(-1, x.shape[-1])
        y, pre = G.gemm(x2, w, bias=b, act=act, want_aux=True) if act else (G.gemm(x2, w, bias=b), None)
        ctx.save_for_backward(x2, w, pre)
        ctx.act, ctx.shape, ctx.has_bias = act, x.shape, b is not None
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        if ctx.act:
            dy2 = K.bias_act_bwd(pre, None, dy2, ctx.act)
        dx = G.gemm(dy2, w, b_layout="kn")
        dw = G.gemm(dy2, x2, a_layout="km", b_layout="kn")
        db = K.column_sum(dy2).to(dy.dtype) if ctx.has_bias else None
        return dx.reshape(ctx.shape), dw, db, None


def fused_linear_act(x, w, b=None, act=0):
    """act: 0 none, 1 gelu, 2 gelu_tanh, 3 relu."""
    native = x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0
    if native:
        return _FusedLinearAct.apply(x.contiguous(), w, b, act)
    y = torch.nn.functional.linear(x, w, b)
    return G._act_ref(y, act) if act else y


class FusedMLP(torch.nn.Module):
    def __init__(self, in_features, hidden_features, out_features, hidden_dropout_rate=None, out_dropout_rate=0.0,
                 skip_final_activation=False, device=None, dtype=None, placement=None, sbp=None):
        super().__init__()
        dims = [in_features] + list(hidden_features) + [out_features]
        self.skip_final_activation = skip_final_activation
        self.hidden_dropout_rate = list(hidden_dropout_rate) if hidden_dropout_rate else [0.0] * len(hidden_features)
        self.out_dropout_rate = out_dropout_rate
        self.weights = torch.nn.ParameterList()
        self.biases = torch.nn.ParameterList()
        for i in range(len(dims) - 1):
            lin = torch.nn.Linear(dims[i], dims[i + 1], device=device, dtype=dtype)
            self.weights.append(lin.weight)
            self.biases.append(lin.bias)
        if placement is not None:
            self.to_global(placement, sbp)

    def weight(self, i):
        return self.weights[i]

    def bias(self, i):
        return self.biases[i]

    def forward(self, x):
        n = len(self.weights)
        rates = list(self.hidden_dropout_rate) + [self.out_dropout_rate]
        if not self.training or not any(rates):
            # no dropout between the layers: the whole stack is one chain whose hidden activations are private to it
            from ...framework import fused_ops
            return fused_ops.mlp_chain(x, list(self.weights), list(self.biases), act="relu",
                                       skip_final_activation=self.skip_final_activation)
        for i in range(n):
            last = i == n - 1
            act = 0 if (last and self.skip_final_activation) else 3
            x = fused_linear_act(x, self.weights[i], self.biases[i], act)
            rate = self.out_dropout_rate if last else self.hidden_dropout_rate[i]
            if rate and self.training:
                x = torch.nn.functional.dropout(x, rate, True)
        return x
