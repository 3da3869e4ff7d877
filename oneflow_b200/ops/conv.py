"""Convolution on NHWC bf16 tensors: implicit GEMM on tcgen05 (csrc/kernels/conv_igemm.cu) for R x S filters with
stride 1 and "same" padding, the plain GEMM for 1 x 1 filters, and thin data-movement kernels for stride 2
(csrc/kernels/conv_aux.cu). Weights are [Cout, R, S, Cin]. CPU tensors take a PyTorch fp32 statement of the same
maths, which is also what the tests compare the kernels against.

Reference: oneflow/user/kernels/conv_cudnn_kernels.cpp (fprop / dgrad / wgrad through cuDNN),
oneflow/user/ops/conv_op.cpp (shape rules).
"""
from __future__ import annotations

from ctypes import c_int

import torch
import torch.nn.functional as F

from . import gemm as G
from . import kernels as K
from ._native import check, ptr, stream_ptr


def _lib():
    from . import _native
    return _native.kernels()


def _igemm_ok(x, w):
    Cout, R, S, Cin = w.shape
    return x.is_cuda and x.dtype == torch.bfloat16 and Cin % 64 == 0 and Cout % 64 == 0 and R % 2 == 1 and S % 2 == 1 and R <= 7


def _ref_conv(x, w, stride=1):
    Cout, R, S, Cin = w.shape
    y = F.conv2d(x.float().permute(0, 3, 1, 2), w.float().permute(0, 3, 1, 2), stride=stride, padding=((R - 1) // 2, (S - 1) // 2))
    return y.permute(0, 2, 3, 1).contiguous()


def conv_fprop(x, w):
    """x [N, H, W, Cin], w [Cout, R, S, Cin] -> y [N, H, W, Cout]; stride 1, padding (R-1)/2."""
    N, H, W, Cin = x.shape
    Cout, R, S, _ = w.shape
    if R == 1 and S == 1:
        return G.gemm(x.reshape(-1, Cin), w.reshape(Cout, Cin)).view(N, H, W, Cout)
    if not _igemm_ok(x, w):
        if x.is_cuda:
            raise ValueError("conv_fprop: channels must be multiples of 64 and the filter odd-sized (<= 7) on CUDA")
        return _ref_conv(x, w).to(x.dtype)
    y = torch.empty((N, H, W, Cout), dtype=x.dtype, device=x.device)
    check(_lib().ofb_conv_fprop(ptr(x), ptr(w), ptr(y), c_int(N), c_int(H), c_int(W), c_int(Cin), c_int(Cout), c_int(R), c_int(S),
                                stream_ptr()), "conv_fprop")
    K._count()
    return y


def conv_dgrad(dy, w, residual=None):
    """Gradient of conv_fprop wrt x (+ ``residual`` of the same shape, added in the GEMM epilogue for 1x1 filters)."""
    N, H, W, Cout = dy.shape
    _, R, S, Cin = w.shape
    if R == 1 and S == 1:
        res2d = residual.reshape(-1, Cin) if residual is not None else None
        return G.gemm(dy.reshape(-1, Cout), w.reshape(Cout, Cin), b_layout="kn", residual=res2d).view(N, H, W, Cin)
    if residual is not None:
        return K.bias_mask_scale(conv_dgrad(dy, w), None, None, 1.0, addend=residual)
    if not _igemm_ok(dy, w):
        if dy.is_cuda:
            raise ValueError("conv_dgrad: unsupported shape on CUDA")
        x0 = torch.zeros((N, H, W, Cin), requires_grad=True)
        _ref_conv(x0, w).backward(dy.float())
        return x0.grad.to(dy.dtype)
    dx = torch.empty((N, H, W, Cin), dtype=dy.dtype, device=dy.device)
    check(_lib().ofb_conv_dgrad(ptr(dy), ptr(w), ptr(dx), c_int(N), c_int(H), c_int(W), c_int(Cin), c_int(Cout), c_int(R), c_int(S),
                                stream_ptr()), "conv_dgrad")
    K._count()
    return dx


def conv_wgrad(x, dy, filter_hw, out=None, accumulate=False):
    """Gradient of conv_fprop wrt w as fp32 [Cout, R, S, Cin] (added to ``out`` when ``accumulate``)."""
    N, H, W, Cin = x.shape
    Cout = dy.shape[-1]
    R, S = filter_hw
    if out is None:
        out = torch.empty((Cout, R, S, Cin), dtype=torch.float32, device=x.device)
        accumulate = False
    if R == 1 and S == 1:
        G.gemm(dy.reshape(-1, Cout), x.reshape(-1, Cin), a_layout="km", b_layout="kn", out=out.view(Cout, Cin), out_dtype=torch.float32,
               accumulate=accumulate)
        return out
    if not (x.is_cuda and x.dtype == torch.bfloat16 and Cin % 64 == 0 and Cout % 64 == 0):
        if x.is_cuda:
            raise ValueError("conv_wgrad: unsupported shape on CUDA")
        w0 = torch.zeros((Cout, R, S, Cin), requires_grad=True)
        _ref_conv(x, w0).backward(dy.float())
        if accumulate:
            out += w0.grad
        else:
            out.copy_(w0.grad)
        return out
    check(_lib().ofb_conv_wgrad(ptr(x), ptr(dy), ptr(out), c_int(N), c_int(H), c_int(W), c_int(Cin), c_int(Cout), c_int(R), c_int(S),
                                c_int(int(accumulate)), stream_ptr()), "conv_wgrad")
    K._count()
    return out
