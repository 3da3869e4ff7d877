"""Batch norm (+ residual add + ReLU), pooling and stride-2 helpers on NHWC bf16 tensors
(csrc/kernels/conv_aux.cu), each with a PyTorch fp32 statement for CPU tensors.

Reference: oneflow/user/kernels/normalization_kernel.cu, max_pool / avg_pool kernels, python/oneflow/nn/modules/batchnorm.py.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch
import torch.nn.functional as F

from . import kernels as K
from ._native import check, ptr, stream_ptr


def _lib():
    from . import _native
    return _native.kernels()


# ------------------------------------------------------------------------------------------------ batch norm
def bn_train_fwd(x, gamma, beta, residual=None, relu=False, eps=1e-5, momentum=0.1, running_mean=None, running_var=None):
    """x [..., C] bf16; gamma / beta fp32 [C]. Returns (y, mean, rstd) with batch statistics over all leading dims."""
    C = x.shape[-1]
    rows = x.numel() // C
    if not x.is_cuda:
        xf = x.float().reshape(rows, C)
        mean = xf.mean(0)
        var = xf.var(0, unbiased=False)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean) * rstd * gamma + beta
        if residual is not None:
            y = y + residual.float().reshape(rows, C)
        if relu:
            y = torch.relu(y)
        if running_mean is not None:
            running_mean.mul_(1 - momentum).add_(mean, alpha=momentum)
            running_var.mul_(1 - momentum).add_(var * (rows / max(rows - 1, 1)), alpha=momentum)
        return y.to(x.dtype).view(x.shape), mean, rstd
    sums = torch.zeros(2 * C, dtype=torch.float32, device=x.device)
    stats = torch.empty(4, C, dtype=torch.float32, device=x.device)
    mean, rstd, scale, shift = stats[0], stats[1], stats[2], stats[3]
    y = torch.empty_like(x)
    lib = _lib()
    check(lib.ofb_bn_reduce(c_int(0), ptr(x), None, None, None, None, c_longlong(rows), c_int(C), c_int(0), ptr(sums), stream_ptr()),
          "bn_reduce")
    check(lib.ofb_bn_finalize(ptr(sums), c_longlong(rows), c_float(eps), c_float(momentum), c_int(C), ptr(gamma), ptr(beta), ptr(mean),
                              ptr(rstd), ptr(scale), ptr(shift), ptr(running_mean), ptr(running_var), stream_ptr()), "bn_finalize")
    check(lib.ofb_bn_apply(ptr(x), ptr(residual), ptr(scale), ptr(shift), c_longlong(rows), c_int(C), c_int(int(relu)), ptr(y),
                           stream_ptr()), "bn_apply")
    K._count(3)
    return y, mean, rstd


def bn_eval_fwd(x, gamma, beta, running_mean, running_var, residual=None, relu=False, eps=1e-5):
    C = x.shape[-1]
    rows = x.numel() // C
    rstd = torch.rsqrt(running_var.float() + eps)
    if not x.is_cuda:
        y = (x.float() - running_mean) * rstd * gamma + beta
        if residual is not None:
            y = y + residual.float()
        return (torch.relu(y) if relu else y).to(x.dtype)
    y = torch.empty_like(x)
    scale = (gamma.float() * rstd).contiguous()
    shift = (beta.float() - running_mean.float() * scale).contiguous()
    check(_lib().ofb_bn_apply(ptr(x), ptr(residual), ptr(scale), ptr(shift), c_longlong(rows), c_int(C), c_int(int(relu)), ptr(y),
                              stream_ptr()), "bn_apply")
    K._count()
    return y


def bn_train_bwd(dy, x, y, mean, rstd, gamma, relu=False, want_residual_grad=False):
    """Returns (dx, d_residual or None, dgamma, dbeta); y is only read when relu."""
    C = x.shape[-1]
    rows = x.numel() // C
    if not x.is_cuda:
        g = dy.float().reshape(rows, C)
        if relu:
            g = g * (y.float().reshape(rows, C) > 0)
        xhat = (x.float().reshape(rows, C) - mean) * rstd
        s1, s2 = g.sum(0), (g * xhat).sum(0)
        dx = gamma * rstd * (g - s1 / rows - xhat * s2 / rows)
        return dx.to(x.dtype).view(x.shape), (g.to(x.dtype).view(x.shape) if want_residual_grad else None), s2, s1
    sums = torch.zeros(2 * C, dtype=torch.float32, device=x.device)
    coef = torch.empty(3 * C, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x)
    dres = torch.empty_like(x) if want_residual_grad else None
    lib = _lib()
    dy = dy.contiguous()
    check(lib.ofb_bn_reduce(c_int(1), ptr(dy), ptr(x), ptr(y), ptr(mean), ptr(rstd), c_longlong(rows), c_int(C), c_int(int(relu)), ptr(sums),
                            stream_ptr()), "bn_reduce")
    check(lib.ofb_bn_bwd_apply(ptr(dy), ptr(x), ptr(y), ptr(mean), ptr(rstd), ptr(gamma), ptr(sums), ptr(coef), c_longlong(rows), c_int(C),
                               c_int(int(relu)), ptr(dx), ptr(dres), stream_ptr()), "bn_bwd_apply")
    K._count(2)
    return dx, dres, sums[C:], sums[:C]


# ------------------------------------------------------------------------------------------------ pooling
def maxpool3x3s2_fwd(x):
    """x [N, H, W, C] -> (y [N, ceil(H/2), ceil(W/2), C], idx uint8 of the winning tap)."""
    N, H, W, C = x.shape
    OH, OW = (H + 1) // 2, (W + 1) // 2
    if not x.is_cuda:
        y, ind = F.max_pool2d(x.float().permute(0, 3, 1, 2), 3, 2, 1, return_indices=True)
        return y.permute(0, 2, 3, 1).contiguous().to(x.dtype), ind
    y = torch.empty((N, OH, OW, C), dtype=x.dtype, device=x.device)
    idx = torch.empty((N, OH, OW, C), dtype=torch.uint8, device=x.device)
    check(_lib().ofb_maxpool3x3s2_fwd(ptr(x), ptr(y), ptr(idx), c_int(N), c_int(H), c_int(W), c_int(C), stream_ptr()), "maxpool_fwd")
    K._count()
    return y, idx


def maxpool3x3s2_bwd(dy, idx, in_shape):
    N, H, W, C = in_shape
    if not dy.is_cuda:
        g = dy.float().permute(0, 3, 1, 2).reshape(N, C, -1)
        dx = torch.zeros((N, C, H * W)).scatter_add_(2, idx.reshape(N, C, -1), g)      # overlapping windows accumulate
        return dx.view(N, C, H, W).permute(0, 2, 3, 1).contiguous().to(dy.dtype)
    dx = torch.empty(in_shape, dtype=dy.dtype, device=dy.device)
    check(_lib().ofb_maxpool3x3s2_bwd(ptr(dy.contiguous()), ptr(idx), ptr(dx), c_int(N), c_int(H), c_int(W), c_int(C), stream_ptr()),
          "maxpool_bwd")
    K._count()
    return dx


def avgpool_fwd(x):
    N, H, W, C = x.shape
    if not x.is_cuda:
        return x.float().mean((1, 2)).to(x.dtype)
    y = torch.empty((N, C), dtype=x.dtype, device=x.device)
    check(_lib().ofb_avgpool_fwd(ptr(x), ptr(y), c_int(N), c_int(H * W), c_int(C), stream_ptr()), "avgpool_fwd")
    K._count()
    return y


def avgpool_bwd(dy, in_shape):
    N, H, W, C = in_shape
    if not dy.is_cuda:
        return (dy.float() / (H * W))[:, None, None, :].expand(in_shape).contiguous().to(dy.dtype)
    dx = torch.empty(in_shape, dtype=dy.dtype, device=dy.device)
    check(_lib().ofb_avgpool_bwd(ptr(dy.contiguous()), ptr(dx), c_int(N), c_int(H * W), c_int(C), stream_ptr()), "avgpool_bwd")
    K._count()
    return dx


# ------------------------------------------------------------------------------------------------ stride 2
def subsample2(x):
    N, H, W, C = x.shape
    if not x.is_cuda:
        return x[:, ::2, ::2].contiguous()
    y = torch.empty((N, (H + 1) // 2, (W + 1) // 2, C), dtype=x.dtype, device=x.device)
    check(_lib().ofb_subsample2(ptr(x), ptr(y), c_int(N), c_int(H), c_int(W), c_int(C), stream_ptr()), "subsample2")
    K._count()
    return y


def upsample2_zero(dy, in_shape):
    N, H, W, C = in_shape
    if not dy.is_cuda:
        dx = torch.zeros(in_shape, dtype=dy.dtype)
        dx[:, ::2, ::2] = dy
        return dx
    dx = torch.empty(in_shape, dtype=dy.dtype, device=dy.device)
    check(_lib().ofb_upsample2_zero(ptr(dy.contiguous()), ptr(dx), c_int(N), c_int(H), c_int(W), c_int(C), stream_ptr()), "upsample2_zero")
    K._count()
    return dx


def im2col_small(x, R, S, stride, pad, ldc):
    """Patches of a few-channel image as rows of a matrix [N * OH * OW, ldc] (columns (r, s, c), zero padded)."""
    N, H, W, Cin = x.shape
    OH, OW = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    if not x.is_cuda:
        cols = F.unfold(x.float().permute(0, 3, 1, 2), (R, S), padding=pad, stride=stride)          # [N, Cin*R*S, L], (c, r, s) order
        cols = cols.view(N, Cin, R * S, OH * OW).permute(0, 3, 2, 1).reshape(N * OH * OW, R * S * Cin)  # -> (r, s, c)
        out = torch.zeros((N * OH * OW, ldc), dtype=x.dtype)
        out[:, :R * S * Cin] = cols.to(x.dtype)
        return out, (OH, OW)
    cols = torch.empty((N * OH * OW, ldc), dtype=x.dtype, device=x.device)
    check(_lib().ofb_im2col_small(ptr(x), ptr(cols), c_int(N), c_int(H), c_int(W), c_int(Cin), c_int(R), c_int(S), c_int(stride), c_int(pad),
                                  c_int(ldc), stream_ptr()), "im2col_small")
    K._count()
    return cols, (OH, OW)
