"""``flow.nn.Conv2d`` / ``flow.nn.functional.conv2d`` on the implicit-GEMM tcgen05 kernels.

bf16 CUDA tensors in channels-last memory format with a stride-1 "same" convolution (odd filter, padding (k-1)/2,
no groups or dilation, channel counts that are multiples of 64) run forward, input gradient and weight gradient on
ops/conv.py; every other call takes PyTorch's convolution. An NCHW-shaped channels-last tensor *is* an NHWC array,
so no data is rearranged (reference: python/oneflow/nn/modules/conv.py with ONEFLOW_ENABLE_NHWC,
oneflow/user/kernels/conv_cudnn_kernels.cpp)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import conv as C


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def _eligible(x, w, stride, padding, dilation, groups):
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 4 and groups == 1):
        return False
    if _pair(stride) != (1, 1) or _pair(dilation) != (1, 1) or isinstance(padding, str):
        return False
    cout, cin, r, s = w.shape
    if r % 2 == 0 or s % 2 == 0 or r > 7 or s > 7 or _pair(padding) != ((r - 1) // 2, (s - 1) // 2):
        return False
    if cin % 64 or cout % 64:
        return False
    return x.is_contiguous(memory_format=torch.channels_last)


class _ConvNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        xn = x.permute(0, 2, 3, 1).contiguous()          # [N, H, W, C] view of the channels-last tensor (no copy)
        wn = w.permute(0, 2, 3, 1).contiguous()          # [Cout, R, S, Cin]
        y = C.conv_fprop(xn, wn)
        ctx.save_for_backward(xn, wn)
        ctx.wshape = tuple(w.shape)
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        xn, wn = ctx.saved_tensors
        dyn = dy.permute(0, 2, 3, 1).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = C.conv_dgrad(dyn, wn).permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1]:
            r, s = ctx.wshape[2], ctx.wshape[3]
            dw = C.conv_wgrad(xn, dyn, (r, s)).permute(0, 3, 1, 2).to(wn.dtype)
        return dx, dw


def conv2d(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    if _eligible(input, weight, stride, padding, dilation, groups):
        y = _ConvNHWC.apply(input, weight)
        if bias is not None:
            y = y + bias.view(1, -1, 1, 1)
        return y
    return F.conv2d(input, weight, bias, stride, padding, dilation, groups)


class Conv2d(torch.nn.Conv2d):
    def _conv_forward(self, input, weight, bias):
        if self.padding_mode == "zeros" and _eligible(input, weight, self.stride, self.padding, self.dilation, self.groups):
            return conv2d(input, weight, bias, self.stride, self.padding, self.dilation, self.groups)
        return super()._conv_forward(input, weight, bias)
