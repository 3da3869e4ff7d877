"""Layers of the reference that torch.nn does not provide."""
from __future__ import annotations

import math

import torch
import torch.nn as nn


class CombinedMarginLoss(nn.Module):
    """ArcFace / CosFace / SphereFace margins on cosine logits: cos(m1*theta + m2) - m3 on the label column
    (reference: python/oneflow/nn/modules/loss.py CombinedMarginLoss, combined_margin_loss_kernel.cu)."""

    def __init__(self, m1: float = 1.0, m2: float = 0.0, m3: float = 0.0):
        super().__init__()
        self.m1, self.m2, self.m3 = m1, m2, m3

    def forward(self, x, label):
        onehot = torch.nn.functional.one_hot(label.long(), x.shape[-1]).bool()
        theta = torch.acos(x.clamp(-1 + 1e-7, 1 - 1e-7))
        target = torch.cos(self.m1 * theta + self.m2) - self.m3
        return torch.where(onehot, target, x)


class FusedBatchNorm1d(nn.BatchNorm1d):
    """BatchNorm(+add)(+ReLU) in one module (reference: FusedBatchNorm*, cudnn_fused_normalization_add_relu)."""

    def forward(self, x, addend=None):
        y = super().forward(x)
        if addend is not None:
            y = y + addend
        return torch.relu(y)


class FusedBatchNorm2d(nn.BatchNorm2d):
    def forward(self, x, addend=None):
        y = super().forward(x)
        if addend is not None:
            y = y + addend
        return torch.relu(y)


class FusedBatchNorm3d(nn.BatchNorm3d):
    def forward(self, x, addend=None):
        y = super().forward(x)
        if addend is not None:
            y = y + addend
        return torch.relu(y)


def _qparams(mn, mx, bits, scheme, formula):
    if formula == "google":
        if scheme == "symmetric":
            denom = 2.0 ** (bits - 1) - 1
            scale = torch.maximum(mn.abs(), mx.abs()) / denom
            zp = torch.zeros_like(scale)
        else:
            denom = 2.0 ** bits - 1
            scale = (mx - mn) / denom
            zp = -torch.round(mn / scale)
    else:  # cambricon: power-of-two shift
        scale = torch.floor(torch.log2(torch.maximum(mn.abs(), mx.abs()))) - (bits - 2)
        zp = torch.zeros_like(scale)
    return scale, zp


class MinMaxObserver(nn.Module):
    """Computes quantisation scale / zero-point from the min and max of a tensor
    (reference: python/oneflow/nn/modules/min_max_observer.py, min_max_observer_kernel.cu)."""

    def __init__(self, quantization_formula="google", quantization_bit=8, quantization_scheme="symmetric",
                 per_layer_quantization=True):
        super().__init__()
        self.formula, self.bits, self.scheme, self.per_layer = quantization_formula, quantization_bit, quantization_scheme, per_layer_quantization

    def forward(self, x):
        if self.per_layer:
            mn, mx = x.min().reshape(1), x.max().reshape(1)
        else:
            flat = x.reshape(x.shape[0], -1)
            mn, mx = flat.min(1).values, flat.max(1).values
        return _qparams(mn, mx, self.bits, self.scheme, self.formula)


class MovingAverageMinMaxObserver(nn.Module):
    def __init__(self, stop_update_after_iters=1, quantization_formula="google", quantization_bit=8,
                 quantization_scheme="symmetric", momentum=0.95):
        super().__init__()
        self.stop, self.formula, self.bits, self.scheme, self.momentum = stop_update_after_iters, quantization_formula, quantization_bit, quantization_scheme, momentum
        self.register_buffer("moving_max", torch.zeros(1))
        self.register_buffer("moving_min", torch.zeros(1))

    def forward(self, x, current_train_step):
        step = int(torch.as_tensor(current_train_step).reshape(-1)[0])
        if self.training and step <= self.stop:
            mn, mx = x.min().reshape(1), x.max().reshape(1)
            if step == 0:
                self.moving_min.copy_(mn)
                self.moving_max.copy_(mx)
            else:
                self.moving_min.mul_(self.momentum).add_(mn * (1 - self.momentum))
                self.moving_max.mul_(self.momentum).add_(mx * (1 - self.momentum))
        return _qparams(self.moving_min, self.moving_max, self.bits, self.scheme, self.formula)


class FakeQuantization(nn.Module):
    """Quantise-dequantise with a straight-through gradient (fake_quantization_kernel.cu)."""

    def __init__(self, quantization_formula="google", quantization_bit=8, quantization_scheme="symmetric"):
        super().__init__()
        self.formula, self.bits, self.scheme = quantization_formula, quantization_bit, quantization_scheme

    def forward(self, x, scale, zero_point):
        shape = [-1] + [1] * (x.dim() - 1) if scale.numel() > 1 else [1]
        s, z = scale.reshape(shape), zero_point.reshape(shape)
        if self.formula == "google":
            if self.scheme == "symmetric":
                hi = 2.0 ** (self.bits - 1) - 1
                q = torch.clamp(torch.round(x / s), -hi, hi) * s
            else:
                hi = 2.0 ** self.bits - 1
                q = (torch.clamp(torch.round(x / s + z), 0, hi) - z) * s
        else:
            hi = 2.0 ** (self.bits - 1) - 1
            sc = 2.0 ** s
            q = torch.clamp(torch.round(x / sc), -hi, hi) * sc
        return x + (q - x).detach()


class Quantization(FakeQuantization):
    """Quantise only (integers carried in the input dtype)."""

    def forward(self, x, scale, zero_point):
        shape = [-1] + [1] * (x.dim() - 1) if scale.numel() > 1 else [1]
        s, z = scale.reshape(shape), zero_point.reshape(shape)
        if self.scheme == "symmetric":
            hi = 2.0 ** (self.bits - 1) - 1
            return torch.clamp(torch.round(x / s), -hi, hi)
        return torch.clamp(torch.round(x / s + z), 0, 2.0 ** self.bits - 1)
