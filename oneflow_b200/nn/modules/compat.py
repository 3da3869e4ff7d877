"""Small ``flow.nn`` modules that torch.nn has no equivalent of: activations, RMSLayerNorm, the eager all-reduce
module, partial-FC sampling as a module, and the quantisation-aware convolutions."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import functional as F
from ..extra_modules import FakeQuantization, MinMaxObserver, MovingAverageMinMaxObserver
from .partial_fc import distributed_partial_fc_sample


class QuickGELU(nn.Module):
    """``x * sigmoid(1.702 * x)`` (reference: python/oneflow/nn/modules/activation.py, QuickGELU)."""

    def forward(self, x):
        return F.quick_gelu(x)


class SquareReLU(nn.Module):
    """``relu(x) ** 2`` (reference: python/oneflow/nn/modules/activation.py, SquareReLU)."""

    def forward(self, x):
        return F.square_relu(x)


class RMSLayerNorm(nn.Module):
    """T5-style layer norm: scale by the root mean square of the last axis, no mean subtraction, no bias
    (reference: python/oneflow/nn/modules/normalization.py:351-395)."""

    def __init__(self, hidden_size, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states):
        from ..._C import rms_layer_norm
        return rms_layer_norm(hidden_states, self.weight, self.variance_epsilon)


class AllReduce(nn.Module):
    """Sums a CUDA tensor over the ranks of a parallel description such as ``"cuda:0-3"`` or a list of ranks
    (reference: python/oneflow/nn/modules/all_reduce.py:22-33).  The sum runs as the peer-memory all-reduce kernel."""

    def __init__(self, parallel_conf_str=None):
        super().__init__()
        self.parallel_conf = parallel_conf_str

    def forward(self, x):
        from ... import comm
        y = x.clone()
        comm.all_reduce(y)
        return y


class DistributedPariticalFCSample(nn.Module):
    """Module form of partial-FC class sampling: ``(mapped_label, sampled_label, sampled_weight)`` for this rank's
    shard of the class weights (reference: python/oneflow/nn/modules/distributed_partial_fc_sample.py:22-40)."""

    def __init__(self, num_sample):
        super().__init__()
        self.num_sample = num_sample

    def forward(self, weight, label):
        return distributed_partial_fc_sample(weight, label, self.num_sample)


class _QatMixin:
    """Fake-quantises the input (moving-average min / max observer) and the weight (min / max observer, per layer or
    per output channel) before the convolution; gradients pass straight through
    (reference: python/oneflow/nn/qat/conv.py:20-60)."""

    def _init_qat(self, quantization_formula, quantization_bit, quantization_scheme, weight_quant_per_layer, input_quant_momentum):
        self.input_min_max_observer = MovingAverageMinMaxObserver(
            stop_update_after_iters=1, quantization_formula=quantization_formula, quantization_bit=quantization_bit,
            quantization_scheme=quantization_scheme, momentum=input_quant_momentum)
        self.register_buffer("current_train_step", torch.zeros(1, dtype=torch.int64))
        self.weight_min_max_observer = MinMaxObserver(
            quantization_formula=quantization_formula, quantization_bit=quantization_bit,
            quantization_scheme=quantization_scheme, per_layer_quantization=weight_quant_per_layer)
        self.fake_quantizer = FakeQuantization(quantization_formula=quantization_formula, quantization_bit=quantization_bit,
                                               quantization_scheme=quantization_scheme)

    def forward(self, x):
        in_scale, in_zp = self.input_min_max_observer(x, self.current_train_step)
        xq = self.fake_quantizer(x, in_scale, in_zp)
        w_scale, w_zp = self.weight_min_max_observer(self.weight)
        wq = self.fake_quantizer(self.weight, w_scale, w_zp)
        return self._conv_forward(xq, wq, self.bias)


def _qat_conv(base, name, ref_lines):
    class _Qat(_QatMixin, base):
        def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                     padding_mode="zeros", quantization_formula="google", quantization_bit=8,
                     quantization_scheme="symmetric", weight_quant_per_layer=True, input_quant_momentum=0.95):
            base.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode)
            self.channel_pos = "channels_first"
            self._init_qat(quantization_formula, quantization_bit, quantization_scheme, weight_quant_per_layer,
                           input_quant_momentum)

    _Qat.__name__ = _Qat.__qualname__ = name
    _Qat.__doc__ = (f"{base.__name__} whose input and weight are fake-quantised for quantisation-aware training "
                    f"(reference: python/oneflow/nn/qat/conv.py:{ref_lines}).")
    return _Qat


QatConv1d = _qat_conv(nn.Conv1d, "QatConv1d", "61-170")
QatConv2d = _qat_conv(nn.Conv2d, "QatConv2d", "173-283")
QatConv3d = _qat_conv(nn.Conv3d, "QatConv3d", "286-396")
