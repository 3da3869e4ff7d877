"""Channels-last (NHWC) layers selected by the environment variable ``ONEFLOW_ENABLE_NHWC=1`` or by
``module.to_memory_format(flow.channels_last)``.

In that mode 4-D activations are laid out ``[N, H, W, C]`` and a convolution weight ``[Cout, kH, kW, Cin/groups]``
(reference: python/oneflow/nn/modules/conv.py:417-423, pooling.py:244-247 and 750-753, batchnorm.py:305-307). An
``[N, H, W, C]`` array permuted to ``[N, C, H, W]`` is exactly a channels-last tensor, so the layers below hand the
library (and the implicit-GEMM convolution of ops/conv.py) such views and no data is rearranged on the way in or out.
"""
from __future__ import annotations

import os

import torch

from . import conv as _conv

__all__ = ["nhwc_enabled", "Conv2d", "MaxPool2d", "AvgPool2d", "BatchNorm2d"]


def nhwc_enabled():
    return os.getenv("ONEFLOW_ENABLE_NHWC") == "1"


def _in(x):        # [N, H, W, C] -> channels-last [N, C, H, W] view
    return x.permute(0, 3, 1, 2)


def _out(y):       # back to [N, H, W, C]
    return y.permute(0, 2, 3, 1)


class _MemoryFormat:
    channel_pos = "channels_first"

    def _set_channel_pos(self, pos):
        self.channel_pos = pos

    def to_memory_format(self, memory_format) -> None:
        """Switches the layout this layer expects: ``flow.channels_last`` ([N, H, W, C]) or
        ``flow.contiguous_format`` ([N, C, H, W])."""
        if memory_format is torch.channels_last:
            self._set_channel_pos("channels_last")
        elif memory_format is torch.contiguous_format:
            self._set_channel_pos("channels_first")


class Conv2d(_MemoryFormat, _conv.Conv2d):
    __doc__ = _conv.Conv2d.__doc__

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.channel_pos = "channels_first"
        if nhwc_enabled():
            self._set_channel_pos("channels_last")

    def _set_channel_pos(self, pos):
        if pos == self.channel_pos:
            return
        w = self.weight.data
        w = w.permute(0, 2, 3, 1) if pos == "channels_last" else w.permute(0, 3, 1, 2)
        self.weight = torch.nn.Parameter(w.contiguous(), requires_grad=self.weight.requires_grad)
        self.channel_pos = pos

    def forward(self, input):
        if self.channel_pos != "channels_last" or input.dim() != 4:
            return super().forward(input)
        return _out(self._conv_forward(_in(input), _in(self.weight), self.bias))

    def extra_repr(self):
        s = super().extra_repr()
        return s + ", channel_pos=channels_last" if self.channel_pos == "channels_last" else s


def _pool(base):
    class _Pool(_MemoryFormat, base):
        __doc__ = base.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self.channel_pos = "channels_last" if nhwc_enabled() else "channels_first"

        def forward(self, input):
            if self.channel_pos != "channels_last" or input.dim() != 4:
                return super().forward(input)
            res = super().forward(_in(input))
            if isinstance(res, tuple):
                return tuple(_out(r) for r in res)
            return _out(res)
    _Pool.__name__ = _Pool.__qualname__ = base.__name__
    return _Pool


MaxPool2d = _pool(torch.nn.MaxPool2d)
AvgPool2d = _pool(torch.nn.AvgPool2d)


class BatchNorm2d(_MemoryFormat, torch.nn.BatchNorm2d):
    __doc__ = torch.nn.BatchNorm2d.__doc__

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.channel_axis = 3 if nhwc_enabled() else 1

    def _set_channel_pos(self, pos):
        self.channel_axis = 3 if pos == "channels_last" else 1

    def _check_input_dim(self, input):
        if input.dim() != 4:
            raise ValueError(f"expected 4D input (got {input.dim()}D input)")

    def forward(self, input):
        if self.channel_axis != 3:
            return super().forward(input)
        return _out(super().forward(_in(input)))
