"""``flow.nn.init``: torch.nn.init (the in-place initialisers work on global tensors through the dispatch)."""
from torch.nn.init import *  # noqa: F401,F403
import torch.nn.init as _I


def __getattr__(name):
    return getattr(_I, name)


def get_data_format(data_format):
    """``"NC..."`` -> ``"channels_first"``, ``"N...C"`` -> ``"channels_last"``, ``""`` -> ``""``
    (reference: python/oneflow/ops/util/initializer_util.py:39-49)."""
    if not isinstance(data_format, str):
        raise TypeError("data_format must be a string")
    if data_format.startswith("NC"):
        return "channels_first"
    if data_format.startswith("N") and data_format.endswith("C"):
        return "channels_last"
    if data_format != "":
        raise ValueError('data_format must be "N...C" or "NC..." or ""')
    return ""


def calc_fan(shape, mode, data_format):
    """Fan-in, fan-out or their sum of a weight of ``shape`` (out channels first) for ``mode`` in ``fan_in`` /
    ``fan_out`` / ``fan_sum`` (reference: python/oneflow/ops/util/initializer_util.py:52-81)."""
    if len(shape) < 2:
        raise ValueError("fan in and fan out need a tensor of at least 2 dimensions")
    fan_in = 1.0
    for d in shape[1:]:
        fan_in *= d
    fan_out = float(shape[0])
    if len(shape) > 2:
        if data_format == "channels_first":
            spatial = shape[2:]
        elif data_format == "channels_last":
            spatial = shape[1:-1]
        else:
            raise NotImplementedError("only 'channels_first' and 'channels_last' data formats are supported")
        for d in spatial:
            fan_out *= d
    if mode == "fan_sum":
        return fan_in + fan_out
    if mode == "fan_in":
        return fan_in
    if mode == "fan_out":
        return fan_out
    raise NotImplementedError("only 'fan_in', 'fan_out' and 'fan_sum' modes are supported")


def _nhwc_aware(fn):
    """The fan-based initialisers read a 4-D weight as [Cout, kH, kW, Cin] while ``ONEFLOW_ENABLE_NHWC=1`` (or with
    ``data_format="NHWC"``): they then run on the [Cout, Cin, kH, kW] view of the same memory
    (reference: python/oneflow/nn/init.py:141-142, 204-205, 246-247)."""
    import functools
    import os

    @functools.wraps(fn)
    def init(tensor, *args, data_format="NCHW", **kwargs):
        if tensor.dim() == 4 and (os.getenv("ONEFLOW_ENABLE_NHWC") == "1" or get_data_format(data_format) == "channels_last"):
            fn(tensor.permute(0, 3, 1, 2), *args, **kwargs)
            return tensor
        return fn(tensor, *args, **kwargs)
    return init


xavier_uniform_, xavier_normal_ = _nhwc_aware(_I.xavier_uniform_), _nhwc_aware(_I.xavier_normal_)
kaiming_uniform_, kaiming_normal_ = _nhwc_aware(_I.kaiming_uniform_), _nhwc_aware(_I.kaiming_normal_)
