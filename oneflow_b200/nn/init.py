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
