"""dtypes: the flow dtype objects are the torch dtypes; this table adds the reference's DataType enum
values used by the checkpoint format (oneflow/core/common/data_type.proto:4-27)."""
import numpy as np
import torch

# name, torch dtype, DataType enum value, proto name
_TABLE = [
    ("char", torch.int8, 1, "kChar"), ("float32", torch.float32, 2, "kFloat"), ("float64", torch.float64, 3, "kDouble"),
    ("int8", torch.int8, 4, "kInt8"), ("int32", torch.int32, 5, "kInt32"), ("int64", torch.int64, 6, "kInt64"),
    ("uint8", torch.uint8, 7, "kUInt8"), ("float16", torch.float16, 9, "kFloat16"), ("bfloat16", torch.bfloat16, 11, "kBFloat16"),
    ("bool", torch.bool, 12, "kBool"), ("int16", torch.int16, 15, "kInt16"), ("complex64", torch.complex64, 20, "kComplex64"),
    ("complex128", torch.complex128, 21, "kComplex128"),
]
ENUM_OF = {t: e for _, t, e, _ in reversed(_TABLE)}
ENUM_OF[torch.int8] = 4
PROTO_NAME_OF = {t: p for _, t, _, p in reversed(_TABLE)}
PROTO_NAME_OF[torch.int8] = "kInt8"
DTYPE_OF_ENUM = {e: t for _, t, e, _ in _TABLE}
DTYPE_OF_PROTO_NAME = {p: t for _, t, _, p in _TABLE}

_NP = {torch.float32: np.float32, torch.float64: np.float64, torch.float16: np.float16, torch.int8: np.int8,
       torch.int16: np.int16, torch.int32: np.int32, torch.int64: np.int64, torch.uint8: np.uint8, torch.bool: np.bool_,
       torch.complex64: np.complex64, torch.complex128: np.complex128}


def to_numpy_dtype(dt):
    if dt == torch.bfloat16:
        return np.uint16  # raw bits; numpy has no bfloat16
    return _NP[dt]
