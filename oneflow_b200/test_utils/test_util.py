"""Argument grids and small array helpers of the reference's tests
(reference: python/oneflow/test_utils/test_util.py:27-123)."""
import itertools
import os
from collections import OrderedDict
from collections.abc import Iterable

import numpy as np
import torch


def GenCartesianProduct(sets):
    sets = [list(s) for s in sets]
    if os.getenv("ONEFLOW_TEST_CPU_ONLY") or not torch.cuda.is_available():
        sets = [[v for v in s if v != "cuda"] if "cuda" in s and len(s) > 1 else s for s in sets]
    return itertools.product(*sets)


def GenArgList(arg_dict):
    if not isinstance(arg_dict, OrderedDict) or not all(isinstance(v, list) for v in arg_dict.values()):
        raise TypeError("GenArgList takes an OrderedDict of lists")
    return GenCartesianProduct(arg_dict.values())


def GenArgDict(arg_dict):
    return [dict(zip(arg_dict.keys(), x)) for x in GenArgList(arg_dict)]


class Args:
    def __init__(self, flow_args, tf_args=None):
        self.flow_args = flow_args
        self.tf_args = flow_args if tf_args is None else tf_args

    def __repr__(self):
        return f"flow_args={self.flow_args} tf_args={self.tf_args}"


type_name_to_flow_type = {
    "bool": torch.bool, "float16": torch.float16, "float32": torch.float32, "double": torch.float64, "float64": torch.float64,
    "int8": torch.int8, "int32": torch.int32, "int64": torch.int64, "uint8": torch.uint8, "half": torch.float16,
    "bfloat16": torch.bfloat16, "complex64": torch.complex64, "complex128": torch.complex128,
}
type_name_to_np_type = {
    "float16": np.float16, "float32": np.float32, "double": np.float64, "int8": np.int8, "int32": np.int32, "int64": np.int64,
    "uint8": np.uint8, "complex64": np.complex64, "complex128": np.complex128,
}


def FlattenArray(input_array):
    return [x.tolist() for x in np.nditer(input_array)]


def Array2Numpy(input_array, target_shape):
    return np.array(input_array).reshape(target_shape, order="C")


def Index2Coordinate(idx, tensor_shape):
    return [int(c) for c in np.unravel_index(int(idx), tuple(tensor_shape))]


def Coordinate2Index(coordinate, tensor_shape):
    if len(coordinate) != len(tensor_shape):
        raise ValueError("wrong coordinate or shape")
    return int(np.ravel_multi_index(tuple(coordinate), tuple(tensor_shape)))
