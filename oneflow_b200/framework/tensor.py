"""``oneflow.framework.tensor``: the import path of the tensor classes
(reference: python/oneflow/framework/tensor.py:24-25).  Tensor methods are installed by ``framework.tensor_api``."""
from .tensor_api import Tensor  # noqa: F401

TensorTuple = tuple


def register_tensor_op(op_name):
    """Decorator that publishes a function as the tensor method ``op_name`` (local and global tensors alike)."""
    import torch

    def deco(fn):
        setattr(torch.Tensor, op_name, fn)
        return fn
    return deco
