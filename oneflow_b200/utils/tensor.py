"""Zero-copy interop with torch (reference: python/oneflow/utils/tensor/from_or_to_torch_tensor.py).
Local flow tensors already are torch tensors, so both directions are the identity."""


def from_torch(t):
    return t


def to_torch(t):
    from ..framework.global_tensor import GlobalTensor
    return t._local if isinstance(t, GlobalTensor) else t
