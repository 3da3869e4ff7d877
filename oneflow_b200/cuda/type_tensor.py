"""``flow.cuda.HalfTensor`` and friends: legacy typed constructors that build on the current CUDA device
(reference: python/oneflow/cuda/type_tensor.py:18-45)."""
import torch


def _typed(name, dtype, device="cuda"):
    class _T:
        def __new__(cls, *args, **kwargs):
            dev = kwargs.pop("device", device)
            if len(args) == 1 and not isinstance(args[0], (int, torch.Size)):
                return torch.as_tensor(args[0], dtype=dtype, device=dev)
            if not args:
                args = (0,)
            return torch.empty(*args, dtype=dtype, device=dev, **kwargs)

    class _Meta(type):
        def __instancecheck__(cls, obj):
            return isinstance(obj, torch.Tensor) and obj.is_cuda == (device == "cuda") and obj.dtype == dtype

    T = _Meta(name, (_T,), {"dtype": dtype, "is_cuda": device == "cuda"})
    return T


def host_types():
    """The host-side typed constructors (``flow.FloatTensor`` ...): like the CUDA ones they convert whatever data or
    tensor they are given to their dtype."""
    return {n: _typed(n, globals()[n].dtype, "cpu") for n in __all__}


HalfTensor = _typed("HalfTensor", torch.float16)
FloatTensor = _typed("FloatTensor", torch.float32)
DoubleTensor = _typed("DoubleTensor", torch.float64)
BoolTensor = _typed("BoolTensor", torch.bool)
ByteTensor = _typed("ByteTensor", torch.uint8)
CharTensor = _typed("CharTensor", torch.int8)
IntTensor = _typed("IntTensor", torch.int32)
LongTensor = _typed("LongTensor", torch.int64)
ComplexFloatTensor = _typed("ComplexFloatTensor", torch.complex64)
ComplexDoubleTensor = _typed("ComplexDoubleTensor", torch.complex128)
BFloat16Tensor = _typed("BFloat16Tensor", torch.bfloat16)

__all__ = ["HalfTensor", "FloatTensor", "DoubleTensor", "BoolTensor", "ByteTensor", "CharTensor", "IntTensor", "LongTensor",
           "ComplexFloatTensor", "ComplexDoubleTensor", "BFloat16Tensor"]
