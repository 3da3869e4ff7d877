"""``flow.cuda``: device management, synchronisation, seeds and memory statistics (torch.cuda)."""
from torch.cuda import *  # noqa: F401,F403
from torch.cuda import (current_device, current_stream, device_count, empty_cache, is_available, manual_seed,  # noqa: F401
                        manual_seed_all, max_memory_allocated, memory_allocated, memory_reserved, set_device, synchronize)
from .type_tensor import (BFloat16Tensor, BoolTensor, ByteTensor, CharTensor, ComplexDoubleTensor, ComplexFloatTensor,  # noqa: F401,E402
                          DoubleTensor, FloatTensor, HalfTensor, IntTensor, LongTensor)
from torch.cuda import amp, random  # noqa: F401,E402


def __getattr__(name):
    import torch.cuda as _c
    return getattr(_c, name)
