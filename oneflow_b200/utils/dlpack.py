"""Zero-copy exchange through DLPack (reference: python/oneflow/utils/dlpack.py); tensors here are torch tensors."""
from torch.utils.dlpack import from_dlpack, to_dlpack  # noqa: F401
