"""``flow.multiprocessing``: torch.multiprocessing (tensors cross process boundaries through shared memory) plus
the reference's clean-up hook (reference: python/oneflow/multiprocessing/__init__.py:75-100)."""
from torch.multiprocessing import *  # noqa: F401,F403
import torch.multiprocessing as _mp


def unlink_all_shared_memory():
    """Shared-memory segments are reference counted and unlinked by their owners here; nothing is left to remove."""
    return None


def __getattr__(name):
    return getattr(_mp, name)
