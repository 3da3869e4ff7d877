"""Small helpers of the reference's harness (python/oneflow/test_utils/automated_test_util/util.py)."""
import os


def broadcast(obj, src=0):
    from .generators import _broadcast_obj
    return _broadcast_obj(obj)


def is_cpu_only():
    import torch
    return bool(os.getenv("ONEFLOW_TEST_CPU_ONLY")) or not torch.cuda.is_available()
