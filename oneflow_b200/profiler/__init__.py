"""``flow.profiler``: ``profile(activities, record_shapes, ...)`` context manager, ``record_function`` and
``key_averages()`` tables on top of torch.profiler (kineto/CUPTI), NVTX ranges for device timelines, and a
CUDA-event kernel timer. Reference: python/oneflow/profiler/profiler.py:42-117, core/profiler/*."""
import contextlib

import torch
from torch.profiler import ProfilerActivity, record_function  # noqa: F401


class ProfilerActivityAlias:
    CPU = ProfilerActivity.CPU
    CUDA = ProfilerActivity.CUDA


def profile(activities=None, record_shapes=False, record_attrs=False, record_bandwidth_for_cuda=False, **kwargs):
    if activities is None:
        activities = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    return torch.profiler.profile(activities=activities, record_shapes=record_shapes or record_attrs, **kwargs)


@contextlib.contextmanager
def nvtx_range(name):
    """Device-timeline range (the reference's nvtx_start / nvtx_end ops, user/kernels/nvtx_range_kernel.cu)."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class CudaTimer:
    """CUDA-event timing on the current stream: ``with CudaTimer() as t: ...; t.ms``."""

    def __enter__(self):
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self.e0.record()
        return self

    def __exit__(self, *exc):
        self.e1.record()
        torch.cuda.synchronize()
        self.ms = self.e0.elapsed_time(self.e1)
        return False


from torch.profiler import ProfilerAction, tensorboard_trace_handler  # noqa: E402,F401


def range_push(range_name):
    """Open an NVTX range on the calling thread (reference: python/oneflow/profiler/__init__.py:40-45)."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(range_name)


def range_pop():
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def profiler_start():
    """Start the CUDA profiler's capture window (``cudaProfilerStart``), for tools run with a capture range."""
    if torch.cuda.is_available():
        torch.cuda.profiler.start()


def profiler_stop():
    if torch.cuda.is_available():
        torch.cuda.profiler.stop()


def kineto_available():
    return torch.autograd.kineto_available()
