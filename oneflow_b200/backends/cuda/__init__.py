"""``flow.backends.cuda.matmul``: precision switches of the library GEMM path
(reference: python/oneflow/backends/cuda/__init__.py:20-41).  The tcgen05 kernels of this package are bf16 with fp32
accumulation whatever these say; the switches govern fp32 / fp16 matmuls that go to cuBLAS."""
import torch


class cuMatmulMode:
    def __getattr__(self, name):
        if name in ("allow_tf32", "allow_fp16_reduced_precision_reduction", "allow_bf16_reduced_precision_reduction"):
            return getattr(torch.backends.cuda.matmul, name)
        raise AssertionError("Unknown attribute " + name)

    def __setattr__(self, name, value):
        if name in ("allow_tf32", "allow_fp16_reduced_precision_reduction", "allow_bf16_reduced_precision_reduction"):
            return setattr(torch.backends.cuda.matmul, name, bool(value))
        raise AssertionError("Unknown attribute " + name)


matmul = cuMatmulMode()


def __getattr__(name):
    return getattr(torch.backends.cuda, name)
