"""``flow.version``: version string, CUDA toolkit the kernels were built for, source revision
(reference: python/oneflow/version.py, generated at build time)."""
import torch as _torch

__version__ = "0.1.0+b200"
cuda = _torch.version.cuda
git_commit = "unknown"
