"""oneflow_b200 — a Blackwell-native deep-learning framework with the OneFlow API.

``import oneflow_b200 as flow`` (or ``import oneflow as flow`` through the alias package in this
repository). Local tensors are torch tensors; ``to_global(placement, sbp)`` gives global tensors whose ops
dispatch through SBP rules and boxing; ``nn.Graph`` provides the static-graph training contract;
hot paths run hand-written sm_100a kernels (``oneflow_b200/csrc``).
Any attribute not defined here resolves to the torch function of the same name.
"""
import atexit as _atexit

import torch as _torch

__version__ = "0.1.0+b200"

from . import sbp  # noqa: E402
from .framework.placement import placement  # noqa: E402
from .framework.global_tensor import GlobalTensor, to_global, to_local  # noqa: E402
from .framework import tensor_api as _tensor_api  # noqa: E402
from .framework.tensor_api import (Tensor, arange, empty, eye, from_numpy, full, linspace, ones, rand, randint, randn,  # noqa: E402
                                   randperm, tensor, zeros, zeros_like, ones_like, full_like, empty_like, rand_like,
                                   randn_like, randint_like, logspace, hann_window, normal)
from .framework.check_point import load, save  # noqa: E402
from . import _C, amp, autograd, comm, env, nn, optim, utils  # noqa: E402
from . import distributed, one_embedding, profiler, cuda, backends, mock_torch, framework, models, ops, parallel  # noqa: E402
from . import fx, remat, sysconfig, unittest, version  # noqa: E402

_tensor_api.install_tensor_methods()

device = _tensor_api.device
Size = _torch.Size
Generator = _torch.Generator
manual_seed = _torch.manual_seed
no_grad, enable_grad, set_grad_enabled, inference_mode = (_torch.no_grad, _torch.enable_grad, _torch.set_grad_enabled,
                                                          _torch.inference_mode)
autocast = _torch.autocast
for _n in ("float", "float16", "float32", "float64", "double", "half", "bfloat16", "int8", "int16", "int32", "int64", "int",
           "long", "uint8", "bool", "complex64", "complex128", "char"):
    globals()[_n] = getattr(_torch, _n if _n != "char" else "int8")
del _n
boxing = framework.boxing

_SUBMODULES = ["nn", "nn.functional", "nn.graph", "nn.parallel", "nn.utils", "nn.init", "optim", "optim.lr_scheduler", "comm",
               "env", "sbp", "amp", "autograd", "utils", "utils.data", "distributed", "distributed.launch", "one_embedding",
               "profiler", "cuda", "backends", "mock_torch", "framework", "models", "ops", "parallel", "_C", "remat", "sysconfig",
               "unittest", "asyncs", "hub", "multiprocessing", "fx", "version", "support", "autoprof", "model", "data", "experimental"]

__all__ = ["sbp", "placement", "GlobalTensor", "to_global", "to_local", "Tensor", "tensor", "zeros", "ones", "empty", "full",
           "randn", "rand", "randint", "randperm", "arange", "eye", "linspace", "from_numpy", "save", "load", "nn", "optim",
           "comm", "env", "amp", "autograd", "utils", "distributed", "one_embedding", "profiler", "cuda", "backends",
           "mock_torch", "device", "Size", "Generator", "manual_seed", "no_grad", "enable_grad", "set_grad_enabled",
           "inference_mode", "autocast", "_C", "boxing", "models", "ops", "parallel", "framework"]

from .framework import toplevel_extra as _extra  # noqa: E402

for _n in dir(_extra):
    if not _n.startswith("_") and _n not in ("os", "types", "np", "torch", "F", "builtins_slice", "TensorBuffer") and _n not in globals():
        globals()[_n] = getattr(_extra, _n)
globals()["Generator"] = _extra.Generator
from .cuda.type_tensor import host_types as _host_types  # noqa: E402
globals().update(_host_types())
globals()["slice"] = _extra.slice
globals()["view"] = _extra.view
globals()["repeat"] = _extra.repeat
globals()["expand"] = _extra.expand
globals()["cast"] = _extra.cast
globals()["pad"] = _extra.pad
globals()["gelu"] = _extra.gelu
del _n

from .framework import compat_ops as _compat  # noqa: E402

_compat.install()

env.init()
_atexit.register(env.shutdown)


def __getattr__(name):
    """flow.X for the long tail of tensor functions: the torch function of the same name."""
    if name.startswith("__"):
        raise AttributeError(name)
    if hasattr(_torch, name):
        return getattr(_torch, name)
    raise AttributeError(f"module 'oneflow' has no attribute {name!r}")
