"""Stand-ins for the classes the reference's C extension exposes and that appear by name in pickled
checkpoints: ``oneflow._oneflow_internal.dtype`` (state: DataType enum int), ``.placement`` (state:
{"type", "ranks"}) and ``.sbp.sbp`` (state: ("S", axis) | ("B", -1) | ("P", -1)).
Reference: oneflow/api/python/framework/dtype.cpp:37-44, symbol/placement_symbol.cpp,
symbol/sbp_symbol.cpp:62-106."""
import sys
import types

import torch

from oneflow_b200.framework import dtype as _D
from oneflow_b200.framework.placement import placement as _Placement
from oneflow_b200 import sbp as _S


class dtype:
    __slots__ = ("enum",)

    def __init__(self, enum=2):
        self.enum = enum

    @classmethod
    def of(cls, torch_dtype):
        return cls(_D.ENUM_OF[torch_dtype])

    @property
    def torch_dtype(self):
        return _D.DTYPE_OF_ENUM[self.enum]

    def __getstate__(self):
        return self.enum

    def __setstate__(self, state):
        self.enum = int(state)

    def __eq__(self, other):
        if isinstance(other, dtype):
            return self.enum == other.enum
        if isinstance(other, torch.dtype):
            return self.torch_dtype == other
        return NotImplemented

    def __hash__(self):
        return hash(self.enum)

    def __repr__(self):
        return "oneflow." + str(self.torch_dtype).split(".")[-1]


class placement(_Placement):
    @classmethod
    def of(cls, p):
        return cls(p.type, p.ranks.tolist())


sbp = types.ModuleType("oneflow._oneflow_internal.sbp")


class _sbp:
    __slots__ = ("kind", "axis")

    def __init__(self, kind="B", axis=-1):
        self.kind, self.axis = kind, axis

    @classmethod
    def of(cls, s):
        return cls(s.kind, s.axis)

    def to_sbp(self):
        return _S.sbp(self.kind, self.axis)

    def __getstate__(self):
        return (self.kind, self.axis)

    def __setstate__(self, state):
        self.kind, self.axis = state[0], int(state[1])

    def __repr__(self):
        return repr(self.to_sbp())


_sbp.__name__ = _sbp.__qualname__ = "sbp"
_sbp.__module__ = "oneflow._oneflow_internal.sbp"
sbp.sbp = _sbp
sys.modules["oneflow._oneflow_internal.sbp"] = sbp
dtype.__module__ = "oneflow._oneflow_internal"
placement.__module__ = "oneflow._oneflow_internal"


# ------------------------------------------------------------------------------------------------ runtime hooks
# Entry points of the C extension that user code and tests call directly.


def _ns(name, **members):
    m = types.ModuleType(f"oneflow._oneflow_internal.{name}")
    m.__dict__.update(members)
    sys.modules[m.__name__] = m
    return m


def _sync():
    """Wait for everything queued on the current device (the reference drains its virtual machine)."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def _cuda_version():
    v = torch.version.cuda or "0.0"
    major, minor = (int(x) for x in v.split(".")[:2])
    return major * 1000 + minor * 10


flags = _ns("flags", with_cuda=lambda: True, cuda_version=_cuda_version, with_mlir=lambda: False,
            with_mlir_cuda_codegen=lambda: False, with_rdma=lambda: False, has_rpc_backend_grpc=lambda: False,
            has_rpc_backend_local=lambda: True, cmake_build_type=lambda: "Release", use_cxx11_abi=lambda: True)
eager = _ns("eager", Sync=_sync, ClusterSync=_sync)
eager.multi_client = _ns("eager.multi_client", Sync=_sync)


# Exception types of the C extension: the builtin ones, so that ``except RuntimeError`` and
# ``except oneflow._oneflow_internal.exception.RuntimeError`` catch the same errors.
exception = _ns("exception", Exception=Exception, RuntimeError=RuntimeError, ValueError=ValueError, TypeError=TypeError,
                IndexError=IndexError, NotImplementedError=NotImplementedError, CheckFailedError=RuntimeError,
                InvalidValueError=ValueError, UnimplementedError=NotImplementedError)


def max_alignment_size():
    return 512


def default_generator(device="cpu"):
    return torch.default_generator if str(device) == "cpu" else torch.cuda.default_generators[torch.cuda.current_device()]


def GetEnvContext(*args, **kwargs):
    from oneflow_b200 import env
    return env


def CurrentMachineId():
    from oneflow_b200 import env
    return env.get_node_size() - 1 if False else 0


class TensorTuple(list):
    """The reference's container for several tensors crossing into C++; a list here."""

    def __init__(self, items=()):
        super().__init__(items)

