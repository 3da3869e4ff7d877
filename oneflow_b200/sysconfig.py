"""``flow.sysconfig``: where the headers and libraries of this build live and how to link against them
(reference: python/oneflow/sysconfig.py:17-36, python/oneflow/framework/sysconfig.py)."""
import os

import torch

_ROOT = os.path.dirname(os.path.abspath(__file__))


def get_include():
    """Directory of the public C++ inference header (``oneflow_api.h``)."""
    return os.path.join(_ROOT, "csrc", "api")


def get_lib():
    """Directory of the built shared libraries."""
    return os.path.join(_ROOT, "lib")


def get_compile_flags():
    return ["-I" + get_include(), "-std=c++17", "-DWITH_CUDA"]


def get_link_flags():
    return ["-L" + get_lib(), "-Wl,-rpath," + get_lib(), "-lofb_api"]


def get_liboneflow_link_flags():
    return get_link_flags()


def with_cuda():
    return True


def get_cuda_version():
    """CUDA version as an integer, 1000 * major + 10 * minor (12080 for 12.8)."""
    v = torch.version.cuda or "0.0"
    major, minor = (int(x) for x in v.split(".")[:2])
    return major * 1000 + minor * 10


def with_rdma():
    return False


def with_mlir():
    return False


def with_mlir_cuda_codegen():
    return False


def has_rpc_backend_grpc():
    return False


def has_rpc_backend_local():
    return True


def cmake_build_type():
    return "Release"
