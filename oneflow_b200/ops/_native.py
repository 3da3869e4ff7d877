"""ctypes bindings of the in-tree native libraries.

``libofb_kernels.so`` holds the hand-written sm_100a CUDA kernels, ``libofb_core.so`` the
C++ runtime pieces (placement/SBP maths, control store, allocator, embedding store, data
readers). Both are built by ``oneflow_b200/build.py`` into ``oneflow_b200/lib`` and loaded
lazily. On a machine with a GPU a missing kernel library is an error, never a silent
fallback to PyTorch ops.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_void_p

_LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
_lock = threading.Lock()
_kernels = None
_core = None


class NativeLibraryError(RuntimeError):
    pass


class GemmArgs(Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p),
        ("bias", c_void_p), ("residual", c_void_p), ("aux_in", c_void_p), ("aux_out", c_void_p),
        ("lda", c_longlong), ("ldb", c_longlong), ("ldc", c_longlong), ("ldr", c_longlong), ("ld_aux", c_longlong),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("a_mn_major", c_int), ("b_mn_major", c_int),
        ("act", c_int), ("out_fp32", c_int), ("accumulate", c_int), ("bn", c_int), ("max_ctas", c_int),
        ("alpha", c_float),
    ]


def lib_path(name: str) -> str:
    return os.path.join(_LIB_DIR, name)


def _load(name: str):
    path = lib_path(name)
    if not os.path.exists(path):
        raise NativeLibraryError(
            f"{path} is missing: run `python -m oneflow_b200.build` (or __graft_entry__.build()) first")
    return ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)


class _ProfiledLibrary:
    """Stands in for the kernel library while a ``flow.profiler.profile`` is active: every exported function is bracketed
    with CUDA events on the current stream and a host timer, and reported to the recorder together with the tensors that
    ``ptr()`` converted for the call (their shapes and bytes)."""

    def __init__(self, lib, recorder):
        self._lib, self._rec = lib, recorder

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("ofb_") or name in ("ofb_last_error", "ofb_read_status") or name.endswith(("_floats", "_parts", "_max_cols")):
            return fn
        rec = self._rec

        def call(*args):
            return rec.native_call(name, fn, args)
        call.__name__ = name
        return call


_recorder = None     # set by flow.profiler.profile while it is active


def set_recorder(rec):
    global _recorder
    _recorder = rec


def kernels():
    """The CUDA kernel library (raises NativeLibraryError when it was not built)."""
    global _kernels
    if _recorder is not None and _kernels is not None:
        return _ProfiledLibrary(_kernels, _recorder)
    if _kernels is None:
        with _lock:
            if _kernels is None:
                lib = _load("libofb_kernels.so")
                lib.ofb_last_error.restype = c_char_p
                lib.ofb_gemm_bf16.argtypes = [POINTER(GemmArgs), c_void_p]
                lib.ofb_gemm_bf16.restype = c_int
                _kernels = lib
    return _kernels


def core():
    """The C++ runtime library."""
    global _core
    if _core is None:
        with _lock:
            if _core is None:
                lib = _load("libofb_core.so")
                lib.ofc_last_error.restype = c_char_p
                _core = lib
    return _core


def kernels_available() -> bool:
    return os.path.exists(lib_path("libofb_kernels.so"))


def core_available() -> bool:
    return os.path.exists(lib_path("libofb_core.so"))


def check(rc: int, what: str = "native call") -> None:
    if rc != 0:
        msg = kernels().ofb_last_error()
        raise NativeLibraryError(f"{what} failed: {msg.decode() if msg else 'unknown error'}")


def read_status(clear: bool = True):
    """Returns (code, detail) of the device status block that kernels with bounded waits write
    when they give up. Synchronises the device."""
    code, detail = c_int(0), c_int(0)
    check(kernels().ofb_read_status(1 if clear else 0, ctypes.byref(code), ctypes.byref(detail)), "read_status")
    return code.value, detail.value


def stream_ptr():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    if _recorder is not None and t is not None:
        _recorder.saw_tensor(t)
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)
