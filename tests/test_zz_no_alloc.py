"""The allocation-free LayerNorm backward (csrc/kernels/ofb_noalloc.h).

Some users of the kernel library cannot allocate device memory when they need this gradient (a server
with a frozen memory pool, a plug-in that only receives raw pointers). For them the library keeps the
scratch in a static device array. This test calls that entry point through its exported C symbol, twice
in a row on different data (the array keeps the first call's leftovers, which must not leak into the
second result), and compares with the regular entry point that takes caller-provided scratch.
The file name sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from oneflow_b200.ops import _native
from oneflow_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _noalloc_bwd(lib, dy, x, gamma, mean, rstd, add, accumulate_into=None, dx=None):
    rows, cols = x.shape
    dx = torch.empty_like(x) if dx is None else dx
    if accumulate_into is None:
        dg = torch.empty(cols, dtype=torch.float32, device=x.device)
        db = torch.empty(cols, dtype=torch.float32, device=x.device)
        acc = 0
    else:
        dg, db = accumulate_into
        acc = 1
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ofb_layer_norm_bwd_noalloc(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(add), _ptr(dx),
                                        _ptr(dg), _ptr(db), c_int(acc), c_int(rows), c_int(cols), stream)
    return rc, dx, dg, db


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    scale = b.abs().max().item() + 1e-6
    assert (a - b).abs().max().item() <= tol * max(1.0, scale)


def test_layer_norm_bwd_noalloc_matches_regular_entry_point_twice():
    lib = ctypes.CDLL(_native.lib_path("libofb_kernels.so"))  # the exported C symbol, not the Python wrapper
    lib.ofb_layer_norm_bwd_noalloc.restype = c_int
    lib.ofb_last_error.restype = ctypes.c_char_p
    assert lib.ofb_layer_norm_bwd_noalloc_max_cols() == 4096
    dev = "cuda"
    for call, (rows, cols, seed) in enumerate([(1500, 4096, 21), (333, 1024, 22)]):
        torch.manual_seed(seed)
        x = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16) * 1.5 + 0.3
        g = torch.randn(cols, device=dev, dtype=torch.bfloat16)
        b = torch.randn(cols, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
        add = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
        _, mean, rstd = K.layer_norm_fwd(x, g, b, 1e-5)
        ref_dx, ref_dg, ref_db = K.layer_norm_bwd(dy, x, g, mean, rstd, add_to_dx=add)
        rc, dx, dg, db = _noalloc_bwd(lib, dy, x, g, mean, rstd, add)
        assert rc == 0, lib.ofb_last_error()
        torch.cuda.synchronize()
        # same kernels, same inputs: the two entry points agree to within the tolerance used for the op
        _close(dx, ref_dx, 2e-2)
        _close(dg, ref_dg, 5e-2)
        _close(db, ref_db, 5e-2)
    # accumulation into existing gradients on a third call; by now the module is loaded and the array's address is
    # known, so the device's free memory must be the same before and after the call (nothing was allocated)
    acc = (dg.clone(), db.clone())
    dx_out = torch.empty_like(x)                      # every output exists before the measurement starts
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    rc, _, dg2, db2 = _noalloc_bwd(lib, dy, x, g, mean, rstd, add, accumulate_into=acc, dx=dx_out)
    assert rc == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_reserved() == reserved_before      # torch's pool did not grow either
    assert free_after == free_before, f"device free memory moved by {free_before - free_after} bytes across the call"
    _close(dg2, 2 * ref_dg, 5e-2)
    _close(db2, 2 * ref_db, 5e-2)
    assert _native.read_status() == (0, 0)


def test_layer_norm_bwd_noalloc_rejects_oversized_problem():
    lib = ctypes.CDLL(_native.lib_path("libofb_kernels.so"))
    lib.ofb_last_error.restype = ctypes.c_char_p
    rows, cols = 8, 8192
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    mean = torch.zeros(rows, device="cuda")
    rstd = torch.ones(rows, device="cuda")
    rc, *_ = _noalloc_bwd(lib, x, x, None, mean, rstd, None)
    assert rc == -1
    assert b"exceeds the built-in scratch" in lib.ofb_last_error()


def test_layer_norm_bwd_noalloc_rejects_half_given_param_grads_and_bad_cols():
    """One of dgamma / dbeta without the other, or a non-positive column count, is refused before anything launches."""
    lib = ctypes.CDLL(_native.lib_path("libofb_kernels.so"))
    lib.ofb_layer_norm_bwd_noalloc.restype = c_int
    lib.ofb_layer_norm_bwd.restype = c_int
    lib.ofb_last_error.restype = ctypes.c_char_p
    rows, cols = 16, 256
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    mean = torch.zeros(rows, device="cuda")
    rstd = torch.ones(rows, device="cuda")
    dx = torch.empty_like(x)
    dg = torch.zeros(cols, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ofb_layer_norm_bwd_noalloc(_ptr(x), _ptr(x), _ptr(None), _ptr(mean), _ptr(rstd), _ptr(None), _ptr(dx),
                                        _ptr(dg), _ptr(None), c_int(0), c_int(rows), c_int(cols), stream)
    assert rc == -1 and b"together" in lib.ofb_last_error()
    rc = lib.ofb_layer_norm_bwd_noalloc(_ptr(x), _ptr(x), _ptr(None), _ptr(mean), _ptr(rstd), _ptr(None), _ptr(dx),
                                        _ptr(None), _ptr(None), c_int(0), c_int(rows), c_int(0), stream)
    assert rc == -1 and b"positive multiple of 8" in lib.ofb_last_error()
    scratch = torch.empty(2 * rows * cols, device="cuda")
    rc = lib.ofb_layer_norm_bwd(_ptr(x), _ptr(x), _ptr(None), _ptr(mean), _ptr(rstd), _ptr(None), _ptr(dx), _ptr(None),
                                _ptr(dg), _ptr(scratch), c_int(0), c_int(rows), c_int(cols), stream)
    assert rc == -1 and b"together" in lib.ofb_last_error()
    with pytest.raises(ValueError):
        K.layer_norm_bwd(x, x, None, mean, rstd, dgamma=dg, dbeta=None)
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)
