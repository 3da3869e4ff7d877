"""ctypes bindings of libofb_core.so: control store with heartbeat failure detection, caching allocator,
persistent (SSD) table, dependency-tracking task executor, record / token readers, SBP geometry."""
from __future__ import annotations

import ctypes
from ctypes import (CFUNCTYPE, POINTER, c_char_p, c_double, c_int, c_int64, c_uint8, c_uint64, c_void_p)

import numpy as np

from ..ops import _native


class CoreError(RuntimeError):
    pass


_configured = False


def lib():
    global _configured
    L = _native.core()
    if not _configured:
        L.ofc_last_error.restype = c_char_p
        for name in ("ofc_store_server_start", "ofc_store_client_connect", "ofc_allocator_create", "ofc_allocator_alloc",
                     "ofc_ptable_open", "ofc_executor_create", "ofc_records_open", "ofc_tokens_open"):
            getattr(L, name).restype = c_void_p
        for name in ("ofc_store_add", "ofc_store_num_keys", "ofc_ptable_get", "ofc_ptable_size", "ofc_ptable_keys", "ofc_executor_completed", "ofc_records_next",
                     "ofc_tokens_count"):
            getattr(L, name).restype = c_int64
        L.ofc_copy_cost.restype = c_double
        _configured = True
    return L


def _err():
    m = lib().ofc_last_error()
    return m.decode() if m else "unknown error"


def _check(rc, what):
    if rc is None or (isinstance(rc, int) and rc < 0):
        raise (TimeoutError if rc == -2 else CoreError)(f"{what}: {_err()}")
    return rc


# ------------------------------------------------------------------------------------------------ sbp geometry
def balanced_split(total, parts, idx):
    b, e = c_int64(), c_int64()
    lib().ofc_balanced_split(c_int64(total), c_int64(parts), c_int64(idx), ctypes.byref(b), ctypes.byref(e))
    return b.value, e.value


_KIND = {"B": 0, "P": 1, "S": 2}


def slice_view(logical_shape, hierarchy, nd_sbp, coords):
    nd, md = len(logical_shape), len(hierarchy)
    shape = (c_int64 * nd)(*logical_shape)
    hier = (c_int64 * md)(*hierarchy)
    kinds = (c_int * md)(*[_KIND[s.kind] for s in nd_sbp])
    axes = (c_int * md)(*[s.axis for s in nd_sbp])
    co = (c_int64 * md)(*coords)
    out = (c_int64 * (2 * nd))()
    _check(lib().ofc_slice_view(shape, nd, hier, md, kinds, axes, co, out), "slice_view")
    return [(out[2 * i], out[2 * i + 1]) for i in range(nd)]


def copy_cost(in_sbp, out_sbp, nbytes, n, same_placement=True):
    return lib().ofc_copy_cost(_KIND[in_sbp.kind], in_sbp.axis, _KIND[out_sbp.kind], out_sbp.axis, c_double(nbytes), n,
                               int(same_placement))


# ------------------------------------------------------------------------------------------------ control store
class ControlServer:
    def __init__(self, world_size, port=0):
        self.h = lib().ofc_store_server_start(port, world_size)
        if not self.h:
            raise CoreError(_err())
        self.port = lib().ofc_store_server_port(c_void_p(self.h))

    def stop(self):
        if self.h:
            lib().ofc_store_server_stop(c_void_p(self.h))
            self.h = None


class ControlClient:
    """KV / counters / barriers with deadlines, plus the heartbeat that lets peers notice a lost rank."""

    def __init__(self, host, port, rank, timeout_s=30.0):
        self.h = lib().ofc_store_client_connect(host.encode(), port, rank, int(timeout_s * 1000))
        if not self.h:
            raise CoreError(_err())
        self.rank = rank

    def set(self, key, value: bytes):
        _check(lib().ofc_store_set(c_void_p(self.h), key.encode(), value, len(value)), "store.set")

    def get(self, key, timeout_s=30.0, cap=1 << 20) -> bytes:
        buf = ctypes.create_string_buffer(cap)
        n = _check(lib().ofc_store_get(c_void_p(self.h), key.encode(), buf, cap, int(timeout_s * 1000)), "store.get")
        return buf.raw[:n]

    def add(self, key, delta=1):
        return _check(lib().ofc_store_add(c_void_p(self.h), key.encode(), c_int64(delta)), "store.add")

    def delete(self, key) -> bool:
        return _check(lib().ofc_store_delete(c_void_p(self.h), key.encode()), "store.delete") > 0

    def has(self, key) -> bool:
        return _check(lib().ofc_store_has(c_void_p(self.h), key.encode()), "store.has") > 0

    def num_keys(self) -> int:
        return _check(lib().ofc_store_num_keys(c_void_p(self.h)), "store.num_keys")

    def compare_set(self, key, expected: bytes, desired: bytes, cap=1 << 20) -> bytes:
        buf = ctypes.create_string_buffer(cap)
        n = _check(lib().ofc_store_compare_set(c_void_p(self.h), key.encode(), expected, len(expected), desired, len(desired),
                                               buf, cap), "store.compare_set")
        return buf.raw[:n]

    def barrier(self, name, world_size, timeout_s=30.0):
        _check(lib().ofc_store_barrier(c_void_p(self.h), name.encode(), world_size, int(timeout_s * 1000)), "store.barrier")

    def start_heartbeat(self, interval_s=1.0):
        _check(lib().ofc_store_heartbeat_start(c_void_p(self.h), int(interval_s * 1000)), "store.heartbeat")

    def lost_ranks(self, max_age_s):
        out = (c_int * 1024)()
        n = _check(lib().ofc_store_lost_ranks(c_void_p(self.h), int(max_age_s * 1000), out, 1024), "store.lost_ranks")
        return [out[i] for i in range(min(n, 1024))]

    def close(self):
        if self.h:
            lib().ofc_store_client_close(c_void_p(self.h))
            self.h = None


# ------------------------------------------------------------------------------------------------ allocator
class BinAllocator:
    def __init__(self, backend="cuda", chunk_bytes=1 << 30):
        self.h = lib().ofc_allocator_create(1 if backend == "cuda" else 0, c_int64(chunk_bytes))
        if not self.h:
            raise CoreError(_err())

    def alloc(self, nbytes):
        p = lib().ofc_allocator_alloc(c_void_p(self.h), c_int64(nbytes))
        if not p:
            raise MemoryError(_err())
        return p

    def free(self, ptr):
        _check(lib().ofc_allocator_free(c_void_p(self.h), c_void_p(ptr)), "allocator.free")

    def shrink(self):
        return lib().ofc_allocator_shrink(c_void_p(self.h))

    def stats(self):
        v = [c_int64() for _ in range(4)]
        lib().ofc_allocator_stats(c_void_p(self.h), *[ctypes.byref(x) for x in v])
        return dict(zip(("reserved", "in_use", "chunks", "free_blocks"), (x.value for x in v)))

    def destroy(self):
        if self.h:
            lib().ofc_allocator_destroy(c_void_p(self.h))
            self.h = None


def use_bin_allocator_for_torch():
    """Routes every CUDA allocation of torch through the native caching allocator. Must be called before the
    first CUDA allocation of the process."""
    import torch
    alloc = torch.cuda.memory.CUDAPluggableAllocator(_native.lib_path("libofb_core.so"), "ofc_torch_alloc", "ofc_torch_free")
    torch.cuda.memory.change_current_allocator(alloc)
    return alloc


# ------------------------------------------------------------------------------------------------ persistent table
class PersistentTable:
    def __init__(self, path, value_bytes, block_bytes=512, read_only=False):
        self.h = lib().ofc_ptable_open(str(path).encode(), value_bytes, block_bytes, int(read_only))
        if not self.h:
            raise CoreError(_err())
        self.value_bytes = value_bytes

    def put(self, keys: np.ndarray, values: np.ndarray):
        keys = np.ascontiguousarray(keys, dtype=np.int64)
        values = np.ascontiguousarray(values)
        assert values.nbytes == keys.size * self.value_bytes
        _check(lib().ofc_ptable_put(c_void_p(self.h), keys.ctypes.data_as(POINTER(c_int64)), values.ctypes.data_as(c_void_p),
                                    c_int64(keys.size)), "ptable.put")

    def get(self, keys: np.ndarray, dtype=np.float32):
        keys = np.ascontiguousarray(keys, dtype=np.int64)
        width = self.value_bytes // np.dtype(dtype).itemsize
        out = np.empty((keys.size, width), dtype=dtype)
        found = np.empty(keys.size, dtype=np.uint8)
        _check(lib().ofc_ptable_get(c_void_p(self.h), keys.ctypes.data_as(POINTER(c_int64)), out.ctypes.data_as(c_void_p),
                                    found.ctypes.data_as(POINTER(c_uint8)), c_int64(keys.size)), "ptable.get")
        return out, found.astype(bool)

    def __len__(self):
        return lib().ofc_ptable_size(c_void_p(self.h))

    def keys(self) -> np.ndarray:
        """All keys of the current index (unspecified order)."""
        out = np.empty(len(self), dtype=np.int64)
        n = lib().ofc_ptable_keys(c_void_p(self.h), out.ctypes.data_as(POINTER(c_int64)), c_int64(out.size))
        return out[:n]

    def save_snapshot(self, name):
        _check(lib().ofc_ptable_save_snapshot(c_void_p(self.h), name.encode()), "ptable.save_snapshot")

    def load_snapshot(self, name):
        _check(lib().ofc_ptable_load_snapshot(c_void_p(self.h), name.encode()), "ptable.load_snapshot")

    def close(self):
        if self.h:
            lib().ofc_ptable_close(c_void_p(self.h))
            self.h = None


# ------------------------------------------------------------------------------------------------ executor
_TASK = CFUNCTYPE(None, c_void_p)


class TaskExecutor:
    """Runs Python callables on per-stream worker threads in dependency order (reads / writes of object ids)."""

    def __init__(self, n_streams=2):
        self.h = lib().ofc_executor_create(n_streams)
        if not self.h:
            raise CoreError(_err())
        self._keep = []

    def submit(self, stream, fn, reads=(), writes=()):
        cb = _TASK(lambda _arg, fn=fn: fn())
        self._keep.append(cb)
        r = (c_int64 * max(len(reads), 1))(*reads)
        w = (c_int64 * max(len(writes), 1))(*writes)
        _check(lib().ofc_executor_submit(c_void_p(self.h), stream, cb, None, r, len(reads), w, len(writes)), "executor.submit")

    def wait_all(self, timeout_s=60.0):
        _check(lib().ofc_executor_wait_all(c_void_p(self.h), int(timeout_s * 1000)), "executor.wait_all")
        self._keep.clear()

    def completed(self):
        return lib().ofc_executor_completed(c_void_p(self.h))

    def destroy(self):
        if self.h:
            lib().ofc_executor_destroy(c_void_p(self.h))
            self.h = None


# ------------------------------------------------------------------------------------------------ readers
def write_records(path, records):
    n = len(records)
    bufs = [ctypes.create_string_buffer(r, len(r)) for r in records]
    ptrs = (c_void_p * n)(*[ctypes.cast(b, c_void_p) for b in bufs])
    lens = (c_int64 * n)(*[len(r) for r in records])
    _check(lib().ofc_records_write(str(path).encode(), ptrs, lens, c_int64(n)), "records.write")


class RecordReader:
    def __init__(self, path, prefetch=8, shuffle_buffer=0, seed=0, max_record_bytes=1 << 20):
        self.h = lib().ofc_records_open(str(path).encode(), prefetch, shuffle_buffer, c_uint64(seed))
        if not self.h:
            raise CoreError(_err())
        self.buf = ctypes.create_string_buffer(max_record_bytes)

    def __iter__(self):
        return self

    def __next__(self):
        n = lib().ofc_records_next(c_void_p(self.h), self.buf, c_int64(len(self.buf)))
        while n == -3 and len(self.buf) < (1 << 31):     # record larger than the buffer: it stays queued, grow and retry
            self.buf = ctypes.create_string_buffer(len(self.buf) * 4)
            n = lib().ofc_records_next(c_void_p(self.h), self.buf, c_int64(len(self.buf)))
        if n == 0:
            raise StopIteration
        if n == -4:
            return b""
        _check(n, "records.next")
        return self.buf.raw[:n]

    def close(self):
        if self.h:
            lib().ofc_records_close(c_void_p(self.h))
            self.h = None


class TokenDataset:
    """Memory-mapped flat token file; ``batch(indices, seq_len)`` -> int64 [len(indices), seq_len + 1]."""

    def __init__(self, path, token_bytes=2):
        self.h = lib().ofc_tokens_open(str(path).encode(), token_bytes)
        if not self.h:
            raise CoreError(_err())

    def __len__(self):
        return lib().ofc_tokens_count(c_void_p(self.h))

    def batch(self, sample_idx, seq_len, stride=None):
        idx = np.ascontiguousarray(sample_idx, dtype=np.int64)
        out = np.empty((idx.size, seq_len + 1), dtype=np.int64)
        _check(lib().ofc_tokens_batch(c_void_p(self.h), idx.ctypes.data_as(POINTER(c_int64)), c_int64(idx.size), c_int64(seq_len),
                                      c_int64(stride if stride is not None else seq_len), out.ctypes.data_as(POINTER(c_int64))),
               "tokens.batch")
        return out

    def close(self):
        if self.h:
            lib().ofc_tokens_close(c_void_p(self.h))
            self.h = None
