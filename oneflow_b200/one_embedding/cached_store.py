"""Tiered embedding store: a device LRU cache in front of a host-memory or SSD table.

What ``make_cached_host_mem_store_options`` / ``make_cached_ssd_store_options`` select (reference:
oneflow/core/embedding/cached_key_value_store.cu over lru_cache.cu, with mock / persistent-table key-value stores
behind it). A lookup asks the cache first; the keys it misses are fetched from the backing table (rows that exist
nowhere yet are created by the table's initializer), the fetched rows are put into the cache, and the rows the cache
pushes out to make room are written back to the backing table. Updated rows are put the same way. So the device holds
the hot rows only (``cache_memory_budget_mb``), while the table itself lives in host memory or on disk.

On CUDA the cache is the set-associative kernel of csrc/kernels/lru_cache.cu; on CPU (tests without a GPU) an ordered
dictionary with the same interface stands in. The class offers the ``RowStore`` interface of ``embedding.py`` (``lookup``
-> slots, ``rows``, ``put``): slots index a per-step staging tensor that holds the rows of the current batch.
"""
from __future__ import annotations

import ctypes
from collections import OrderedDict
from ctypes import Structure, c_int, c_longlong, c_uint, c_void_p

import numpy as np
import torch

from ..ops import _native


class _LruStruct(Structure):
    _fields_ = [("keys", c_void_p), ("ticks", c_void_p), ("lines", c_void_p), ("locks", c_void_p), ("n_sets", c_longlong), ("line", c_int)]


class DeviceLruCache:
    """32-way set-associative LRU cache of fp32 rows in device memory (csrc/kernels/lru_cache.cu)."""

    WAYS = 32

    def __init__(self, capacity_rows, line, device):
        self.device = torch.device(device)
        self.line = int(line)
        if self.line % 4:
            raise ValueError("the cached row length must be a multiple of 4 floats")
        self.n_sets = max(1, int(capacity_rows) // self.WAYS)
        n = self.n_sets * self.WAYS
        self.keys = torch.zeros(n, dtype=torch.int64, device=self.device)
        self.ticks = torch.zeros(n, dtype=torch.int32, device=self.device)
        self.lines = torch.zeros((n, self.line), dtype=torch.float32, device=self.device)
        self.locks = torch.zeros(self.n_sets, dtype=torch.int32, device=self.device)
        self.tick = 0
        self.c = _LruStruct(self.keys.data_ptr(), self.ticks.data_ptr(), self.lines.data_ptr(), self.locks.data_ptr(), self.n_sets, self.line)
        self._cnt = torch.zeros(1, dtype=torch.int32, device=self.device)

    @property
    def capacity(self):
        return self.n_sets * self.WAYS

    def _next_tick(self):
        self.tick += 1
        if self.tick >= 0x7FFFFFFF:          # renumber before the counter wraps: ages keep their order
            self.ticks.copy_(torch.where(self.ticks > 0, torch.ones_like(self.ticks), self.ticks))
            self.tick = 2
        return self.tick

    def get(self, keys):
        """rows [n, line] (zero where missed), hit mask [n] bool, indices of the misses [m] (int64)."""
        n = keys.numel()
        out = torch.zeros((n, self.line), dtype=torch.float32, device=self.device)
        hit = torch.zeros(n, dtype=torch.uint8, device=self.device)
        miss_index = torch.empty(n, dtype=torch.int32, device=self.device)
        miss_keys = torch.empty(n, dtype=torch.int64, device=self.device)
        self._cnt.zero_()
        if n:
            _native.check(_native.kernels().ofb_lru_get(
                ctypes.byref(self.c), _native.ptr(keys), c_longlong(n), _native.ptr(out), c_uint(self._next_tick()), _native.ptr(self._cnt),
                _native.ptr(miss_index), _native.ptr(miss_keys), _native.ptr(hit), _native.stream_ptr()), "lru_get")
        m = int(self._cnt.item())
        # the kernel lists misses in the order its warps found them; callers get them in batch order (row creation
        # draws from a stream, so the order must not depend on scheduling)
        return out, hit.bool(), miss_index[:m].long().sort().values

    def put(self, keys, rows):
        """Inserts / overwrites; returns the (keys, rows) pushed out of the cache."""
        n = keys.numel()
        ek = torch.empty(n, dtype=torch.int64, device=self.device)
        er = torch.empty((n, self.line), dtype=torch.float32, device=self.device)
        self._cnt.zero_()
        if n:
            _native.check(_native.kernels().ofb_lru_put(
                ctypes.byref(self.c), _native.ptr(keys), _native.ptr(rows.contiguous()), c_longlong(n), c_uint(self._next_tick()),
                _native.ptr(self._cnt), _native.ptr(ek), _native.ptr(er), _native.stream_ptr()), "lru_put")
        m = int(self._cnt.item())
        return ek[:m], er[:m]

    def dump(self):
        cap = self.capacity
        k = torch.empty(cap, dtype=torch.int64, device=self.device)
        r = torch.empty((cap, self.line), dtype=torch.float32, device=self.device)
        self._cnt.zero_()
        _native.check(_native.kernels().ofb_lru_dump(ctypes.byref(self.c), _native.ptr(self._cnt), _native.ptr(k), _native.ptr(r),
                                                     c_longlong(cap), _native.stream_ptr()), "lru_dump")
        m = int(self._cnt.item())
        return k[:m], r[:m]


class HostLruCache:
    """The same interface on CPU tensors (an ordered dictionary): used where no GPU is present."""

    def __init__(self, capacity_rows, line, device="cpu"):
        self.capacity, self.line, self.device = max(1, int(capacity_rows)), int(line), torch.device("cpu")
        self.d = OrderedDict()

    def get(self, keys):
        n = keys.numel()
        out = torch.zeros((n, self.line), dtype=torch.float32)
        hit = torch.zeros(n, dtype=torch.bool)
        miss = []
        for i, k in enumerate(keys.tolist()):
            row = self.d.get(k)
            if row is None:
                miss.append(i)
            else:
                self.d.move_to_end(k)
                out[i] = row
                hit[i] = True
        return out, hit, torch.tensor(miss, dtype=torch.int64)

    def put(self, keys, rows):
        ek, er = [], []
        for k, row in zip(keys.tolist(), rows):
            if k in self.d:
                self.d.move_to_end(k)
            elif len(self.d) >= self.capacity:
                old, old_row = self.d.popitem(last=False)
                ek.append(old)
                er.append(old_row)
            self.d[k] = row.clone()
        if ek:
            return torch.tensor(ek, dtype=torch.int64), torch.stack(er)
        return torch.empty(0, dtype=torch.int64), torch.empty((0, self.line))

    def dump(self):
        if not self.d:
            return torch.empty(0, dtype=torch.int64), torch.empty((0, self.line))
        return torch.tensor(list(self.d.keys()), dtype=torch.int64), torch.stack(list(self.d.values()))


class HostTable:
    """The full table in host memory: key -> row of a growing pinned array (the "full" host tier)."""

    def __init__(self, line, capacity):
        self.line, self.capacity = int(line), int(capacity)
        self.index = {}
        self.values = np.zeros((min(self.capacity, 4096), self.line), dtype=np.float32)

    def __len__(self):
        return len(self.index)

    def get(self, keys_np):
        found = np.zeros(len(keys_np), dtype=bool)
        out = np.zeros((len(keys_np), self.line), dtype=np.float32)
        for i, k in enumerate(keys_np.tolist()):
            r = self.index.get(k)
            if r is not None:
                out[i] = self.values[r]
                found[i] = True
        return out, found

    def put(self, keys_np, rows_np):
        for k, row in zip(keys_np.tolist(), rows_np):
            r = self.index.get(k)
            if r is None:
                r = len(self.index)
                if r >= self.capacity:
                    raise RuntimeError(f"host embedding table is full ({self.capacity} rows)")
                if r >= self.values.shape[0]:
                    grown = np.zeros((min(self.capacity, self.values.shape[0] * 2), self.line), dtype=np.float32)
                    grown[:self.values.shape[0]] = self.values
                    self.values = grown
                self.index[k] = r
            self.values[r] = row

    def items(self):
        keys = np.fromiter(self.index.keys(), dtype=np.int64, count=len(self.index))
        return keys, self.values[np.fromiter(self.index.values(), dtype=np.int64, count=len(self.index))]


class SsdTable:
    """The full table on disk (csrc/core/persistent_table.cpp through runtime.PersistentTable)."""

    def __init__(self, line, path, block_bytes=512):
        from ..runtime.core import PersistentTable
        self.line = int(line)
        self.t = PersistentTable(path, value_bytes=self.line * 4, block_bytes=block_bytes)

    def __len__(self):
        return len(self.t)

    def get(self, keys_np):
        vals, found = self.t.get(np.ascontiguousarray(keys_np, dtype=np.int64))
        return np.frombuffer(vals, dtype=np.float32).reshape(len(keys_np), self.line) if not isinstance(vals, np.ndarray) else \
            vals.view(np.float32).reshape(len(keys_np), self.line), np.asarray(found, dtype=bool)

    def put(self, keys_np, rows_np):
        if len(keys_np):
            self.t.put(np.ascontiguousarray(keys_np, dtype=np.int64), np.ascontiguousarray(rows_np, dtype=np.float32))

    def items(self):
        keys = self.t.keys()
        vals, _ = self.get(keys)
        return keys, vals


class CachedRowStore:
    """``RowStore`` interface over (device LRU cache, backing table)."""

    def __init__(self, line, device, cache_rows, backing, init_rows_fn):
        self.line, self.device = int(line), torch.device(device)
        self.backing = backing
        self._init_rows = init_rows_fn          # (keys, table_ids) -> fresh rows [n, line] on the device
        self.cache = DeviceLruCache(cache_rows, line, device) if self.device.type == "cuda" else HostLruCache(cache_rows, line)
        self.size = 0                           # rows ever created (the initializer's stream position)
        self._step_keys = None
        self._step_rows = None
        self.stats = {"hits": 0, "misses": 0, "created": 0, "evicted": 0}

    def _write_back(self, ek, er):
        if ek.numel():
            self.stats["evicted"] += int(ek.numel())
            self.backing.put(ek.cpu().numpy(), er.cpu().numpy())

    def lookup(self, keys, table_ids, insert=True):
        n = keys.numel()
        rows, hit, miss = self.cache.get(keys)
        self.stats["hits"] += int(n - miss.numel())
        self.stats["misses"] += int(miss.numel())
        slots = torch.arange(n, device=self.device)
        if miss.numel():
            mk = keys[miss]
            vals, found = self.backing.get(mk.cpu().numpy())
            found_t = torch.from_numpy(found).to(self.device)
            fetched = torch.from_numpy(np.ascontiguousarray(vals)).to(self.device)
            new = (~found_t).nonzero()[:, 0]
            if new.numel():
                if insert:
                    fetched[new] = self._init_rows(mk[new], table_ids[miss][new], self.size)
                    self.size += int(new.numel())
                    self.stats["created"] += int(new.numel())
                else:
                    slots[miss[new]] = -1
            rows[miss] = fetched
            keep = miss if insert else miss[found_t]
            if keep.numel():
                self._write_back(*self.cache.put(keys[keep], rows[keep]))
        self._step_keys, self._step_rows = keys, rows
        return slots

    def rows(self, slots):
        return self._step_rows[slots]

    def put(self, slots, rows):
        self._step_rows[slots] = rows
        self._write_back(*self.cache.put(self._step_keys[slots], rows))

    def flush(self):
        """Writes every cached row to the backing table (before a snapshot)."""
        k, r = self.cache.dump()
        if k.numel():
            self.backing.put(k.cpu().numpy(), r.cpu().numpy())

    def snapshot(self):
        self.flush()
        keys, vals = self.backing.items()
        return {"keys": torch.from_numpy(np.ascontiguousarray(keys)), "values": torch.from_numpy(np.ascontiguousarray(vals)),
                "size": self.size, "cached": True}

    def load_snapshot(self, snap):
        self.size = int(snap["size"])
        self.backing.put(snap["keys"].numpy(), snap["values"].numpy())
