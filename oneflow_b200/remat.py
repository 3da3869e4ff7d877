"""``flow.remat``: dynamic tensor rematerialisation under a memory budget.

What the reference does inside its allocator and virtual machine (oneflow/core/vm/remat/allocator.cpp, remat/env.cpp,
remat/util.cpp; python/oneflow/remat/__init__.py:21-54 for the budget calls): every tensor an operator produced remembers
the operator and its inputs; when the memory in use would pass the budget, the tensors that are cheapest to lose are
evicted (their memory is released, the tensor objects stay), and an evicted tensor that is needed again - by a later
operator or by backward - is recomputed from its inputs, recursively. The eviction score is the one of the DTR paper:
compute cost / (bytes * time since the last access), smallest first.

Here the bookkeeping hangs on ``__torch_dispatch__``: inside ``with flow.remat.scope():`` every ATen operator is seen
with its concrete arguments. A fresh output storage becomes an entry (producer = the operator call, cost = its host time,
bytes). Eviction is ``storage.resize_(0)``, rematerialisation re-runs the producer and copies the value back into the same
storage, so every tensor object (views, tensors autograd saved) that shares it is valid again. Backward reaches evicted
tensors through ``saved_tensors_hooks``: unpacking a saved tensor rematerialises it first; on CUDA that happens on
autograd's device thread, so the state is guarded by a lock.

Never evicted: tensors without a producer (parameters, inputs), outputs of random operators (the mask would differ),
storages that an in-place operator rewrote after they were produced, tensors passed to ``disable_eviction``, and - with
the small-pieces optimisation on - tensors below 64 KiB, whose eviction frees little and fragments the allocator.

    flow.remat.set_budget("8GB")
    with flow.remat.scope():
        loss = model(x).sum()
        loss.backward()
    print(flow.remat.stats())       # forced_eviction_num, eager_eviction_num, recomputation_num, peak_bytes

When the scope ends, every tensor the program still references is brought back into memory if it was evicted.
"""
import re
import threading
import time
import weakref

import torch
from torch.utils._python_dispatch import TorchDispatchMode

_state = {"budget": None, "small_pieces": True}
_SMALL_PIECE = 64 * 1024
_RANDOM = ("dropout", "rand", "bernoulli", "normal", "uniform", "multinomial", "randperm", "random")


def parse_size(size):
    units = {"B": 1, "KB": 2 ** 10, "MB": 2 ** 20, "GB": 2 ** 30, "TB": 2 ** 40, "": 1,
             "KIB": 10 ** 3, "MIB": 10 ** 6, "GIB": 10 ** 9, "TIB": 10 ** 12}
    m = re.match(r"^([\d\.]+)\s*([a-zA-Z]{0,3})$", str(size).strip())
    if m is None or m.group(2).upper() not in units:
        raise ValueError(f"cannot parse size {size!r}")
    return int(float(m.group(1)) * units[m.group(2).upper()])


def set_budget(budget):
    _state["budget"] = parse_size(budget)


def get_budget():
    return _state["budget"]


def set_small_pieces_optimization(mode=True):
    _state["small_pieces"] = bool(mode)


def is_small_pieces_optimization_enabled():
    return _state["small_pieces"]


def is_enabled():
    return _state["budget"] is not None


class _Entry:
    __slots__ = ("storage", "nbytes", "producer", "out_index", "meta", "cost", "last_access", "pinned", "evicted", "device", "seq",
                 "__weakref__")

    def __init__(self, storage, nbytes, device):
        self.storage = weakref.ref(storage)
        self.nbytes, self.device = nbytes, device
        self.producer = None          # (func, args, kwargs) with tensors kept as they were passed
        self.out_index = 0
        self.meta = None              # (dtype, shape, stride, storage_offset) of the produced tensor
        self.cost = 0.0
        self.last_access = 0
        self.pinned = False
        self.evicted = False
        self.seq = 0                  # creation order


class _Remat(TorchDispatchMode):
    def __init__(self, budget):
        super().__init__()
        self.budget = budget
        self.entries = {}             # storage._cdata -> _Entry
        self.bytes = {}               # device type -> tracked bytes in memory
        self.lock = threading.RLock()
        self.clock = 0
        self.stats = {"forced_eviction_num": 0, "eager_eviction_num": 0, "recomputation_num": 0, "peak_bytes": 0}
        self._hooks = None
        self._in_remat = 0

    # ---- bookkeeping
    def _entry_of(self, t):
        st = t.untyped_storage()
        e = self.entries.get(st._cdata)
        if e is not None and e.storage() is not st:
            # the address of a storage that died was handed out again before its entry was dropped
            self.entries.pop(st._cdata, None)
            if not e.evicted:
                self.bytes[e.device] -= e.nbytes
            return None
        return e

    def _track(self, t, producer, out_index, cost):
        st = t.untyped_storage()
        key = st._cdata
        if key in self.entries or st.nbytes() == 0:
            return
        e = _Entry(st, st.nbytes(), t.device.type)
        e.producer, e.out_index, e.cost = producer, out_index, cost
        e.meta = (t.dtype, tuple(t.shape), tuple(t.stride()), t.storage_offset())
        e.last_access = self.clock
        e.seq = self.clock
        self.entries[key] = e
        self.bytes[e.device] = self.bytes.get(e.device, 0) + e.nbytes
        weakref.finalize(st, self._forget, key)

    def _forget(self, key):
        with self.lock:
            e = self.entries.get(key)
            if e is None or e.storage() is not None:
                return                 # already dropped, or the key belongs to a newer storage at the same address
            del self.entries[key]
            if not e.evicted:
                self.bytes[e.device] -= e.nbytes

    def _evictable(self, e, locked):
        if e.pinned or e.evicted or e.producer is None or id(e) in locked:
            return False
        if _state["small_pieces"] and e.nbytes < _SMALL_PIECE:
            return False
        return e.storage() is not None

    def _evict(self, e, forced):
        st = e.storage()
        if st is None or e.evicted:
            return
        st.resize_(0)
        e.evicted = True
        self.bytes[e.device] -= e.nbytes
        self.stats["forced_eviction_num" if forced else "eager_eviction_num"] += 1

    def _enforce(self, device, locked, incoming=0):
        """Evicts, cheapest first, until ``device`` holds at most the budget (less ``incoming`` bytes about to be allocated)."""
        if self.budget is None:
            return
        while self.bytes.get(device, 0) + incoming > self.budget:
            best, best_h = None, None
            for e in self.entries.values():
                if e.device != device or not self._evictable(e, locked):
                    continue
                h = (e.cost + 1e-7) / (e.nbytes * (self.clock - e.last_access + 1))
                if best is None or h < best_h:
                    best, best_h = e, h
            if best is None:
                return                 # nothing left to give up: the caller runs over budget rather than fail
            self._evict(best, forced=True)

    def _tensors(self, args, kwargs):
        out = []

        def walk(x):
            if torch.is_tensor(x):
                out.append(x)
            elif isinstance(x, (list, tuple)):
                for y in x:
                    walk(y)
        walk(args)
        walk(list(kwargs.values()))
        return out

    def materialize(self, t, locked=None):
        """Makes ``t``'s storage hold its value again (recomputing its producer, and that one's evicted inputs first)."""
        with self.lock:
            e = self._entry_of(t)
            if e is not None:
                self._materialize_entry(e, set() if locked is None else locked)
            return t

    def _materialize_entry(self, e, locked):
        self.clock += 1
        e.last_access = self.clock
        st = e.storage()              # held for the whole recomputation
        if not e.evicted or st is None:
            return
        locked.add(id(e))
        func, args, kwargs = e.producer
        ins = self._tensors(args, kwargs)
        for x in ins:
            xe = self._entry_of(x)
            if xe is not None:
                locked.add(id(xe))
        for x in ins:
            self.materialize(x, locked)
        self._enforce(e.device, locked, incoming=e.nbytes)
        self._in_remat += 1           # the recomputation and the copy back are not operators of the program
        try:
            with torch.no_grad():
                out = func(*args, **kwargs)
                value = (out if isinstance(out, (list, tuple)) else (out,))[e.out_index]
                st.resize_(e.nbytes)
                dtype, shape, stride, offset = e.meta
                torch.empty(0, dtype=dtype, device=value.device).set_(st, offset, shape, stride).copy_(value)
        finally:
            self._in_remat -= 1
        e.evicted = False
        self.bytes[e.device] = self.bytes.get(e.device, 0) + e.nbytes
        self.stats["recomputation_num"] += 1
        self.stats["peak_bytes"] = max(self.stats["peak_bytes"], self.bytes[e.device])

    # ---- the operator stream
    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if self._in_remat:
            return func(*args, **kwargs)
        with self.lock:
            self.clock += 1
            ins = self._tensors(args, kwargs)
            locked = set()
            for x in ins:
                e = self._entry_of(x)
                if e is not None:
                    locked.add(id(e))
            for x in ins:
                self.materialize(x, locked)
            name = getattr(getattr(func, "overloadpacket", func), "__name__", str(func))
            # an operator that writes one of its arguments makes that storage's producer record stale
            schema = getattr(func, "_schema", None)
            if schema is not None and schema.is_mutable:
                for a, x in zip(schema.arguments, args):
                    if a.alias_info is not None and a.alias_info.is_write and torch.is_tensor(x):
                        e = self._entry_of(x)
                        if e is not None:
                            e.pinned = True
            dev = ins[0].device.type if ins else "cpu"
            self._enforce(dev, locked)
            t0 = time.perf_counter()
            out = func(*args, **kwargs)
            cost = time.perf_counter() - t0
            random_op = any(r in name for r in _RANDOM)
            known = {x.untyped_storage()._cdata for x in ins}
            outs = out if isinstance(out, (list, tuple)) else (out,)
            for i, o in enumerate(outs):
                if not torch.is_tensor(o) or o.untyped_storage()._cdata in known:
                    continue           # a view of an input, or an input handed back
                self._track(o, None if random_op else (func, args, kwargs), i, cost)
                oe = self._entry_of(o)
                if oe is not None:
                    locked.add(id(oe))
                    self._enforce(o.device.type, locked)
                    self.stats["peak_bytes"] = max(self.stats["peak_bytes"], self.bytes.get(o.device.type, 0))
            return out

    # ---- scope
    def __enter__(self):
        super().__enter__()
        self._hooks = torch.autograd.graph.saved_tensors_hooks(lambda t: t, lambda t: self.materialize(t))
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        self._hooks.__exit__(*exc)
        # Whatever the program still holds must be in memory when the bookkeeping ends. Entries are visited from the newest
        # to the oldest and give up their producer record on the way: when an entry's turn comes, every consumer recorded
        # after it has already let go of its inputs, so its storage is alive only if the program (a variable, autograd's
        # graph) references it - then it is recomputed if evicted - and otherwise it has been freed already.
        with self.lock:
            order = sorted(((e.seq, k) for k, e in self.entries.items()), reverse=True)
            for _, k in order:
                e = self.entries.get(k)
                if e is None:
                    continue
                if e.evicted and e.storage() is not None:
                    self._materialize_entry(e, set())
                e.producer = None
            self.entries.clear()
        return super().__exit__(*exc)


_current = None


class scope:
    """``with flow.remat.scope(budget=None):`` forward and backward inside run under the budget (``set_budget`` if none given)."""

    def __init__(self, budget=None):
        self.budget = parse_size(budget) if isinstance(budget, str) else budget

    def __enter__(self):
        global _current
        if _current is not None:
            raise RuntimeError("remat scopes do not nest")
        b = self.budget if self.budget is not None else _state["budget"]
        _current = _Remat(b)
        _current.__enter__()
        return _current

    def __exit__(self, *exc):
        global _current
        cur, _current = _current, None
        _last_stats.clear()
        _last_stats.update(cur.stats)
        return cur.__exit__(*exc)


_last_stats = {}


def stats():
    """Counters of the running scope, or of the last one that ended."""
    return dict(_current.stats) if _current is not None else dict(_last_stats)


def clear_stats():
    _last_stats.clear()
    if _current is not None:
        for k in _current.stats:
            _current.stats[k] = 0


def _need_scope():
    if _current is None:
        raise RuntimeError("no remat scope is active")
    return _current


def evict(tensor):
    """Releases ``tensor``'s memory now if it can be recomputed (reference: remat.evict in the expensive remat tests)."""
    r = _need_scope()
    with r.lock:
        e = r._entry_of(tensor)
        if e is None or e.producer is None or e.pinned:
            raise RuntimeError("this tensor cannot be evicted: it has no recorded producer or eviction is disabled for it")
        r._evict(e, forced=False)


def is_in_memory(tensor):
    r = _need_scope()
    e = r._entry_of(tensor)
    return True if e is None else not e.evicted


def disable_eviction(tensor):
    r = _need_scope()
    e = r._entry_of(tensor)
    if e is not None:
        e.pinned = True


def allocated_memory(device="cpu"):
    """Bytes of tracked tensors currently in memory on ``device`` ("cpu" / "cuda")."""
    return _need_scope().bytes.get(str(device).split("+")[0].split(":")[0], 0)
