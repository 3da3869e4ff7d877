"""OneEmbedding: embedding tables far larger than one device, hash-sharded over the ranks.

Public surface follows python/oneflow/one_embedding.py (:177-558 Embedding classes, :560-725 store
options, :727-815 initializers, :1301-1340 Optimizer wrapper):

    table = make_table_options(make_uniform_initializer(-0.05, 0.05))
    emb = MultiTableEmbedding("sparse", embedding_dim=128, dtype=flow.float16, key_type=flow.int64,
                              tables=[table] * 26, store_options=make_device_mem_store_options(...))
    y = emb(ids)                    # ids [batch, 26] -> [batch, 26, 128]
    opt = Optimizer(emb, flow.optim.SGD)   # or Adam / Adagrad / Ftrl / SmartDecayAdam, momentum SGD

Data flow per step (the three shuffles of the reference, oneflow/user/kernels/data_shuffle_kernel.cu and
one_embedding_*_p2p_kernel.cu):
  1. id shuffle       : unique the local (id, table) keys, send every key to its owner
                        ``hash(key) % world`` (all-to-all-v), owners unique what they received;
  2. embedding shuffle: owners look rows up in their store (missing rows are initialised by the table's
                        initializer), send them back; an inverse-index gather rebuilds [batch, tables, dim];
  3. gradient shuffle : row gradients are segment-summed per unique key, sent to the owners, summed there
                        and applied by the sparse row optimizer (SGD / momentum / Adam / Adagrad / FTRL), the
                        updated rows are put back into the store.
A stored line is ``storage_dim = size_factor * embedding_dim`` floats: ``[embedding | optimizer state...]``.
Stores: device memory (hash table + dense rows on the GPU), host memory behind a device LRU cache, SSD
(``csrc/core/persistent_table.cpp``) behind the caches. Single-rank jobs skip the exchanges.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import List, Optional

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------ option builders
def make_uniform_initializer(low, high):
    return {"type": "uniform", "low": float(low), "high": float(high)}


def make_normal_initializer(mean, std):
    return {"type": "normal", "mean": float(mean), "std": float(std)}


def make_trunc_normal_initializer(mean=0.0, std=1.0, a=-2.0, b=2.0):
    """Normal(mean, std) re-drawn until it falls inside [a, b]
    (reference: python/oneflow/one_embedding.py:792-813)."""
    return {"type": "trunc_normal", "mean": float(mean), "std": float(std), "a": float(a), "b": float(b)}


def make_constant_initializer(value):
    return {"type": "constant", "value": float(value)}


def make_table_options(param):
    """param: one initializer (whole table) or a list of column options."""
    if isinstance(param, dict) and "type" in param:
        return {"initializer": param}
    if isinstance(param, (list, tuple)):
        return {"columns": list(param)}
    raise ValueError("make_table_options expects an initializer or a list of column options")


make_table = make_table_options


def make_column_options(initializer):
    return {"initializer": initializer}


def _check_capacity(capacity):
    if capacity is None or capacity <= 0:
        raise ValueError("capacity must be a positive number of rows")


def make_device_mem_store_options(persistent_path, capacity, size_factor=1, physical_block_size=512):
    _check_capacity(capacity)
    return {"kv_store": {"caches": [{"policy": "full", "capacity": int(capacity), "value_memory_kind": "device"}],
                         "persistent_table": {"path": persistent_path, "physical_block_size": physical_block_size}},
            "size_factor": size_factor}


def make_cached_ssd_store_options(cache_budget_mb, persistent_path, capacity=None, size_factor=1, physical_block_size=512,
                                  host_cache_budget_mb=0):
    if cache_budget_mb <= 0 and host_cache_budget_mb <= 0:
        raise ValueError("cache_budget_mb or host_cache_budget_mb must be positive")
    caches = []
    if cache_budget_mb > 0:
        caches.append({"policy": "lru", "cache_memory_budget_mb": cache_budget_mb, "value_memory_kind": "device"})
    if host_cache_budget_mb > 0:
        caches.append({"policy": "lru", "cache_memory_budget_mb": host_cache_budget_mb, "value_memory_kind": "host"})
    pt = {"path": persistent_path, "physical_block_size": physical_block_size}
    if capacity is not None:
        pt["capacity_hint"] = int(capacity)
    return {"kv_store": {"caches": caches, "persistent_table": pt}, "size_factor": size_factor}


def make_cached_host_mem_store_options(cache_budget_mb, persistent_path, capacity, size_factor=1, physical_block_size=512):
    _check_capacity(capacity)
    if cache_budget_mb <= 0:
        raise ValueError("cache_budget_mb must be positive")
    return {"kv_store": {"caches": [{"policy": "lru", "cache_memory_budget_mb": cache_budget_mb, "value_memory_kind": "device"},
                                    {"policy": "full", "capacity": int(capacity), "value_memory_kind": "host"}],
                         "persistent_table": {"path": persistent_path, "physical_block_size": physical_block_size}},
            "size_factor": size_factor}


# ------------------------------------------------------------------------------------------------ key hashing
def _mix64(k: torch.Tensor) -> torch.Tensor:
    """64-bit finaliser (splitmix64 constants) on int64 tensors; wraps like the device kernels do."""
    k = k ^ (k >> 30)
    k = k * -4658895280553007687      # 0xBF58476D1CE4E5B9 as a signed 64-bit integer
    k = k ^ (k >> 27)
    k = k * -7723592293110705685      # 0x94D049BB133111EB
    return k ^ (k >> 31)


def owner_of(keys: torch.Tensor, world: int) -> torch.Tensor:
    return (_mix64(keys) & 0x7FFFFFFF) % world


# ------------------------------------------------------------------------------------------------ stores
class RowStore:
    """key -> row of ``line`` floats. Rows live in a dense tensor on ``device``; the key index is a sorted
    key array (searchsorted) that is rebuilt on insertion — the device-resident hash-table kernels of
    csrc/kernels/embedding_store.cu replace it on CUDA when the library provides them."""

    def __init__(self, line, device, capacity, table_inits, embedding_dim, seed=0):
        self.line, self.device, self.capacity = line, torch.device(device), int(capacity)
        self.embedding_dim, self.inits, self.seed = embedding_dim, table_inits, seed
        self.keys = torch.empty(0, dtype=torch.int64, device=self.device)
        self.slot = torch.empty(0, dtype=torch.int64, device=self.device)
        self.values = torch.zeros((min(self.capacity, 1024), line), dtype=torch.float32, device=self.device)
        self.size = 0

    def _grow(self, need):
        if need <= self.values.shape[0]:
            return
        if need > self.capacity:
            raise RuntimeError(f"embedding store is full: {need} rows needed, capacity {self.capacity}")
        new = min(self.capacity, max(need, self.values.shape[0] * 2))
        v = torch.zeros((new, self.line), dtype=torch.float32, device=self.device)
        v[:self.size] = self.values[:self.size]
        self.values = v

    def _init_rows(self, keys, table_ids):
        n = keys.numel()
        rows = torch.zeros((n, self.line), dtype=torch.float32, device=self.device)
        emb = rows[:, :self.embedding_dim]
        for t, init in enumerate(self.inits):
            sel = (table_ids == t).nonzero()[:, 0]
            if sel.numel() == 0:
                continue
            gen = torch.Generator(device=self.device).manual_seed((self.seed * 1315423911 + t * 2654435761 + self.size) & 0x7FFFFFFF)
            if init["type"] == "uniform":
                emb[sel] = torch.rand((sel.numel(), self.embedding_dim), generator=gen, device=self.device) * (init["high"] - init["low"]) + init["low"]
            elif init["type"] == "normal":
                emb[sel] = torch.randn((sel.numel(), self.embedding_dim), generator=gen, device=self.device) * init["std"] + init["mean"]
            elif init["type"] == "trunc_normal":
                v = torch.empty((sel.numel(), self.embedding_dim), device=self.device)
                torch.nn.init.trunc_normal_(v, init["mean"], init["std"], init["a"], init["b"], generator=gen)
                emb[sel] = v
            else:
                emb[sel] = init["value"]
        return rows

    def lookup(self, keys, table_ids, insert=True):
        """Slots of unique ``keys`` (inserting + initialising the missing ones)."""
        n = keys.numel()
        if n == 0:
            return torch.empty(0, dtype=torch.int64, device=self.device)
        pos = torch.searchsorted(self.keys, keys)
        posc = pos.clamp(max=max(self.keys.numel() - 1, 0))
        found = (self.keys[posc] == keys) if self.keys.numel() else torch.zeros(n, dtype=torch.bool, device=self.device)
        slots = torch.full((n,), -1, dtype=torch.int64, device=self.device)
        if self.keys.numel():
            slots[found] = self.slot[posc[found]]
        miss = (~found).nonzero()[:, 0]
        if miss.numel() and insert:
            m = miss.numel()
            self._grow(self.size + m)
            new_slots = torch.arange(self.size, self.size + m, device=self.device)
            self.values[new_slots] = self._init_rows(keys[miss], table_ids[miss])
            slots[miss] = new_slots
            self.size += m
            allk = torch.cat([self.keys, keys[miss]])
            alls = torch.cat([self.slot, new_slots])
            order = torch.argsort(allk)
            self.keys, self.slot = allk[order], alls[order]
        return slots

    def rows(self, slots):
        return self.values[slots]

    def put(self, slots, rows):
        self.values[slots] = rows

    def snapshot(self):
        return {"keys": self.keys.cpu(), "slot": self.slot.cpu(), "values": self.values[:self.size].cpu(), "size": self.size}

    def load_snapshot(self, snap):
        self.size = int(snap["size"])
        self._grow(self.size)
        self.values[:self.size] = snap["values"].to(self.device)
        self.keys, self.slot = snap["keys"].to(self.device), snap["slot"].to(self.device)


# ------------------------------------------------------------------------------------------------ sparse row optimizers
def _row_update(kind, rows, grad, D, hyper, step):
    """rows: [n, line] fp32 lines ``[w | state...]``; grad: [n, D] fp32. Updates in place.
    Maths as in oneflow/user/kernels/one_embedding_update_kernels.cu :60-110."""
    lr, wd = hyper["lr"], hyper.get("weight_decay", 0.0)
    w = rows[:, :D]
    g = grad * hyper.get("scale", 1.0)
    if hyper.get("l2", 0.0):
        g = g + hyper["l2"] * w
    if kind == "sgd":
        w -= lr * (g + wd * w)
    elif kind == "momentum":
        m = rows[:, D:2 * D]
        m.mul_(hyper["momentum"]).add_(g)
        w -= lr * (m + wd * w)
    elif kind == "smart_decay_adam":
        # rows remember the step of their last update (first value after the moments): the moments decay by
        # beta^(steps since then) and the missed steps along the first moment are caught up at once
        # (oneflow/user/kernels/one_embedding_update_kernels.cu:140-186; no bias correction, no weight decay)
        m, v = rows[:, D:2 * D], rows[:, 2 * D:3 * D]
        last = rows[:, 3 * D].view(torch.int32)             # the step counter is kept as an integer in the float slot
        b1, b2, eps = hyper["beta1"], hyper["beta2"], hyper["eps"]
        skip = (int(step) - last).clamp_(min=1).to(rows.dtype)[:, None]
        catchup = torch.where(skip > 1, m * b1 * (1 - b1 ** (skip - 1)) / (1 - b1), torch.zeros_like(m))
        m.copy_(b1 ** skip * m + (1 - b1) * g)
        v.copy_(b2 ** skip * v + (1 - b2) * g * g)
        w -= lr * (m + catchup) / (v.sqrt() + eps)
        last.fill_(int(step))
    elif kind == "adam":
        m, v = rows[:, D:2 * D], rows[:, 2 * D:3 * D]
        b1, b2, eps = hyper["beta1"], hyper["beta2"], hyper["eps"]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1 = 1 - b1 ** step if hyper.get("do_bias_correction", True) else 1.0
        bc2 = 1 - b2 ** step if hyper.get("do_bias_correction", True) else 1.0
        w -= (lr / bc1) * m / (v.sqrt() / math.sqrt(bc2) + eps) + lr * wd * w
    elif kind == "adagrad":
        s = rows[:, D:2 * D]
        s.addcmul_(g, g)
        lr_t = lr / (1 + (step - 1) * hyper.get("lr_decay", 0.0))
        w -= lr_t * g / (s.sqrt() + hyper.get("eps", 1e-10)) + lr * wd * w
    elif kind == "ftrl":
        acc, z = rows[:, D:2 * D], rows[:, 2 * D:3 * D]
        lp, l1, l2, beta = hyper.get("lr_power", -0.5), hyper.get("lambda1", 0.0), hyper.get("lambda2", 0.0), hyper.get("beta", 0.0)
        new_acc = acc + g * g
        sigma = (new_acc.pow(-lp) - acc.pow(-lp)) / lr
        z.add_(g - sigma * w)
        acc.copy_(new_acc)
        denom = (beta + new_acc.pow(-lp)) / lr + l2
        w.copy_(torch.where(z.abs() > l1, -(z - torch.sign(z) * l1) / denom, torch.zeros_like(z)))
    else:
        raise ValueError(f"unknown sparse optimizer {kind}")


_STATE_FACTOR = {"sgd": 1, "momentum": 2, "adam": 3, "smart_decay_adam": 4, "adagrad": 2, "ftrl": 3}


# ------------------------------------------------------------------------------------------------ exchange helpers
def _all_to_all_v(send: torch.Tensor, send_counts: List[int], group=None):
    """Variable all-to-all of rows. Returns (received rows, recv_counts)."""
    world = dist.get_world_size(group)
    counts = torch.tensor(send_counts, dtype=torch.int64, device=send.device if send.is_cuda else "cpu")
    all_counts = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    me = dist.get_rank(group)
    recv_counts = [int(c[me]) for c in all_counts]
    out = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    if send.is_cuda:
        dist.all_to_all_single(out, send.contiguous(), recv_counts, send_counts, group=group)
    else:
        sp = list(send.split(send_counts))
        rp = list(out.split(recv_counts))
        reqs = []
        for r in range(world):
            if r == me:
                rp[r].copy_(sp[r])
            else:
                if send_counts[r]:
                    reqs.append(dist.isend(sp[r].contiguous(), r, group=group))
                if recv_counts[r]:
                    reqs.append(dist.irecv(rp[r], r, group=group))
        for q in reqs:
            q.wait()
    return out, recv_counts


class _LookupFn(torch.autograd.Function):
    """Forward: the id + embedding shuffles. Backward: the gradient shuffle and the sparse update."""

    @staticmethod
    def forward(ctx, shadow, emb, keys, table_ids, out_shape):
        ctx.emb = emb
        out, ctx.plan = emb._forward_impl(keys, table_ids)
        ctx.out_shape = out_shape
        return out.view(out_shape)

    @staticmethod
    def backward(ctx, grad):
        ctx.emb._backward_impl(grad.reshape(-1, grad.shape[-1]), ctx.plan)
        return torch.zeros_like(ctx.emb.shadow), None, None, None, None


class Embedding(torch.nn.Module):
    def __init__(self, name, embedding_dim, dtype, key_type, tables, store_options, default_initializer=None, padding_idx=None,
                 seed=0):
        super().__init__()
        self.name, self.embedding_dim, self.dtype, self.key_type = name, int(embedding_dim), dtype, key_type
        self.tables = list(tables)
        self.store_options = store_options
        self.padding_idx = padding_idx
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.seed = seed
        default = default_initializer or make_normal_initializer(0.0, 0.05)
        self.inits = [t.get("initializer", default) if "columns" not in t else t["columns"][0]["initializer"] for t in self.tables]
        self.size_factor = int(store_options.get("size_factor", 1))
        self.storage_dim = self.size_factor * self.embedding_dim
        caches = store_options["kv_store"]["caches"]
        cap = None
        for c in caches:
            if "capacity" in c:
                cap = c["capacity"]
        if cap is None:
            cap = store_options["kv_store"]["persistent_table"].get("capacity_hint", 1 << 24)
        self.capacity_per_rank = max(1, int(cap) // self.world)
        self.persistent_path = store_options["kv_store"]["persistent_table"].get("path")
        # the reference keeps a scalar "shadow" variable so that the embedding takes part in autograd / graphs
        self.shadow = torch.nn.Parameter(torch.zeros(1))
        self.store: Optional[RowStore] = None
        self.engine = None          # device engine (one_embedding/native.py) once a CUDA batch arrived
        self.max_ids_per_step = int(os.environ.get("ONEFLOW_ONE_EMBEDDING_MAX_IDS_PER_STEP", "0"))
        self.sparse_optimizer = ("sgd", {"lr": 0.0})
        self.step_count = 0
        self.gradient_fp16 = os.environ.get("ONEFLOW_ONE_EMBEDDING_GRADIENT_SHUFFLE_USE_FP16", "1") == "1"
        from . import ops as _ops
        _ops.register(self)                 # reachable by name from the stage ops of flow._C

    # -------------------------------------------------------------- store
    def _ensure_store(self, device):
        if self.store is None:
            full = RowStore(self.storage_dim, device, self.capacity_per_rank, self.inits, self.embedding_dim,
                            seed=self.seed + self.rank)
            caches = self.store_options["kv_store"]["caches"]
            if caches and caches[0].get("policy") == "lru":
                # device LRU cache in front of the full table in host memory or on disk (one_embedding/cached_store.py)
                from . import cached_store as CS
                budget = float(caches[0].get("cache_memory_budget_mb", 64))
                cache_rows = max(32, int(budget * (1 << 20) / (self.storage_dim * 4)))
                host_full = any(c.get("policy") == "full" and c.get("value_memory_kind") == "host" for c in caches[1:])
                pt = self.store_options["kv_store"]["persistent_table"]
                if host_full or not pt.get("path"):
                    backing = CS.HostTable(self.storage_dim, self.capacity_per_rank)
                else:
                    import os as _os
                    path = _os.path.join(pt["path"], f"{self.name}-{self.rank}")
                    _os.makedirs(path, exist_ok=True)
                    backing = CS.SsdTable(self.storage_dim, path, int(pt.get("physical_block_size", 512)))

                def init_rows(keys, table_ids, size, _full=full):
                    _full.size = size
                    return _full._init_rows(keys, table_ids)
                self.store = CS.CachedRowStore(self.storage_dim, device, cache_rows, backing, init_rows)
            else:
                self.store = full
        return self.store

    def set_sparse_optimizer(self, kind, hyper):
        need = _STATE_FACTOR[kind]
        if self.size_factor < need:
            raise ValueError(f"{kind} keeps {need - 1} state vector(s) per row: store_options need size_factor >= {need}")
        self.sparse_optimizer = (kind, hyper)

    # -------------------------------------------------------------- forward / backward
    def forward(self, ids, table_ids=None):
        if ids.dim() == 1:
            ids = ids.unsqueeze(1)
        B, T = ids.shape[0], ids.shape[-1]
        if table_ids is None:
            if len(self.tables) > 1 and T != len(self.tables):
                raise ValueError(f"ids has {T} columns but the embedding has {len(self.tables)} tables")
            table_ids = torch.arange(T, device=ids.device).remainder(len(self.tables)).expand(ids.shape)
        keys = ids.reshape(-1).to(torch.int64)
        tids = table_ids.reshape(-1).to(torch.int64)
        out_shape = tuple(ids.shape) + (self.embedding_dim,)
        return _LookupFn.apply(self.shadow, self, keys, tids, out_shape)

    def _use_engine(self, ids):
        """The device engine serves 16-bit embeddings on CUDA within one node; everything else (CPU tensors,
        fp32 outputs, more than 8 ranks) takes the tensor-op path below."""
        if self.engine is not None:
            return True
        if self.store is not None or self.dtype not in (torch.float16, torch.bfloat16) or self.world > 8:
            return False
        caches = self.store_options["kv_store"]["caches"]
        if caches and caches[0].get("policy") == "lru":
            return False                      # cached host / SSD stores: the device holds an LRU cache, not the table
        if self.embedding_dim % 4 or os.environ.get("ONEFLOW_B200_EMBEDDING_ENGINE", "1") == "0":
            return False
        if any(i["type"] not in ("uniform", "normal", "constant") for i in self.inits):
            return False                      # the device engine draws uniform / normal / constant rows only
        from . import native
        if not native.available(ids.device):
            return False
        kind = self.sparse_optimizer[0]
        state_init = float(self.sparse_optimizer[1].get("initial_accumulator_value", 0.0)) if kind in ("adagrad", "ftrl") else 0.0
        self.engine = native.NativeEmbeddingEngine(
            ids.device, max(ids.numel(), self.max_ids_per_step), self.embedding_dim, self.storage_dim, self.inits,
            self.capacity_per_rank, seed=self.seed, half=self.dtype == torch.float16, state_init=state_init)
        return True

    def _forward_impl(self, ids, tids):
        dev = ids.device
        if ids.is_cuda and self._use_engine(ids):
            nt = max(len(self.tables), 1)
            out = self.engine.forward(ids, tids if nt > 1 else None, insert=True)
            return out.view(-1, self.embedding_dim), {"engine": True}
        store = self._ensure_store(dev)
        nt = max(len(self.tables), 1)
        keys = ids * nt + tids                         # one 64-bit key per (id, table)
        uniq, inverse = torch.unique(keys, return_inverse=True)
        plan = {"inverse": inverse, "n_unique": uniq.numel()}
        if self.world == 1:
            slots = store.lookup(uniq, uniq % nt)
            rows = store.rows(slots)[:, :self.embedding_dim]
            plan.update(slots=slots)
            return rows.to(self.dtype)[inverse], plan
        # 1. id shuffle
        owner = owner_of(uniq, self.world)
        order = torch.argsort(owner, stable=True)
        send_keys = uniq[order]
        send_counts = torch.bincount(owner, minlength=self.world).tolist()
        recv_keys, recv_counts = _all_to_all_v(send_keys, send_counts)
        own_uniq, own_inverse = torch.unique(recv_keys, return_inverse=True)
        # 2. lookup + embedding shuffle
        slots = store.lookup(own_uniq, own_uniq % nt)
        rows = store.rows(slots)[:, :self.embedding_dim].to(self.dtype)
        back, _ = _all_to_all_v(rows[own_inverse], recv_counts)
        unperm = torch.empty_like(order)
        unperm[order] = torch.arange(order.numel(), device=dev)
        plan.update(slots=slots, own_inverse=own_inverse, own_n=own_uniq.numel(), order=order, send_counts=send_counts,
                    recv_counts=recv_counts)
        return back[unperm][inverse], plan

    def _backward_impl(self, grad, plan):
        kind, hyper = self.sparse_optimizer
        D = self.embedding_dim
        self.step_count += 1
        if plan.get("engine"):
            self.engine.backward(grad, kind, hyper, self.step_count)
            return
        seg = torch.zeros((plan["n_unique"], D), dtype=torch.float32, device=grad.device)
        seg.index_add_(0, plan["inverse"], grad.float())
        if self.world > 1:
            # 3. gradient shuffle (fp16/bf16 on the wire by default, like the reference)
            wire = seg[plan["order"]]
            if self.gradient_fp16:
                wire = wire.to(self.dtype if self.dtype in (torch.float16, torch.bfloat16) else torch.float16)
            got, _ = _all_to_all_v(wire, plan["send_counts"])
            seg = torch.zeros((plan["own_n"], D), dtype=torch.float32, device=grad.device)
            seg.index_add_(0, plan["own_inverse"], got.float())
        store = self.store
        rows = store.rows(plan["slots"])
        _row_update(kind, rows, seg, D, hyper, self.step_count)
        store.put(plan["slots"], rows)

    # -------------------------------------------------------------- snapshots
    def save_snapshot(self, snapshot_name):
        store = self.engine if self.engine is not None else self.store
        if store is None or not self.persistent_path:
            return
        d = os.path.join(self.persistent_path, f"rank_{self.rank}", "snapshots", snapshot_name)
        os.makedirs(d, exist_ok=True)
        torch.save(store.snapshot(), os.path.join(d, "rows.pt"))

    def load_snapshot(self, snapshot_name, device="cpu"):
        d = os.path.join(self.persistent_path, f"rank_{self.rank}", "snapshots", snapshot_name)
        snap = torch.load(os.path.join(d, "rows.pt"), weights_only=False)
        if self.engine is not None:
            self.engine.load_snapshot(snap)
        else:
            self._ensure_store(device).load_snapshot(snap)

    def state_dict(self, *args, **kwargs):
        sd = super().state_dict(*args, **kwargs)
        name = [time.strftime("%Y-%m-%d-%H-%M-%S")]
        if dist.is_initialized():
            dist.broadcast_object_list(name, src=0)
        self.save_snapshot(name[0])
        sd[(kwargs.get("prefix", "") or "") + "OneEmbeddingSnapshot"] = name[0]
        return sd

    def load_state_dict(self, state_dict, strict=True, **kwargs):
        sd = dict(state_dict)
        snap = sd.pop("OneEmbeddingSnapshot", None)
        if snap is not None and self.persistent_path:
            dev = self.store.device if self.store is not None else ("cuda" if torch.cuda.is_available() else "cpu")
            self.load_snapshot(snap, dev)
        return super().load_state_dict(sd, strict=False)


class MultiTableEmbedding(Embedding):
    """All tables share ``embedding_dim``; column j of ``ids`` addresses table j."""


class MultiTableMultiColumnEmbedding(Embedding):
    """Tables whose rows are made of several columns with their own initializers (summed dims == embedding_dim)."""


from ..optim.optimizer import Ftrl  # noqa: E402  (the dense FTRL optimizer; sparse rows take the FTRL row update)


class SmartDecayAdam(torch.optim.Adam):
    """Names the sparse-aware Adam for ``one_embedding.Optimizer``: every embedding row remembers the step of its last
    update, its moments decay by ``beta ** (steps since then)`` and the skipped steps are caught up in one move (the
    row update of ``_row_update`` / csrc/comm/emb_shuffle.cu, kind 5; it needs ``size_factor >= 4``). As a dense
    optimizer on ordinary parameters, where every element is touched every step, it is Adam."""


class Optimizer:
    """Binds a dense-style optimizer configuration to the sparse row update of an Embedding: after
    ``loss.backward()`` the rows touched by the step are already updated (fused lookup-grad + update + put);
    ``step()`` only advances the schedule."""

    def __init__(self, embedding: Embedding, optimizer_cls=None, **hyper):
        cls = optimizer_cls or torch.optim.SGD
        name = cls.__name__.lower() if isinstance(cls, type) else str(cls).lower()
        lr = hyper.pop("lr", 1e-3)
        if "sgd" in name:
            mom = hyper.pop("momentum", 0.0)
            kind, h = ("momentum", {"lr": lr, "momentum": mom}) if mom else ("sgd", {"lr": lr})
        elif "smartdecay" in name:
            b = hyper.pop("betas", (0.9, 0.999))
            kind, h = "smart_decay_adam", {"lr": lr, "beta1": b[0], "beta2": b[1], "eps": hyper.pop("eps", 1e-8)}
        elif "adam" in name:
            b = hyper.pop("betas", (0.9, 0.999))
            kind, h = "adam", {"lr": lr, "beta1": b[0], "beta2": b[1], "eps": hyper.pop("eps", 1e-8),
                               "do_bias_correction": hyper.pop("do_bias_correction", True)}
        elif "adagrad" in name:
            kind, h = "adagrad", {"lr": lr, "lr_decay": hyper.pop("lr_decay", 0.0), "eps": hyper.pop("eps", 1e-10)}
        elif "ftrl" in name:
            kind, h = "ftrl", {"lr": lr, "lr_power": hyper.pop("lr_power", -0.5), "lambda1": hyper.pop("lambda1", 0.0),
                               "lambda2": hyper.pop("lambda2", 0.0), "beta": hyper.pop("beta", 0.0)}
        else:
            raise ValueError(f"unsupported optimizer for OneEmbedding: {cls}")
        h["weight_decay"] = hyper.pop("weight_decay", 0.0)
        h.update(hyper)
        self.embedding, self.kind, self.hyper = embedding, kind, h
        embedding.set_sparse_optimizer(kind, h)
        self.param_groups = [{"params": [embedding.shadow], "lr": lr}]

    def step(self):
        self.hyper["lr"] = self.param_groups[0]["lr"]

    def zero_grad(self, set_to_none=True):
        self.embedding.shadow.grad = None

    def state_dict(self):
        return {"kind": self.kind, "hyper": dict(self.hyper), "step": self.embedding.step_count}

    def load_state_dict(self, sd):
        self.hyper.update(sd["hyper"])
        self.embedding.step_count = sd["step"]


# ------------------------------------------------------------------------------------------------ offline table access
_NP = {torch.int64: "int64", torch.int32: "int32", torch.uint64: "uint64", torch.uint32: "uint32", torch.float32: "float32",
       torch.float16: "float16", torch.float64: "float64", torch.bfloat16: None}


def _np_dtype(dt):
    import numpy as np
    if isinstance(dt, torch.dtype):
        name = _NP.get(dt)
        if name is None:
            raise TypeError(f"persistent tables hold numpy-representable values, not {dt}")
        return np.dtype(name)
    return np.dtype(dt)


class PersistentTableWriter:
    """Writes (key, row) pairs into one persistent table directory per path, keys assigned to paths round robin by
    ``key % len(paths)`` — the parallel layout a sharded embedding loads — and seals them with a snapshot on
    :meth:`close` (reference: oneflow/api/python/framework/one_embedding.cpp, ``PersistentTableWriterImpl``)."""

    def __init__(self, paths, snapshot_name, key_type, value_type, storage_dim, target_chunk_size_mb=4096,
                 physical_block_size=4096):
        from ..runtime.core import PersistentTable
        self.key_dtype, self.value_dtype = _np_dtype(key_type), _np_dtype(value_type)
        self.storage_dim, self.snapshot_name = int(storage_dim), snapshot_name
        self.tables = [PersistentTable(p, self.storage_dim * self.value_dtype.itemsize, physical_block_size) for p in paths]
        self.closed = False

    def write(self, keys, values):
        import numpy as np
        keys = np.ascontiguousarray(keys).astype(np.int64).reshape(-1)
        values = np.ascontiguousarray(values, dtype=self.value_dtype).reshape(keys.size, self.storage_dim)
        n = len(self.tables)
        for i, t in enumerate(self.tables):
            sel = (keys % n) == i if n > 1 else slice(None)
            if n == 1 or sel.any():
                t.put(keys[sel], values[sel])

    def close(self):
        if not self.closed:
            for t in self.tables:
                t.save_snapshot(self.snapshot_name)
                t.close()
            self.closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


class PersistentTableReader:
    """Iterates ``(keys, values)`` numpy batches of at most 65536 rows over the named snapshot of each table path
    (reference: oneflow/api/python/framework/one_embedding.cpp:194-275)."""

    kBatchSize = 65536

    def __init__(self, paths, snapshot_name, key_type, value_type, storage_dim, target_chunk_size_mb=4096,
                 physical_block_size=4096):
        from ..runtime.core import PersistentTable
        self.key_dtype, self.value_dtype = _np_dtype(key_type), _np_dtype(value_type)
        self.storage_dim = int(storage_dim)
        self.tables = []
        for p in paths:
            t = PersistentTable(p, self.storage_dim * self.value_dtype.itemsize, physical_block_size, read_only=True)
            t.load_snapshot(snapshot_name)
            self.tables.append(t)
        self._cur, self._keys, self._off = 0, None, 0
        self.closed = False

    def __iter__(self):
        return self

    def __next__(self):
        while self._cur < len(self.tables):
            if self._keys is None:
                self._keys, self._off = self.tables[self._cur].keys(), 0
            if self._off < self._keys.size:
                k = self._keys[self._off:self._off + self.kBatchSize]
                self._off += k.size
                v, _ = self.tables[self._cur].get(k, dtype=self.value_dtype)
                return k.astype(self.key_dtype), v.reshape(k.size, self.storage_dim)
            self._cur, self._keys = self._cur + 1, None
        raise StopIteration

    next = __next__

    def close(self):
        if not self.closed:
            for t in self.tables:
                t.close()
            self.closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def make_persistent_table_reader(paths, snapshot_name, key_type, value_type, storage_dim, physical_block_size=4096):
    """reference: python/oneflow/one_embedding.py:1240-1261"""
    return PersistentTableReader(paths, snapshot_name, key_type, value_type, storage_dim, 4 * 1024, physical_block_size)


def make_persistent_table_writer(paths, snapshot_name, key_type, value_type, storage_dim, physical_block_size=4096):
    """reference: python/oneflow/one_embedding.py:1264-1285"""
    return PersistentTableWriter(paths, snapshot_name, key_type, value_type, storage_dim, 4 * 1024, physical_block_size)
