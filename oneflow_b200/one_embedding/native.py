"""Device-resident OneEmbedding engine: binds csrc/comm/emb_shuffle.cu.

One engine = one rank's table shard (open-addressing key index + fp32 rows with optimizer state in device memory)
plus the exchange buffers in a symmetric arena. ``forward`` runs the id shuffle, the lookup fused with the embedding
shuffle and the final gather as five kernels on the current stream; ``backward`` runs the gradient segment-sum, the
gradient shuffle and the row update as four. Nothing returns to the host in between, and no NCCL call is made.

Reference: python/oneflow/one_embedding.py (MultiTableEmbedding), oneflow/user/kernels/one_embedding_kernels.cu,
one_embedding_id_shuffle_p2p_kernel.cu, one_embedding_update_kernels.cu.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch
import torch.distributed as dist

from ..comm.symmetric import SymmetricArena
from ..ops import _native
from ..ops import kernels as _k


class EmbStoreStruct(Structure):
    _fields_ = [("slots", c_void_p), ("rows", c_void_p),
                ("row_key", c_void_p), ("counters", c_void_p), ("init_kind", c_void_p), ("init_a", c_void_p), ("init_b", c_void_p),
                ("tcap", c_longlong), ("row_cap", c_longlong), ("line", c_int), ("dim", c_int), ("num_tables", c_int),
                ("state_init", c_float), ("seed", c_ulonglong)]


class EmbShuffleStruct(Structure):
    _fields_ = [("keys_off", c_longlong), ("cnt_off", c_longlong), ("emb_off", c_longlong), ("grad_off", c_longlong),
                ("cap", c_longlong), ("dkeys", c_void_p), ("dval", c_void_p), ("dcap", c_longlong), ("cnt", c_void_p),
                ("inv", c_void_p), ("gsum", c_void_p), ("slot_tmp", c_void_p), ("rowidx", c_void_p), ("uoidx", c_void_p),
                ("u_row", c_void_p), ("gacc", c_void_p), ("n_uo", c_void_p), ("done", c_void_p)]


class EmbUpdateStruct(Structure):
    _fields_ = [("kind", c_int)] + [(k, c_float) for k in (
        "lr", "lr_eff", "scale", "weight_decay", "l2", "momentum", "beta1", "beta2", "eps", "bias_corr1", "bias_corr2",
        "lr_power", "lambda1", "lambda2", "beta")] + [("step", c_int)]


_KIND = {"sgd": 0, "momentum": 1, "adam": 2, "smart_decay_adam": 5, "adagrad": 3, "ftrl": 4}
_INIT = {"uniform": 0, "normal": 1, "constant": 2}


def _pow2(n):
    return 1 << max(int(n) - 1, 1).bit_length()


def available(device) -> bool:
    """True on CUDA devices. A missing or stale kernel library raises there instead of silently selecting the
    tensor-op path."""
    if torch.device(device).type != "cuda":
        return False
    if not hasattr(_native.kernels(), "ofb_emb_forward"):
        raise _native.NativeLibraryError("libofb_kernels.so lacks the embedding kernels: rebuild with python -m oneflow_b200.build")
    return True


class NativeEmbeddingEngine:
    def __init__(self, device, max_ids, dim, line, inits, row_capacity, seed=0, half=False, group=None, state_init=0.0, solo=False):
        self.device = torch.device(device)
        self.dim, self.line, self.half = int(dim), int(line), bool(half)
        if self.dim % 4:
            raise ValueError("embedding_dim must be a multiple of 4 for the device engine")
        if dist.is_initialized() and not solo:
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
        else:
            self.world, self.rank, ranks = 1, 0, [0]
        if self.world > 8:
            raise ValueError("the device engine addresses at most 8 peers")
        N, D = self.world, self.dim
        dev = self.device
        i32, i64, f32 = torch.int32, torch.int64, torch.float32
        # ---- table shard
        self.row_cap = int(row_capacity)
        self.tcap = _pow2(2 * self.row_cap)
        # key index: 32-byte slots {key u64 = all ones (empty), row i32 = -1, uo i32, stamp u32, pad}
        self.slots = torch.zeros((self.tcap, 4), dtype=i64, device=dev)
        self.slots[:, 0] = -1
        self.slots[:, 1] = 0xFFFFFFFF
        self.rows = torch.empty((self.row_cap, self.line), dtype=f32, device=dev)
        self.row_key = torch.empty((self.row_cap,), dtype=i64, device=dev)
        self.counters = torch.zeros((4,), dtype=i32, device=dev)
        self.init_kind = torch.tensor([_INIT[i["type"]] for i in inits], dtype=i32, device=dev)
        a, b = [], []
        for i in inits:
            if i["type"] == "uniform":
                a.append(i["low"]); b.append(i["high"])
            elif i["type"] == "normal":
                a.append(i["mean"]); b.append(i["std"])
            else:
                a.append(i["value"]); b.append(0.0)
        self.init_a = torch.tensor(a, dtype=f32, device=dev)
        self.init_b = torch.tensor(b, dtype=f32, device=dev)
        self.num_tables = len(inits)
        self.group, self._ranks, self.arena = group, ranks, None
        self.epoch = 0   # step number: never reset, the table's touch stamps compare against it
        self._alloc_exchange(max(int(max_ids), 1024))
        st = EmbStoreStruct()
        for name in ("slots", "rows", "row_key", "counters", "init_kind", "init_a", "init_b"):
            setattr(st, name, getattr(self, name).data_ptr())
        st.tcap, st.row_cap, st.line, st.dim, st.num_tables = self.tcap, self.row_cap, self.line, D, self.num_tables
        st.state_init, st.seed = float(state_init), int(seed) & 0xFFFFFFFFFFFFFFFF
        self.st = st

    def _alloc_exchange(self, cap):
        """(Re)creates the symmetric exchange buffers and the per-step scratch for ``cap`` ids per rank and step.
        Collective over the engine's ranks; the table shard is untouched."""
        if self.arena is not None:
            torch.cuda.synchronize(self.device)
            self.arena.close()
        self.cap = cap
        N, D, dev = self.world, self.dim, self.device
        i32, i64, f32 = torch.int32, torch.int64, torch.float32
        row_bytes = D * 2
        need = N * self.cap * 8 + 4096 + 2 * (N * self.cap * row_bytes) + (1 << 16)
        self.arena = SymmetricArena(self.group, self._ranks, dev, need)
        sh = EmbShuffleStruct()
        sh.keys_off = self.arena.region(N * self.cap * 8)
        sh.cnt_off = self.arena.region(4096)
        sh.emb_off = self.arena.region(N * self.cap * row_bytes)
        sh.grad_off = self.arena.region(N * self.cap * row_bytes)
        sh.cap = self.cap
        self.dcap = _pow2(2 * self.cap)
        self.dkeys = torch.empty((self.dcap,), dtype=i64, device=dev)
        self.dval = torch.empty((self.dcap,), dtype=i32, device=dev)
        self.cnt = torch.zeros((8,), dtype=i32, device=dev)
        self.inv = torch.empty((self.cap,), dtype=i32, device=dev)
        self.gsum = torch.zeros((N * self.cap, D), dtype=f32, device=dev)
        self.slot_tmp = torch.empty((N * self.cap,), dtype=i32, device=dev)
        self.rowidx = torch.empty((N * self.cap,), dtype=i32, device=dev)
        self.uoidx = torch.empty((N * self.cap,), dtype=i32, device=dev)
        self.u_row = torch.empty((N * self.cap,), dtype=i32, device=dev)
        self.gacc = torch.zeros((N * self.cap, D), dtype=f32, device=dev)
        self.n_uo = torch.zeros((1,), dtype=i32, device=dev)
        self.done = torch.zeros((2,), dtype=i32, device=dev)
        for name in ("dkeys", "dval", "cnt", "inv", "gsum", "slot_tmp", "rowidx", "uoidx", "u_row", "gacc", "n_uo", "done"):
            setattr(sh, name, getattr(self, name).data_ptr())
        sh.dcap = self.dcap
        self.sh = sh
        self._n_last = 0

    # ------------------------------------------------------------------ step
    def forward(self, ids, table_ids=None, insert=True):
        """ids: int64 [..., columns] on this engine's device -> [..., columns, dim] (bf16, or fp16 when ``half``)."""
        ids = ids.contiguous()
        n = ids.numel()
        if n > self.cap:
            if self.world > 1:
                raise ValueError(f"{n} ids in one step but the exchange buffers were sized for {self.cap}: set "
                                 "ONEFLOW_ONE_EMBEDDING_MAX_IDS_PER_STEP to the largest per-rank id count")
            self._alloc_exchange(max(n, 2 * self.cap))
        columns = ids.shape[-1] if ids.dim() > 1 else 1
        tids = None if table_ids is None else table_ids.to(torch.int32).contiguous()
        out = torch.empty(tuple(ids.shape) + (self.dim,), dtype=torch.float16 if self.half else torch.bfloat16, device=self.device)
        self.epoch += 1
        _native.check(_native.kernels().ofb_emb_forward(
            ctypes.byref(self.arena.ctx), ctypes.byref(self.st), ctypes.byref(self.sh), _native.ptr(ids), _native.ptr(tids),
            c_longlong(n), c_int(columns), c_int(int(insert)), c_uint(self.epoch), _native.ptr(out), c_int(int(self.half)),
            _native.stream_ptr()), "emb_forward")
        _k._count(5)
        self._n_last = n
        return out

    def backward(self, grad, kind, hyper, step):
        """Applies the gradient of the most recent ``forward`` (one step may be outstanding at a time)."""
        grad = grad.contiguous()
        want = torch.float16 if self.half else torch.bfloat16
        if grad.dtype != want:
            grad = grad.to(want)
        n = grad.numel() // self.dim
        if n != self._n_last:
            raise ValueError("gradient does not match the last forward")
        u = EmbUpdateStruct()
        u.kind = _KIND[kind]
        lr = float(hyper["lr"])
        u.lr, u.scale = lr, float(hyper.get("scale", 1.0))
        u.weight_decay, u.l2 = float(hyper.get("weight_decay", 0.0)), float(hyper.get("l2", 0.0))
        u.momentum = float(hyper.get("momentum", 0.0))
        u.beta1, u.beta2 = float(hyper.get("beta1", 0.9)), float(hyper.get("beta2", 0.999))
        u.eps = float(hyper.get("eps", 1e-8 if u.kind == 2 else 1e-10))
        bc = hyper.get("do_bias_correction", True)
        u.bias_corr1 = 1.0 - u.beta1 ** step if bc else 1.0
        u.bias_corr2 = 1.0 - u.beta2 ** step if bc else 1.0
        u.lr_eff = lr / (1.0 + (step - 1) * float(hyper.get("lr_decay", 0.0)))
        u.lr_power, u.lambda1 = float(hyper.get("lr_power", -0.5)), float(hyper.get("lambda1", 0.0))
        u.lambda2, u.beta = float(hyper.get("lambda2", 0.0)), float(hyper.get("beta", 0.0))
        u.step = int(step)
        _native.check(_native.kernels().ofb_emb_backward(
            ctypes.byref(self.arena.ctx), ctypes.byref(self.st), ctypes.byref(self.sh), _native.ptr(grad), c_longlong(n),
            c_int(int(self.half)), c_uint(self.epoch), ctypes.byref(u), _native.stream_ptr()), "emb_backward")
        _k._count(4)

    # ------------------------------------------------------------------ inspection / snapshots
    @property
    def size(self):
        return int(self.counters[0].item())

    def find(self, keys, insert=False):
        keys = keys.to(self.device, torch.int64).contiguous()
        rows = torch.empty((keys.numel(),), dtype=torch.int32, device=self.device)
        _native.check(_native.kernels().ofb_emb_find(ctypes.byref(self.st), _native.ptr(keys), c_longlong(keys.numel()),
                                                     c_int(int(insert)), _native.ptr(rows), _native.stream_ptr()), "emb_find")
        _k._count()
        return rows

    def snapshot(self):
        n = self.size
        return {"keys": self.row_key[:n].cpu(), "slot": torch.arange(n), "values": self.rows[:n].cpu(), "size": n}

    def load_snapshot(self, snap):
        keys = snap["keys"].to(self.device)
        vals = snap["values"].to(self.device, torch.float32)
        if "slot" in snap:
            vals = vals[snap["slot"].to(self.device)]
        rows = self.find(keys, insert=True).long()
        if (rows < 0).any():
            raise RuntimeError("embedding store is full while loading a snapshot")
        self.rows[rows, :vals.shape[1]] = vals
