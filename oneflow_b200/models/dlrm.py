"""DLRM with a model-parallel OneEmbedding and data-parallel MLPs.

    dense [B, 13] --bottom MLP (13 -> 512 -> 256 -> 128, ReLU)--------------\\
    ids   [B, 26] --OneEmbedding (26 tables, dim 128, hash-sharded rows)-----+--> dot feature interaction
                                                                                  [dense | 351 pair products | pad]
                                   --top MLP (480 -> 1024 -> 1024 -> 512 -> 256 -> 1)--> BCE with logits

Two forms of the same network:

* ``DLRMTrainer`` — the training engine: explicit forward / backward over a flat parameter store (every Linear is
  one tcgen05 GEMM whose epilogue applies bias + ReLU, or ReLU' for the input gradient), the device embedding engine
  (id shuffle, lookup + embedding shuffle, gradient shuffle + SGD row update over peer memory), the fused
  interaction and loss kernels, a fused all-reduce of the MLP gradients and one fused Adam update.
* ``DLRMModule`` — the same network as a module built from the public pieces (``one_embedding.MultiTableEmbedding``,
  ``nn.FusedMLP``, ``_C.fused_dot_feature_interaction``) for autograd / nn.Graph use.

Model definition after the reference's DLRM example that its OneEmbedding documentation describes
(python/oneflow/one_embedding.py:MultiTableEmbedding docstring; kernels in
oneflow/user/kernels/fused_dot_feature_interaction_kernel.cu, cublas_fused_mlp_kernel.cu, one_embedding_kernels.cu).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import gemm as G
from ..ops import kernels as K
from .gpt import ParamStore


@dataclass
class DLRMConfig:
    num_dense: int = 13
    num_tables: int = 26
    embedding_dim: int = 128
    bottom: Tuple[int, ...] = (512, 256, 128)
    top: Tuple[int, ...] = (1024, 1024, 512, 256, 1)
    table_rows: Tuple[int, ...] = (40_000_000, 10_000_000, 1_000_000, 100_000)   # cycled over the tables
    zipf_alpha: float = 1.05
    global_batch: int = 55296
    positive_rate: float = 0.25
    dense_lr: float = 1e-3
    embedding_lr: float = 0.05
    rows_capacity: int = 1 << 24          # embedding rows this job may touch (all ranks together)

    @property
    def dense_pad(self):
        return (self.num_dense + 7) // 8 * 8

    @property
    def interaction_dim(self):
        f = self.num_tables + 1
        return (self.embedding_dim + f * (f - 1) // 2 + 7) // 8 * 8

    def rows_of(self, table):
        return self.table_rows[table % len(self.table_rows)]


def tiny_config(**kw):
    base = dict(num_tables=6, embedding_dim=32, bottom=(64, 32), top=(64, 32, 1), table_rows=(5000, 700, 90), global_batch=256,
                rows_capacity=1 << 14)
    base.update(kw)
    return DLRMConfig(**base)


def make_batch(cfg: DLRMConfig, batch: int, seed: int = 0, pin: bool = False):
    """Synthetic batch on the host: dense = log(1 + Exp(1)) padded with zero columns to a multiple of 8 (fp32),
    ids ~ truncated Zipf(alpha) per table (int64), labels ~ Bernoulli(positive_rate) (fp32)."""
    g = torch.Generator().manual_seed(seed)
    dense = torch.zeros(batch, cfg.dense_pad)
    dense[:, :cfg.num_dense] = torch.log1p(torch.empty(batch, cfg.num_dense).exponential_(1.0, generator=g))
    ids = torch.empty(batch, cfg.num_tables, dtype=torch.int64)
    e = 1.0 - cfg.zipf_alpha
    for t in range(cfg.num_tables):
        n = cfg.rows_of(t)
        u = torch.rand(batch, generator=g, dtype=torch.float64)
        x = (1.0 + u * (n ** e - 1.0)) ** (1.0 / e) if abs(e) > 1e-9 else torch.exp(u * math.log(n))
        ids[:, t] = (x.floor().long() - 1).clamp_(0, n - 1)
    labels = (torch.rand(batch, generator=g) < cfg.positive_rate).float()
    if pin and torch.cuda.is_available():
        dense, ids, labels = dense.pin_memory(), ids.pin_memory(), labels.pin_memory()
    return dense, ids, labels


def _mlp_specs(prefix, dims, pad_last=False):
    specs = []
    for i in range(len(dims) - 1):
        fan_in, fan_out = dims[i], dims[i + 1]
        out_pad = (fan_out + 7) // 8 * 8 if pad_last and i == len(dims) - 2 else fan_out
        specs.append((f"{prefix}.{i}.w", (out_pad, fan_in), False, math.sqrt(2.0 / (fan_in + fan_out))))
        specs.append((f"{prefix}.{i}.b", (out_pad,), False, math.sqrt(1.0 / fan_out)))
    return specs


class DLRMTrainer:
    """One rank of a DLRM training job (data-parallel MLPs, model-parallel embedding)."""

    def __init__(self, cfg: DLRMConfig, device, group=None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group = group
        if cfg.global_batch % self.world:
            raise ValueError("global batch must divide by the number of ranks")
        self.local_batch = cfg.global_batch // self.world
        D = cfg.embedding_dim
        if cfg.bottom[-1] != D:
            raise ValueError("the bottom MLP must end at the embedding dimension")
        self.bottom_dims = [cfg.dense_pad] + list(cfg.bottom)
        self.top_dims = [cfg.interaction_dim] + list(cfg.top)
        self.store = ParamStore(_mlp_specs("bottom", self.bottom_dims) + _mlp_specs("top", self.top_dims, pad_last=True), self.device)
        self.store.init_(seed)
        # rows and columns that only exist as padding stay zero: padded inputs are zero anyway, padded outputs get no gradient
        self.store.p["bottom.0.w"][:, cfg.num_dense:].zero_()
        last = len(self.top_dims) - 2
        self.store.p[f"top.{last}.w"][cfg.top[-1]:].zero_()
        self.store.p[f"top.{last}.b"][cfg.top[-1]:].zero_()
        from ..parallel.engine import FlatAdamW
        zero = None
        if self.world > 1:
            from ..parallel.zero import GradAllReduce
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
            zero = GradAllReduce(group, ranks, self.device, io_bytes=max(16 << 20, self.store.total * 4 + (1 << 20)))
        self.opt = FlatAdamW(self.store, lr=cfg.dense_lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, clip_grad=None, zero=zero)
        inits = [{"type": "uniform", "low": -math.sqrt(1.0 / cfg.rows_of(t)), "high": math.sqrt(1.0 / cfg.rows_of(t))}
                 for t in range(cfg.num_tables)]
        self.engine = None
        self.emb_module = None
        if self.device.type == "cuda":
            from ..one_embedding.native import NativeEmbeddingEngine
            self.engine = NativeEmbeddingEngine(self.device, self.local_batch * cfg.num_tables, D, D, inits,
                                                max(1024, cfg.rows_capacity // self.world), seed=seed, group=group)
        else:
            from .. import one_embedding as oe
            tables = [oe.make_table_options(i) for i in inits]
            opts = oe.make_device_mem_store_options(None, capacity=cfg.rows_capacity)
            self.emb_module = oe.MultiTableEmbedding("sparse", D, torch.bfloat16, torch.int64, tables, opts, seed=seed)
        self.emb_hyper = {"lr": cfg.embedding_lr, "scale": 1.0 / self.world}
        if self.emb_module is not None:
            self.emb_module.set_sparse_optimizer("sgd", self.emb_hyper)
        self.steps = 0
        self._tids = None
        self.keep_trace = False     # tests: keep the last step's activations and activation gradients
        self.trace = None
        # the embedding shuffles run on their own stream, next to the bottom MLP (forward) and its gradients + the
        # dense optimizer (backward), like the reference's dedicated <name>_EMBEDDING / _ID_SHUFFLE streams
        self.emb_stream = torch.cuda.Stream(device=self.device) if self.engine is not None else None

    # ------------------------------------------------------------------ pieces
    def _emb_forward(self, ids):
        if self.engine is not None:
            return self.engine.forward(ids), None
        T = self.cfg.num_tables
        if self._tids is None or self._tids.numel() != ids.numel():
            self._tids = torch.arange(T).repeat(ids.shape[0])
        out, plan = self.emb_module._forward_impl(ids.reshape(-1), self._tids)
        return out.view(ids.shape[0], T, -1), plan

    def _emb_backward(self, grad, plan):
        if self.engine is not None:
            self.engine.backward(grad, "sgd", self.emb_hyper, self.steps)
        else:
            self.emb_module._backward_impl(grad.reshape(-1, grad.shape[-1]), plan)

    def _mlp_forward(self, prefix, x, n_layers, final_relu):
        acts = [x]
        for i in range(n_layers):
            relu = final_relu or i < n_layers - 1
            x = G.gemm(x, self.store.p[f"{prefix}.{i}.w"], bias=self.store.p[f"{prefix}.{i}.b"], act="relu" if relu else 0)
            acts.append(x)
        return acts

    def _mlp_backward(self, prefix, acts, dz, n_layers, need_dx):
        """dz: gradient wrt the pre-activation of the last layer. Returns the gradient wrt the MLP input."""
        st = self.store
        for i in reversed(range(n_layers)):
            wn, bn = f"{prefix}.{i}.w", f"{prefix}.{i}.b"
            G.gemm(dz, acts[i], a_layout="km", b_layout="kn", out=st.g[wn], out_dtype=torch.float32, accumulate=st.acc_flag(wn))
            if not st.acc_flag(bn):
                st.g[bn].zero_()
            K.column_sum(dz, out=st.g[bn])
            if i > 0:
                # input gradient, times ReLU'(output of the previous layer) in the GEMM epilogue
                dz = G.gemm(dz, st.p[wn], b_layout="kn", aux_in=acts[i], act="relu")
            elif need_dx:
                dz = G.gemm(dz, st.p[wn], b_layout="kn")
            else:
                dz = None
        return dz

    # ------------------------------------------------------------------ step
    def forward(self, dense, ids):
        """Inference: click probabilities [B]."""
        x0 = K.cast_scale(dense, out_dtype=torch.bfloat16)
        bottom = self._mlp_forward("bottom", x0, len(self.bottom_dims) - 1, True)
        if self.emb_stream is not None:
            torch.cuda.current_stream().wait_stream(self.emb_stream)   # a row update may still be running there
        emb, _ = self._emb_forward(ids)
        z = K.interaction_fwd(bottom[-1], emb, False, self.cfg.interaction_dim)
        top = self._mlp_forward("top", z, len(self.top_dims) - 1, False)
        return torch.sigmoid(top[-1][:, 0].float())

    def train_step(self, dense, ids, labels):
        """dense fp32 [B, dense_pad], ids int64 [B, tables], labels fp32 [B], all on this rank's device.
        Returns the mean loss of this rank's samples as a device tensor of one element."""
        cfg = self.cfg
        B = dense.shape[0]
        self.steps += 1
        self.store.start_accumulation()
        nb, nt = len(self.bottom_dims) - 1, len(self.top_dims) - 1
        side = self.emb_stream
        if side is not None:
            main = torch.cuda.current_stream()
            side.wait_stream(main)                      # ids are ready; the previous step's row update is on `side` already
            with torch.cuda.stream(side):
                emb, plan = self._emb_forward(ids)
            ids.record_stream(side)
        x0 = K.cast_scale(dense, out_dtype=torch.bfloat16)
        bottom = self._mlp_forward("bottom", x0, nb, True)
        if side is not None:
            main.wait_stream(side)
            emb.record_stream(main)
        else:
            emb, plan = self._emb_forward(ids)
        z = K.interaction_fwd(bottom[-1], emb, False, cfg.interaction_dim)
        top = self._mlp_forward("top", z, nt, False)
        loss, dlogits = K.bce_logits(top[-1], labels, loss_scale=1.0 / B, grad_scale=1.0 / B)
        dz = self._mlp_backward("top", top, dlogits, nt, need_dx=True)
        d_dense, d_sparse = K.interaction_bwd(bottom[-1], emb, dz, False)
        if self.keep_trace:
            self.trace = {"emb": emb, "d_sparse": d_sparse, "logits": top[-1][:, 0], "d_dense": d_dense, "dz": dz, "bottom": bottom[-1]}
        if side is not None:
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self._emb_backward(d_sparse, plan)
            d_sparse.record_stream(side)
        else:
            self._emb_backward(d_sparse, plan)
        # ReLU' of the bottom MLP's output, then its layers
        d_bottom = K.bias_act_bwd(bottom[-1], None, d_dense, 3)
        self._mlp_backward("bottom", bottom, d_bottom, nb, need_dx=False)
        self.opt.step()
        return loss


class DLRMModule(torch.nn.Module):
    """The network as a module over the public API (autograd; CPU or CUDA)."""

    def __init__(self, cfg: DLRMConfig, dtype=torch.float32, store_path=None, seed: int = 0):
        super().__init__()
        from .. import one_embedding as oe
        from ..nn.modules.fused_mlp import FusedMLP
        self.cfg = cfg
        D = cfg.embedding_dim
        self.bottom = FusedMLP(cfg.num_dense, list(cfg.bottom[:-1]), cfg.bottom[-1], skip_final_activation=False, dtype=dtype)
        f = cfg.num_tables + 1
        self.pad = cfg.interaction_dim - (D + f * (f - 1) // 2)
        self.top = FusedMLP(cfg.interaction_dim, list(cfg.top[:-1]), cfg.top[-1], skip_final_activation=True, dtype=dtype)
        tables = [oe.make_table_options(oe.make_uniform_initializer(-math.sqrt(1.0 / cfg.rows_of(t)), math.sqrt(1.0 / cfg.rows_of(t))))
                  for t in range(cfg.num_tables)]
        self.embedding = oe.MultiTableEmbedding("sparse", D, dtype, torch.int64, tables,
                                                oe.make_device_mem_store_options(store_path, capacity=cfg.rows_capacity), seed=seed)

    def forward(self, dense, ids):
        from .. import _C
        x = self.bottom(dense[:, :self.cfg.num_dense].to(self.bottom.weight(0).dtype))
        emb = self.embedding(ids)
        z = _C.fused_dot_feature_interaction([x, emb], output_concat=x, self_interaction=False, output_padding=self.pad)
        return self.top(z)[:, 0]
