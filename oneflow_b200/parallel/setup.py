"""Builds a ready-to-train GPT/BERT trainer for a (dp, pp, tp) decomposition of the job.

Rank layout (tensor-parallel innermost): ``rank = (dp_idx * pp + pp_idx) * tp + tp_idx``. This is the
2-D / 3-D placement hierarchy the reference writes as nested rank lists in ``flow.placement``
(oneflow/api/python/symbol/placement_symbol.cpp:143-152); each mesh axis gets its own process group,
as the reference's EagerCclCommMgr does per hierarchy axis (core/job/eager_nccl_comm_manager.cpp:178).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.gpt import GPTStage
from .engine import FlatAdamW, PipelineP2P, StagedTrainer


class Mesh3D:
    def __init__(self, dp, pp, tp):
        self.dp, self.pp, self.tp = dp, pp, tp
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if dp * pp * tp != self.world:
            raise ValueError(f"dp*pp*tp = {dp * pp * tp} does not match the world size {self.world}")
        self.tp_idx = self.rank % tp
        self.pp_idx = (self.rank // tp) % pp
        self.dp_idx = self.rank // (tp * pp)
        self.tp_group = self.pp_group = self.dp_group = self.embedding_group = None
        self.tp_ranks = [self.rank]
        self.pp_ranks = [self.rank]
        self.dp_ranks = [self.rank]
        if self.world == 1:
            return
        # every rank must create every group, in the same order
        for d in range(dp):
            for p in range(pp):
                ranks = [(d * pp + p) * tp + t for t in range(tp)]
                g = dist.new_group(ranks) if tp > 1 else None
                if self.rank in ranks:
                    self.tp_group, self.tp_ranks = g, ranks
        for d in range(dp):
            for t in range(tp):
                ranks = [(d * pp + p) * tp + t for p in range(pp)]
                g = dist.new_group(ranks) if pp > 1 else None
                e = dist.new_group([ranks[0], ranks[-1]]) if pp > 1 else None
                if self.rank in ranks:
                    self.pp_group, self.pp_ranks = g, ranks
                    if self.rank in (ranks[0], ranks[-1]):
                        self.embedding_group = e
        for p in range(pp):
            for t in range(tp):
                ranks = [(d * pp + p) * tp + t for d in range(dp)]
                g = dist.new_group(ranks) if dp > 1 else None
                if self.rank in ranks:
                    self.dp_group, self.dp_ranks = g, ranks


class _Trainer:
    """The public training handle: ``train_step(tokens)`` runs one optimizer step on this rank's share of
    the global batch (tokens: int64 [n_micro * micro_batch, seq + 1] on the device) and returns the mean
    loss as a 0-d device tensor (meaningful on ranks where ``has_loss``)."""

    def __init__(self, inner, mesh, stage):
        self.inner, self.mesh, self.stage = inner, mesh, stage
        self.has_loss = stage.last

    def train_step(self, tokens):
        return self.inner.train_step(tokens)

    @property
    def optimizer(self):
        return self.inner.opt


def build_gpt_trainer(cfg, tp=1, pp=1, dp=1, micro_batch=4, n_micro=16, device="cuda", lr=1e-4, weight_decay=0.1,
                      clip_grad=1.0, zero_stage=1, seed=0, stage_cls=GPTStage):
    mesh = Mesh3D(dp, pp, tp)
    device = torch.device(device)
    tp_ctx = None
    if tp > 1:
        from .tensor_parallel import TPContext
        tp_ctx = TPContext(mesh.tp_group, mesh.tp_ranks, device, max_tokens=micro_batch * cfg.seq_len,
                           max_cols=max(cfg.ffn // tp, 3 * cfg.hidden // tp, cfg.hidden, cfg.vocab_size // tp),
                           hidden=cfg.hidden)
    per = cfg.layers // pp
    l0 = mesh.pp_idx * per
    l1 = cfg.layers if mesh.pp_idx == pp - 1 else l0 + per
    stage = stage_cls(cfg, l0, l1, first=mesh.pp_idx == 0, last=mesh.pp_idx == pp - 1, device=device, tp=tp_ctx,
                      seed=seed)
    zero = None
    if dp > 1 and zero_stage >= 1:
        from .zero import ZeroShard
        zero = ZeroShard(mesh.dp_group, mesh.dp_ranks, device)
    elif dp > 1:
        from .zero import GradAllReduce
        zero = GradAllReduce(mesh.dp_group, mesh.dp_ranks, device)
    opt = FlatAdamW(stage.store, lr=lr, weight_decay=weight_decay, clip_grad=clip_grad, zero=zero,
                    norm_groups=(mesh.tp_group, mesh.pp_group), tp_size=tp)
    p2p = None
    if pp > 1:
        tokens = micro_batch * cfg.seq_len // tp
        prev_rank = mesh.pp_ranks[mesh.pp_idx - 1] if mesh.pp_idx > 0 else None
        next_rank = mesh.pp_ranks[mesh.pp_idx + 1] if mesh.pp_idx < pp - 1 else None
        p2p = PipelineP2P(None, prev_rank, next_rank, (tokens, cfg.hidden), torch.bfloat16, device)
    inner = StagedTrainer(stage, opt, n_micro, p2p=p2p, pp_rank=mesh.pp_idx, pp_size=pp,
                          embedding_group=mesh.embedding_group)
    return _Trainer(inner, mesh, stage)
