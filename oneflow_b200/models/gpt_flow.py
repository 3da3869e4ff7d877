"""GPT written against the flow API only: ``flow.nn`` modules, global tensors with SBP annotations, ``nn.Graph``
with ``set_stage`` pipeline stages, ``flow.optim.AdamW``. This is the model the headline benchmark trains.

Parallelism is declared, not coded: every parameter is a global tensor on a 2-D placement ``[dp, tp]`` of its pipeline
stage (tensor-parallel ranks innermost),

    token / position embedding   wte [V, H]  (B, S(0))  vocabulary parallel      wpe [S, H]  (B, B)
    QKV projection               w [3, H, H] (B, S(1))  heads split              b [3, H]    (B, S(1))
    attention output projection  w [H, H]    (B, S(1))  row parallel             b [H]       (B, B)
    MLP up / down                w1 [F, H]   (B, S(0)), b1 (B, S(0));            w2 [H, F]   (B, S(1)), b2 (B, B)
    LayerNorms                   (B, B)
    LM head                      w [V, H]    (B, S(0))  vocabulary parallel logits, vocabulary-parallel cross entropy

and the activations between the blocks are ``[tokens, H]`` with the tokens split over both mesh axes
``(S(0), S(0))`` (data parallel x sequence parallel). The ops pick their SBP signatures from these annotations
(framework/fused_ops.py): the column-parallel products run as one all-gather->GEMM kernel, the row-parallel ones as
one GEMM->reduce-scatter kernel, LayerNorm / attention / embedding / loss on the local shards.

The same layer stack in the reference's terms: LiBai's GPT on SBP signatures (matmul ``S(0),B->S(0)`` /
``B,S(1)->S(1)`` / ``S(1),S(0)->P``, oneflow/user/ops/matmul_op.cpp:123-175; stages through
python/oneflow/nn/graph/graph_block.py:119-151).
"""
from __future__ import annotations

import math
import zlib

import torch

import oneflow_b200 as flow
from oneflow_b200 import nn
from ..framework import boxing, fused_ops as F, global_tensor as GT
from .gpt import GPTConfig

S, B = flow.sbp.split, flow.sbp.broadcast


class Layout:
    """Placements of a (dp, pp, tp) decomposition: ``rank = (dp_idx * pp + pp_idx) * tp + tp_idx``; the placement of
    pipeline stage s is the 2-D mesh [dp, tp] of the ranks with that pp index."""

    def __init__(self, tp=1, pp=1, dp=1, device_type="cuda"):
        self.tp, self.pp, self.dp, self.device_type = tp, pp, dp, device_type
        self.stages = [flow.placement(device_type, [[(d * pp + s) * tp + t for t in range(tp)] for d in range(dp)])
                       for s in range(pp)]

    def stage_of_layer(self, i, layers):
        per = layers // self.pp
        return min(i // per, self.pp - 1)


def make_param(name, shape, nd, pl, std, seed=0, dtype=torch.bfloat16, const=None):
    """A global parameter whose logical values depend only on (name, seed): the full tensor is drawn from its own
    generator and this rank keeps its shard, so every parallel layout starts from the same model."""
    me = GT._rank()
    coords = pl.coords(me)
    dev = pl.device()
    if coords is None:
        local = torch.empty((0,), dtype=dtype, device=dev)
        return torch.nn.Parameter(GT.wrap(local, shape, pl, tuple(nd)), requires_grad=True)
    if const is not None:
        full = torch.full(shape, float(const), dtype=dtype, device=dev)
    else:
        gen = torch.Generator(device=dev)
        gen.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
        full = torch.empty(shape, dtype=dtype, device=dev)
        flat = full.view(-1)
        step = 1 << 26
        for s0 in range(0, flat.numel(), step):
            c = min(step, flat.numel() - s0)
            flat[s0:s0 + c].copy_(torch.randn(c, generator=gen, device=dev).mul_(std))
    local = boxing.from_all_broadcast(full, pl, tuple(nd), coords)
    local = local.clone() if local.data_ptr() == full.data_ptr() and local.numel() != full.numel() else local
    return torch.nn.Parameter(GT.wrap(local.contiguous(), shape, pl, tuple(nd)), requires_grad=True)


class GPTEmbedding(nn.Module):
    def __init__(self, cfg: GPTConfig, pl, seed=0, dtype=torch.bfloat16):
        super().__init__()
        self.cfg, self.pl = cfg, pl
        self.wte = make_param("wte", (cfg.vocab_size, cfg.hidden), (B, S(0)), pl, cfg.init_std, seed, dtype)
        self.wpe = make_param("wpe", (cfg.seq_len, cfg.hidden), (B, B), pl, cfg.init_std, seed, dtype)
        self._pos = {}

    def _positions(self, batch, seq):
        """Global int64 [batch * seq] tensor of positions, rows split like the activations."""
        key = (batch, seq)
        p = self._pos.get(key)
        if p is None:
            pl = self.pl
            nd = (S(0), S(0))
            coords = pl.coords(GT._rank())
            if coords is None:
                p = GT._placeholder(torch.empty((batch * seq,), dtype=torch.int64, device="meta"), pl, nd)
            else:
                from ..framework.nd_sbp import slice_view
                lo, hi = slice_view((batch * seq,), pl.hierarchy, nd, coords)[0]
                p = GT.wrap(torch.arange(lo, hi, device=pl.device()) % seq, (batch * seq,), pl, nd)
            self._pos[key] = p
        return p

    def forward(self, tokens):
        batch, seq = tokens.shape
        ids = tokens.reshape(-1)
        tok = F.embedding(ids, self.wte)                       # (S(0), P): every rank looked up its vocabulary shard
        x = tok.to_global(sbp=(S(0), S(0)))                    # reduce-scatter into sequence shards
        pos = F.embedding(self._positions(batch, seq), self.wpe)
        return x + pos


class TransformerLayer(nn.Module):
    def __init__(self, cfg: GPTConfig, idx, pl, seed=0, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        h, f = cfg.hidden, cfg.ffn
        std_out = cfg.init_std / math.sqrt(2.0 * cfg.layers)
        p = f"h.{idx}."
        mk = lambda n, shape, nd, std=None, const=None: make_param(p + n, shape, nd, pl, std or cfg.init_std, seed, dtype, const)  # noqa: E731
        self.ln1_w, self.ln1_b = mk("ln1.g", (h,), (B, B), const=1.0), mk("ln1.b", (h,), (B, B), const=0.0)
        self.wqkv, self.bqkv = mk("attn.wqkv", (3, h, h), (B, S(1))), mk("attn.bqkv", (3, h), (B, S(1)), const=0.0)
        self.wo, self.bo = mk("attn.wo", (h, h), (B, S(1)), std_out), mk("attn.bo", (h,), (B, B), const=0.0)
        self.ln2_w, self.ln2_b = mk("ln2.g", (h,), (B, B), const=1.0), mk("ln2.b", (h,), (B, B), const=0.0)
        self.w1, self.b1 = mk("mlp.w1", (f, h), (B, S(0))), mk("mlp.b1", (f,), (B, S(0)), const=0.0)
        self.w2, self.b2 = mk("mlp.w2", (h, f), (B, S(1)), std_out), mk("mlp.b2", (h,), (B, B), const=0.0)

    def forward(self, x):
        cfg = self.cfg
        # (LayerNorm output, the input again for the residual branch: both gradients meet inside the LayerNorm backward kernel)
        h, x = F.layer_norm_residual(x, (cfg.hidden,), self.ln1_w, self.ln1_b, cfg.eps)
        qkv = F.linear(h, self.wqkv, self.bqkv)                                   # all-gather -> GEMM, heads split
        a = F.fused_attention_qkv_packed(qkv, seq_len=cfg.seq_len, head_size=cfg.head_dim, causal=cfg.causal)
        x = F.linear(a, self.wo, self.bo, residual=x)                             # GEMM -> reduce-scatter (+bias +residual)
        h, x = F.layer_norm_residual(x, (cfg.hidden,), self.ln2_w, self.ln2_b, cfg.eps)
        # all-gather -> GEMM -> bias + GELU, then GEMM -> reduce-scatter (+bias +residual); as one unit, so that backward folds
        # the GELU gradient into the data-gradient GEMM of the second layer
        return F.mlp(h, self.w1, self.b1, self.w2, self.b2, act=cfg.act, residual=x)


class GPTHead(nn.Module):
    def __init__(self, cfg: GPTConfig, pl, seed=0, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.lnf_w = make_param("lnf.g", (cfg.hidden,), (B, B), pl, 0, seed, dtype, const=1.0)
        self.lnf_b = make_param("lnf.b", (cfg.hidden,), (B, B), pl, 0, seed, dtype, const=0.0)
        self.lm_head = make_param("lm_head", (cfg.vocab_size, cfg.hidden), (B, S(0)), pl, cfg.init_std, seed, dtype)

    def forward(self, x, labels):
        cfg = self.cfg
        h = F.layer_norm(x, (cfg.hidden,), self.lnf_w, self.lnf_b, cfg.eps)
        logits = F.linear(h, self.lm_head)                                         # [tokens, V], vocabulary split
        rows = F.sparse_softmax_cross_entropy(logits, labels.reshape(-1))
        return rows.mean()


class GPTModel(nn.Module):
    def __init__(self, cfg: GPTConfig, layout: Layout, seed=0, dtype=torch.bfloat16):
        super().__init__()
        self.cfg, self.layout = cfg, layout
        self.embedding = GPTEmbedding(cfg, layout.stages[0], seed, dtype)
        self.layers = nn.ModuleList([TransformerLayer(cfg, i, layout.stages[layout.stage_of_layer(i, cfg.layers)], seed, dtype)
                                     for i in range(cfg.layers)])
        self.head = GPTHead(cfg, layout.stages[-1], seed, dtype)

    def forward(self, tokens, labels):
        x = self.embedding(tokens)
        for layer in self.layers:
            x = layer(x)
        return self.head(x, labels)


class GPTTrainGraph(nn.Graph):
    """One call = one optimizer step over ``grad_acc`` micro-batches; stages declared with ``set_stage``."""

    def __init__(self, model: GPTModel, optimizer, grad_acc=1, zero_stage=1, lr_sch=None):
        super().__init__()
        self.model = model
        lay = model.layout
        GM = nn.graph.GraphModule
        self.model.embedding.to(GM).set_stage(0, lay.stages[0])
        for i in range(model.cfg.layers):
            s = lay.stage_of_layer(i, model.cfg.layers)
            self.model.layers[i].to(GM).set_stage(s, lay.stages[s])
        self.model.head.to(GM).set_stage(lay.pp - 1, lay.stages[-1])
        self.config.set_gradient_accumulation_steps(grad_acc)
        if zero_stage:
            self.config.enable_zero(True, stage=zero_stage)
        self.add_optimizer(optimizer, lr_sch=lr_sch)

    def build(self, tokens, labels):
        loss = self.model(tokens, labels)
        loss.backward()
        return loss


def param_groups(model, weight_decay):
    """Matrices are decayed, vectors (biases, LayerNorm parameters) are not."""
    decay = [p for p in model.parameters() if p.dim() >= 2]
    rest = [p for p in model.parameters() if p.dim() < 2]
    return [{"params": decay, "weight_decay": weight_decay}, {"params": rest, "weight_decay": 0.0}]


def build_gpt_graph(cfg: GPTConfig, tp=1, pp=1, dp=1, grad_acc=1, device_type="cuda", lr=1e-4, weight_decay=0.1,
                    clip_grad=1.0, zero_stage=1, seed=0, dtype=torch.bfloat16):
    """(graph, model, layout) ready for ``graph(tokens, labels)``."""
    layout = Layout(tp, pp, dp, device_type)
    model = GPTModel(cfg, layout, seed, dtype)
    groups = param_groups(model, weight_decay)
    if clip_grad:
        for g in groups:
            g["clip_grad_max_norm"], g["clip_grad_norm_type"] = clip_grad, 2.0
    opt = flow.optim.AdamW(groups, lr=lr, betas=(0.9, 0.95), eps=1e-8)
    graph = GPTTrainGraph(model, opt, grad_acc=grad_acc, zero_stage=zero_stage if dp > 1 else 0)
    return graph, model, layout


def make_inputs(layout: Layout, tokens_local):
    """``tokens_local``: int64 [local_batch, seq + 1] on this rank's device (the same batch on the ranks of one
    data-parallel slice). Returns (inputs on the first stage, labels on the last stage) as global tensors; the ranks
    of the other stages pass placeholders."""
    inp = tokens_local[:, :-1]
    lab = tokens_local[:, 1:]
    x = GT.to_global(inp, layout.stages[0], (S(0), B), check_meta=False, sync_data=False)
    y = GT.to_global(lab, layout.stages[-1], (S(0), B), check_meta=False, sync_data=False)
    return x, y
