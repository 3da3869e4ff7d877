"""GPT decoder (pre-LN, causal fused attention, tied embedding / LM head) on the native kernels.

The model is written as explicit forward / backward stages instead of going through
autograd: every micro-batch saves the minimum set of activations (10 x hidden bf16 values
per token per layer: layer input, packed QKV, attention output, post-attention residual and
the pre-GELU FFN activation) and recomputes the cheap memory-bound pieces (LayerNorm
outputs, GELU) in the backward. All matrix products run on the tcgen05 GEMM with their
bias / GELU / residual / GELU-gradient epilogues fused; weight gradients accumulate in
fp32 straight into a flat gradient buffer from the GEMM epilogue.

Parallelism (see oneflow_b200/parallel): tensor parallel with sequence-parallel LayerNorm
regions (all-gather -> GEMM and GEMM -> reduce-scatter fused kernels), pipeline stages
(a ``GPTStage`` owns a contiguous range of layers), data parallel with ZeRO-1.

Reference model definition this mirrors: the Megatron-style GPT that LiBai builds on the
reference's SBP signatures (matmul ``S(0),B->S(0)`` / ``B,S(1)->S(1)`` / ``S(1),S(0)->P``,
oneflow/user/ops/matmul_op.cpp:123-175) with fused_bias_add_gelu, layer_norm and
fused attention ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import embedding as E
from ..ops import gemm as G
from ..ops import kernels as K


@dataclass
class GPTConfig:
    vocab_size: int = 50304
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    ffn: int = 16384
    seq_len: int = 2048
    eps: float = 1e-5
    act: str = "gelu_tanh"      # "gelu" (erf) or "gelu_tanh"
    init_std: float = 0.02
    causal: bool = True

    @property
    def head_dim(self):
        return self.hidden // self.heads

    def num_params(self):
        h, f = self.hidden, self.ffn
        per_layer = 4 * h + 3 * h * h + 3 * h + h * h + h + f * h + f + h * f + h
        return self.layers * per_layer + self.vocab_size * h + self.seq_len * h + 2 * h

    def flops_per_token(self, with_attention=True):
        """Training FLOPs per token (forward + backward = 3x forward matmul FLOPs)."""
        h, f, s = self.hidden, self.ffn, self.seq_len
        mm = self.layers * (2 * 3 * h * h + 2 * h * h + 2 * 2 * h * f) + 2 * h * self.vocab_size
        attn = self.layers * (2 * 2 * s * h) * (0.5 if self.causal else 1.0) if with_attention else 0
        return 3 * (mm + attn)


GPT_6_7B = GPTConfig()
GPT_TINY = GPTConfig(vocab_size=512, hidden=128, layers=2, heads=2, ffn=512, seq_len=128)

_ACT = {"gelu": G.ACT_GELU, "gelu_tanh": G.ACT_GELU_TANH, "relu": G.ACT_RELU}


def _align(n, a=64):
    return (n + a - 1) // a * a


class ParamStore:
    """Flat parameter storage: one bf16 buffer for the model weights and one fp32 buffer for the
    accumulated gradients, with named views. Weight-decayed tensors come first so that the
    optimizer can treat the buffer as two contiguous segments."""

    def __init__(self, specs, device, dtype=torch.bfloat16, grad_dtype=torch.float32):
        # specs: list of (name, shape, decay: bool, init_std or ("const", value)[, rep]) where rep tells how the
        # tensor relates to the tensor-parallel group: 0 = a shard unique to this rank, 1 = replicated and its
        # gradient is a partial sum over the ranks' token shards, 2 = replicated with a complete gradient.
        specs = [tuple(s) + (0,) * (5 - len(s)) for s in specs]
        order = sorted(range(len(specs)), key=lambda i: (not specs[i][2], specs[i][4] != 0, i))
        self.specs5 = [specs[i] for i in order]
        self.specs = [s[:4] for s in self.specs5]
        off = 0
        self.offsets = {}
        self.decay_end = 0
        self.replicated_ranges = []   # [lo, hi) element ranges holding replicated tensors (count once in norms)
        self.partial_names = []       # replicated tensors whose gradients must be summed over the tp group
        for name, shape, dec, _, rep in self.specs5:
            n = math.prod(shape)
            self.offsets[name] = (off, n, tuple(shape))
            if rep:
                if self.replicated_ranges and self.replicated_ranges[-1][1] == off:
                    self.replicated_ranges[-1][1] = off + _align(n)
                else:
                    self.replicated_ranges.append([off, off + _align(n)])
                if rep == 1:
                    self.partial_names.append(name)
            off += _align(n)
            if dec:
                self.decay_end = off
        self.total = off
        self.flat = torch.zeros(self.total, dtype=dtype, device=device)
        self.grad = torch.zeros(self.total, dtype=grad_dtype, device=device)
        self.p: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}
        for name, (o, n, shape) in self.offsets.items():
            self.p[name] = self.flat[o:o + n].view(shape)
            self.g[name] = self.grad[o:o + n].view(shape)
        self.grad_ready = set()  # names whose gradient holds a value for the current accumulation window

    def init_(self, seed=0, shard_offset=0):
        """Every tensor draws from its own stream seeded by (seed, name), so the values do not depend on
        which other tensors share the store (any pipeline split initialises identically)."""
        import zlib
        dev = self.flat.device
        gen = torch.Generator(device=dev)
        for name, shape, _, init, rep in self.specs5:
            # shards differ between tensor-parallel ranks, replicated tensors must not
            s = seed + (0 if rep else shard_offset)
            gen.manual_seed((s * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
            if isinstance(init, tuple):
                self.p[name].fill_(init[1])
            else:
                # generated in chunks (on the tensor's own device) to bound the fp32 temporary
                t = self.p[name].view(-1)
                n = t.numel()
                step = 1 << 26
                for s0 in range(0, n, step):
                    c = min(step, n - s0)
                    t[s0:s0 + c].copy_(torch.randn(c, generator=gen, device=dev).mul_(init).to(t.dtype))

    def named_parameters(self):
        return [(n, self.p[n]) for n, _, _, _ in self.specs]

    def start_accumulation(self):
        self.grad_ready.clear()

    def acc_flag(self, name):
        """True when the gradient of `name` already holds a partial sum (so the producer must add)."""
        if name in self.grad_ready:
            return True
        self.grad_ready.add(name)
        return False


def layer_specs(cfg: GPTConfig, li: int, tp: int = 1):
    h, f = cfg.hidden, cfg.ffn
    std_out = cfg.init_std / math.sqrt(2.0 * cfg.layers)
    p = f"h.{li}."
    rep = 1 if tp > 1 else 0  # LayerNorm parameters and row-parallel biases see only this rank's token shard
    return [
        (p + "ln1.g", (h,), False, ("const", 1.0), rep), (p + "ln1.b", (h,), False, ("const", 0.0), rep),
        (p + "attn.wqkv", (3 * h // tp, h), True, cfg.init_std), (p + "attn.bqkv", (3 * h // tp,), False, ("const", 0.0)),
        (p + "attn.wo", (h, h // tp), True, std_out), (p + "attn.bo", (h,), False, ("const", 0.0), rep),
        (p + "ln2.g", (h,), False, ("const", 1.0), rep), (p + "ln2.b", (h,), False, ("const", 0.0), rep),
        (p + "mlp.w1", (f // tp, h), True, cfg.init_std), (p + "mlp.b1", (f // tp,), False, ("const", 0.0)),
        (p + "mlp.w2", (h, f // tp), True, std_out), (p + "mlp.b2", (h,), False, ("const", 0.0), rep),
    ]


class GPTStage:
    """Layers [layer_begin, layer_end) of a GPT, plus the embedding on the first stage and the final
    LayerNorm + tied LM head + loss on the last stage. ``tp`` is a tensor-parallel context
    (oneflow_b200.parallel.tensor_parallel.TPContext) or None."""

    def __init__(self, cfg: GPTConfig, layer_begin=0, layer_end=None, first=True, last=True, device="cuda", tp=None,
                 seed=0, grad_dtype=torch.float32):
        self.cfg = cfg
        self.l0, self.l1 = layer_begin, cfg.layers if layer_end is None else layer_end
        self.first, self.last = first, last
        self.tp = tp
        self.tp_size = tp.size if tp is not None else 1
        self.tp_rank = tp.rank if tp is not None else 0
        self.act = _ACT[cfg.act]
        self.device = torch.device(device)
        tpn = self.tp_size
        if cfg.heads % tpn or cfg.ffn % tpn or cfg.vocab_size % tpn:
            raise ValueError("heads, ffn and vocab must be divisible by the tensor-parallel size")
        specs = []
        self.vocab_local = cfg.vocab_size // tpn
        if first or last:
            specs.append(("wte", (self.vocab_local, cfg.hidden), True, cfg.init_std))
        if first:
            specs.append(("wpe", (cfg.seq_len, cfg.hidden), True, cfg.init_std, 2 if tpn > 1 else 0))
        for li in range(self.l0, self.l1):
            specs += layer_specs(cfg, li, tpn)
        if last:
            rep = 1 if tpn > 1 else 0
            specs += [("lnf.g", (cfg.hidden,), False, ("const", 1.0), rep), ("lnf.b", (cfg.hidden,), False, ("const", 0.0), rep)]
        self.store = ParamStore(specs, self.device, grad_dtype=grad_dtype)
        # Different tensor-parallel ranks hold different shards: decorrelate their random init.
        self.store.init_(seed, shard_offset=7919 * self.tp_rank)
        self.saved: Dict[int, dict] = {}

    # ------------------------------------------------------------------ helpers
    def _p(self, name):
        return self.store.p[name]

    def _wgrad(self, name, dy, x):
        """grad[name] (+)= dy^T @ x, accumulated in fp32 by the GEMM epilogue."""
        g = self.store.g[name]
        acc = self.store.acc_flag(name)
        G.gemm(dy, x, a_layout="km", b_layout="kn", out=g, accumulate=acc)

    def _bgrad(self, name, dy):
        g = self.store.g[name]
        if not self.store.acc_flag(name):
            g.zero_()
        K.column_sum(dy, out=g)

    def _lngrad(self, gname, bname, dgamma, dbeta):
        for n, v in ((gname, dgamma), (bname, dbeta)):
            g = self.store.g[n]
            if self.store.acc_flag(n):
                g.add_(v)
            else:
                g.copy_(v)

    # ------------------------------------------------------------------ one transformer layer
    def _layer_fwd(self, li, x, B, S, sv):
        cfg, p = self.cfg, f"h.{li}."
        tp = self.tp
        Hl, D = cfg.heads // self.tp_size, cfg.head_dim
        ln1, mean1, rstd1 = K.layer_norm_fwd(x, self._p(p + "ln1.g"), self._p(p + "ln1.b"), cfg.eps)
        if tp is None:
            qkv = G.gemm(ln1, self._p(p + "attn.wqkv"), bias=self._p(p + "attn.bqkv"))
        else:
            # the gathered LayerNorm output is kept for the weight gradient: copying it out of the exchange buffer is
            # several times cheaper than gathering it again in the backward pass
            ln1_g, qkv = tp.ag_gemm(ln1, self._p(p + "attn.wqkv"), bias=self._p(p + "attn.bqkv"), return_gathered=True)
            ln1_full = ln1_g.clone() if ln1_g.is_cuda else ln1_g
        del ln1
        q5 = qkv.view(B, S, 3, Hl, D)
        attn, lse = K.fmha_fwd(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], causal=cfg.causal)
        attn2 = attn.view(B * S, Hl * D)
        if tp is None:
            x1 = G.gemm(attn2, self._p(p + "attn.wo"), bias=self._p(p + "attn.bo"), residual=x)
        else:
            x1 = tp.gemm_rs(attn2, self._p(p + "attn.wo"), bias=self._p(p + "attn.bo"), residual=x)
        ln2, mean2, rstd2 = K.layer_norm_fwd(x1, self._p(p + "ln2.g"), self._p(p + "ln2.b"), cfg.eps)
        if tp is None:
            a, h1 = G.gemm(ln2, self._p(p + "mlp.w1"), bias=self._p(p + "mlp.b1"), act=self.act, want_aux=True)
            y = G.gemm(a, self._p(p + "mlp.w2"), bias=self._p(p + "mlp.b2"), residual=x1)
        else:
            ln2_g, a, h1 = tp.ag_gemm(ln2, self._p(p + "mlp.w1"), bias=self._p(p + "mlp.b1"), act=self.act, want_aux=True,
                                      return_gathered=True)
            ln2_full = ln2_g.clone() if ln2_g.is_cuda else ln2_g
            y = tp.gemm_rs(a, self._p(p + "mlp.w2"), bias=self._p(p + "mlp.b2"), residual=x1)
        sv[li] = (x, mean1, rstd1, qkv, attn, lse, x1, mean2, rstd2, h1) + ((ln1_full, ln2_full) if tp is not None else (None, None))
        return y

    def _layer_bwd(self, li, dy, B, S, sv):
        cfg, p = self.cfg, f"h.{li}."
        tp = self.tp
        Hl, D = cfg.heads // self.tp_size, cfg.head_dim
        x, mean1, rstd1, qkv, attn, lse, x1, mean2, rstd2, h1, ln1_full, ln2_full = sv.pop(li)
        # ---- MLP
        a = K.bias_act_fwd(h1, None, self.act)
        self._bgrad(p + "mlp.b2", dy)
        if tp is None:
            self._wgrad(p + "mlp.w2", dy, a)
            dh1 = G.gemm(dy, self._p(p + "mlp.w2"), b_layout="kn", aux_in=h1, act=self.act)
        else:
            # dy is a sequence shard: gather it once, use it for both the weight and the data gradient
            dy_full, dh1 = tp.ag_gemm(dy, self._p(p + "mlp.w2"), b_layout="kn", aux_in=h1, act=self.act, return_gathered=True)
            self._wgrad(p + "mlp.w2", dy_full, a)
            del dy_full
        del a, h1
        self._bgrad(p + "mlp.b1", dh1)
        if tp is None:
            ln2, _, _ = K.layer_norm_fwd(x1, self._p(p + "ln2.g"), self._p(p + "ln2.b"), cfg.eps)
            self._wgrad(p + "mlp.w1", dh1, ln2)
            dln2 = G.gemm(dh1, self._p(p + "mlp.w1"), b_layout="kn")
            del ln2
        else:
            self._wgrad(p + "mlp.w1", dh1, ln2_full)
            dln2 = tp.gemm_rs(dh1, self._p(p + "mlp.w1"), b_layout="kn")
            del ln2_full
        del dh1
        dx1, dg, db = K.layer_norm_bwd(dln2, x1, self._p(p + "ln2.g"), mean2, rstd2, add_to_dx=dy)
        self._lngrad(p + "ln2.g", p + "ln2.b", dg, db)
        del dln2, dy
        # ---- attention
        attn2 = attn.view(B * S, Hl * D)
        self._bgrad(p + "attn.bo", dx1)
        if tp is None:
            self._wgrad(p + "attn.wo", dx1, attn2)
            dattn = G.gemm(dx1, self._p(p + "attn.wo"), b_layout="kn")
        else:
            dx1_full, dattn = tp.ag_gemm(dx1, self._p(p + "attn.wo"), b_layout="kn", return_gathered=True)
            self._wgrad(p + "attn.wo", dx1_full, attn2)
            del dx1_full
        q5 = qkv.view(B, S, 3, Hl, D)
        dqkv5 = torch.empty((B, S, 3, Hl, D), dtype=qkv.dtype, device=qkv.device)
        K.fmha_bwd(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], attn, dattn.view(B, S, Hl, D), lse, causal=cfg.causal, dqkv=dqkv5)
        dqkv = dqkv5.view(B * S, 3 * Hl * D)
        del dattn, attn, qkv
        self._bgrad(p + "attn.bqkv", dqkv)
        if tp is None:
            ln1, _, _ = K.layer_norm_fwd(x, self._p(p + "ln1.g"), self._p(p + "ln1.b"), cfg.eps)
            self._wgrad(p + "attn.wqkv", dqkv, ln1)
            dln1 = G.gemm(dqkv, self._p(p + "attn.wqkv"), b_layout="kn")
            del ln1
        else:
            self._wgrad(p + "attn.wqkv", dqkv, ln1_full)
            dln1 = tp.gemm_rs(dqkv, self._p(p + "attn.wqkv"), b_layout="kn")
            del ln1_full
        del dqkv
        dx, dg, db = K.layer_norm_bwd(dln1, x, self._p(p + "ln1.g"), mean1, rstd1, add_to_dx=dx1)
        self._lngrad(p + "ln1.g", p + "ln1.b", dg, db)
        return dx

    # ------------------------------------------------------------------ stage API
    def forward(self, mb, inp, labels=None, loss_scale=1.0, bs=None):
        """First stage: ``inp`` = token ids [B, S]; other stages: activations [B*S(/tp), hidden].
        Last stage returns the (already scaled) mean loss as a 0-d fp32 tensor, others the activations."""
        cfg = self.cfg
        sv = {}
        if self.first:
            B, S = inp.shape
            x = E.embedding_fwd(inp, self._p("wte"), self._p("wpe"), seq=S, vocab_start=self.tp_rank * self.vocab_local)
            sv["ids"] = inp
            if self.tp is not None:
                x = self.tp.reduce_scatter_rows(x)  # vocabulary-parallel partial sums -> sequence shards
        else:
            x = inp
            B, S = labels.shape if labels is not None else bs
        sv["bs"] = (B, S)
        for li in range(self.l0, self.l1):
            x = self._layer_fwd(li, x, B, S, sv)
        out = x
        if self.last:
            lnf, meanf, rstdf = K.layer_norm_fwd(x, self._p("lnf.g"), self._p("lnf.b"), cfg.eps)
            if self.tp is not None:
                lnf_full = self.tp.all_gather_rows(lnf)
            else:
                lnf_full = lnf
            logits = G.gemm(lnf_full, self._p("wte"))
            lab = labels.reshape(-1)
            ntok = lab.numel()
            stats = K.xent_stats(logits, lab, vocab_start=self.tp_rank * self.vocab_local)
            if self.tp is not None:
                stats = self.tp.merge_xent_stats(stats)
            loss_rows, dlogits = K.xent_grad(logits, lab, stats, grad_scale=loss_scale / ntok,
                                             vocab_start=self.tp_rank * self.vocab_local, inplace=True)
            sv["head"] = (x, meanf, rstdf, dlogits, lnf_full)
            out = loss_rows.sum() * (loss_scale / ntok)
        self.saved[mb] = sv
        return out

    def backward(self, mb, dout=None):
        """``dout``: gradient of this stage's output activations (None on the last stage, where the loss
        gradient was formed in the forward). Returns the gradient for the previous stage (None on the first)."""
        cfg = self.cfg
        sv = self.saved.pop(mb)
        B, S = sv["bs"]
        if self.last:
            x, meanf, rstdf, dlogits, lnf_full = sv.pop("head")
            self._wgrad("wte", dlogits, lnf_full)
            if self.tp is None:
                dlnf = G.gemm(dlogits, self._p("wte"), b_layout="kn")
            else:
                dlnf = self.tp.gemm_rs(dlogits, self._p("wte"), b_layout="kn")
            del dlogits, lnf_full
            dy, dg, db = K.layer_norm_bwd(dlnf, x, self._p("lnf.g"), meanf, rstdf)
            self._lngrad("lnf.g", "lnf.b", dg, db)
        else:
            dy = dout
        for li in range(self.l1 - 1, self.l0 - 1, -1):
            dy = self._layer_bwd(li, dy, B, S, sv)
        if self.first:
            if self.tp is not None:
                dy = self.tp.all_gather_rows(dy)
            first_wte = not self.store.acc_flag("wte")
            first_wpe = not self.store.acc_flag("wpe")
            if first_wte:
                self.store.g["wte"].zero_()
            if first_wpe:
                self.store.g["wpe"].zero_()
            E.embedding_bwd(sv["ids"], dy, self.store.g["wte"], self.store.g["wpe"], seq=S,
                            vocab_start=self.tp_rank * self.vocab_local)
            return None
        return dy

    def sync_replicated_grads(self):
        """Sums over the tensor-parallel group the gradients of replicated parameters that were formed from
        this rank's token shard only (LayerNorm parameters, row-parallel biases)."""
        if self.tp is None or not self.store.partial_names:
            return
        views = [self.store.g[n].reshape(-1) for n in self.store.partial_names]
        flat = torch.cat(views)
        flat = self.tp.all_reduce(flat)
        o = 0
        for v in views:
            v.copy_(flat[o:o + v.numel()])
            o += v.numel()

    def num_local_params(self):
        return sum(math.prod(s[1]) for s in self.store.specs)
