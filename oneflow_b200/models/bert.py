"""BERT encoder for pre-training (post-LN, GELU, masked-LM + next-sentence heads) on the native kernels,
written like models/gpt.py as explicit forward / backward stages with minimal saved activations.

Batch layout (one int64 row per sequence, produced by ``make_batch``):
    [0, S)            input ids
    [S, 2S)           token type ids
    [2S, 2S+P)        positions of the P masked tokens (P = max predictions per sequence)
    [2S+P, 2S+2P)     their labels
    2S+2P             next-sentence label
    2S+2P+1           number of valid (non-padding) tokens
The MLM head only runs on the gathered masked positions. The vocabulary is padded to a multiple of 64
(30522 -> 30528) so that every GEMM dimension is TMA friendly; padded logits never win the softmax because
their weights are zero-initialised and never receive gradient from labels.

Parallelism: same tensor-parallel scheme as the GPT (heads / FFN columns / vocabulary sharded, activations
sequence-sharded between the tensor-parallel regions); data parallel through the trainer's ZeRO shard.

Reference model: the BERT that LiBai / OneFlow-Benchmark build from matmul, fused_bias_add_gelu,
fused_scale_mask_softmax(_dropout) and layer_norm ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import embedding as E
from ..ops import gemm as G
from ..ops import kernels as K
from .gpt import ParamStore


@dataclass
class BertConfig:
    vocab_size: int = 30528          # 30522 padded to a multiple of 64
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    ffn: int = 4096
    seq_len: int = 512
    type_vocab: int = 2
    max_predictions: int = 76        # ~15 % of 512
    eps: float = 1e-12
    init_std: float = 0.02
    causal: bool = False

    @property
    def head_dim(self):
        return self.hidden // self.heads

    def flops_per_token(self, with_attention=True):
        h, f, s = self.hidden, self.ffn, self.seq_len
        mm = self.layers * (2 * 3 * h * h + 2 * h * h + 2 * 2 * h * f)
        head = (2 * h * h + 2 * h * self.vocab_size) * self.max_predictions / s
        attn = self.layers * (2 * 2 * s * h) if with_attention else 0
        return 3 * (mm + head + attn)


BERT_LARGE = BertConfig()
BERT_TINY = BertConfig(vocab_size=512, hidden=128, layers=2, heads=2, ffn=512, seq_len=64, max_predictions=8)


def make_batch(cfg: BertConfig, batch, generator=None, device="cpu", pad_fraction=0.0):
    """Synthetic pre-training batch: uniform tokens, P masked positions per sequence, Bernoulli(0.5) NSP labels."""
    S, P = cfg.seq_len, cfg.max_predictions
    g = generator
    ids = torch.randint(0, min(cfg.vocab_size, 30522), (batch, S), generator=g)
    types = (torch.arange(S)[None, :] >= S // 2).long().expand(batch, S)
    pos = torch.stack([torch.randperm(S, generator=g)[:P].sort().values for _ in range(batch)])
    lab = torch.gather(ids, 1, pos)
    ids = ids.scatter(1, pos, 103)                      # [MASK]
    nsp = torch.randint(0, 2, (batch, 1), generator=g)
    lens = torch.full((batch, 1), S, dtype=torch.long)
    if pad_fraction > 0:
        lens = torch.randint(int(S * (1 - pad_fraction)), S + 1, (batch, 1), generator=g)
    return torch.cat([ids, types, pos, lab, nsp, lens], 1).to(device)


class BertStage:
    """All layers [l0, l1) plus embeddings (first stage) and the pre-training heads (last stage)."""

    def __init__(self, cfg: BertConfig, layer_begin=0, layer_end=None, first=True, last=True, device="cuda", tp=None, seed=0,
                 grad_dtype=torch.float32):
        self.cfg = cfg
        self.l0, self.l1 = layer_begin, cfg.layers if layer_end is None else layer_end
        self.first, self.last, self.tp = first, last, tp
        self.tp_size = tp.size if tp is not None else 1
        self.tp_rank = tp.rank if tp is not None else 0
        self.device = torch.device(device)
        n = self.tp_size
        h, f = cfg.hidden, cfg.ffn
        rep = 1 if n > 1 else 0
        self.vocab_local = cfg.vocab_size // n
        specs = []
        if first or last:
            specs.append(("wte", (self.vocab_local, h), True, cfg.init_std))
        if first:
            specs += [("wpe", (cfg.seq_len, h), True, cfg.init_std, 2 if n > 1 else 0),
                      ("wtt", (cfg.type_vocab, h), True, cfg.init_std, 2 if n > 1 else 0),
                      ("emb_ln.g", (h,), False, ("const", 1.0), rep), ("emb_ln.b", (h,), False, ("const", 0.0), rep)]
        for li in range(self.l0, self.l1):
            p = f"l.{li}."
            specs += [
                (p + "wqkv", (3 * h // n, h), True, cfg.init_std), (p + "bqkv", (3 * h // n,), False, ("const", 0.0)),
                (p + "wo", (h, h // n), True, cfg.init_std), (p + "bo", (h,), False, ("const", 0.0), rep),
                (p + "ln1.g", (h,), False, ("const", 1.0), rep), (p + "ln1.b", (h,), False, ("const", 0.0), rep),
                (p + "w1", (f // n, h), True, cfg.init_std), (p + "b1", (f // n,), False, ("const", 0.0)),
                (p + "w2", (h, f // n), True, cfg.init_std), (p + "b2", (h,), False, ("const", 0.0), rep),
                (p + "ln2.g", (h,), False, ("const", 1.0), rep), (p + "ln2.b", (h,), False, ("const", 0.0), rep)]
        if last:
            # heads run on gathered rows that every tensor-parallel rank holds in full: replicated, complete grads
            r2 = 2 if n > 1 else 0
            specs += [("mlm.w", (h, h), True, cfg.init_std, r2), ("mlm.b", (h,), False, ("const", 0.0), r2),
                      ("mlm.ln.g", (h,), False, ("const", 1.0), r2), ("mlm.ln.b", (h,), False, ("const", 0.0), r2),
                      ("mlm.bias", (self.vocab_local,), False, ("const", 0.0)),
                      ("pool.w", (h, h), True, cfg.init_std, r2), ("pool.b", (h,), False, ("const", 0.0), r2),
                      ("nsp.w", (8, h), True, cfg.init_std, r2), ("nsp.b", (8,), False, ("const", 0.0), r2)]
        self.store = ParamStore(specs, self.device, grad_dtype=grad_dtype)
        self.store.init_(seed, shard_offset=7919 * self.tp_rank)
        self.saved = {}

    # ------------------------------------------------------------------ helpers shared with the GPT stage
    def _p(self, n):
        return self.store.p[n]

    def _wgrad(self, name, dy, x):
        G.gemm(dy, x, a_layout="km", b_layout="kn", out=self.store.g[name], accumulate=self.store.acc_flag(name))

    def _bgrad(self, name, dy):
        g = self.store.g[name]
        if not self.store.acc_flag(name):
            g.zero_()
        K.column_sum(dy, out=g)

    def _lngrad(self, gname, bname, dg, db):
        for n, v in ((gname, dg), (bname, db)):
            g = self.store.g[n]
            if self.store.acc_flag(n):
                g.add_(v)
            else:
                g.copy_(v)

    def split_batch(self, tokens, n):
        mb = tokens.shape[0] // n
        parts = [tokens[i * mb:(i + 1) * mb] for i in range(n)]
        return parts, parts

    sync_replicated_grads = None  # bound below (same implementation as the GPT stage)

    # ------------------------------------------------------------------ one encoder layer (post-LN)
    def _layer_fwd(self, li, x, B, S, kv_len, sv):
        cfg, p, tp = self.cfg, f"l.{li}.", self.tp
        Hl, D = cfg.heads // self.tp_size, cfg.head_dim
        if tp is None:
            qkv = G.gemm(x, self._p(p + "wqkv"), bias=self._p(p + "bqkv"))
        else:
            # gathered inputs are kept for the weight gradients (a copy is cheaper than a second gather)
            x_g, qkv = tp.ag_gemm(x, self._p(p + "wqkv"), bias=self._p(p + "bqkv"), return_gathered=True)
            x_full = x_g.clone() if x_g.is_cuda else x_g
        q5 = qkv.view(B, S, 3, Hl, D)
        attn, lse = K.fmha_fwd(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], causal=False, kv_len=kv_len)
        a2 = attn.view(B * S, Hl * D)
        if tp is None:
            y1 = G.gemm(a2, self._p(p + "wo"), bias=self._p(p + "bo"), residual=x)
        else:
            y1 = tp.gemm_rs(a2, self._p(p + "wo"), bias=self._p(p + "bo"), residual=x)
        x1, m1, r1 = K.layer_norm_fwd(y1, self._p(p + "ln1.g"), self._p(p + "ln1.b"), cfg.eps)
        if tp is None:
            a, h1 = G.gemm(x1, self._p(p + "w1"), bias=self._p(p + "b1"), act=G.ACT_GELU, want_aux=True)
            y2 = G.gemm(a, self._p(p + "w2"), bias=self._p(p + "b2"), residual=x1)
        else:
            x1_g, a, h1 = tp.ag_gemm(x1, self._p(p + "w1"), bias=self._p(p + "b1"), act=G.ACT_GELU, want_aux=True, return_gathered=True)
            x1_full = x1_g.clone() if x1_g.is_cuda else x1_g
            y2 = tp.gemm_rs(a, self._p(p + "w2"), bias=self._p(p + "b2"), residual=x1)
        out, m2, r2 = K.layer_norm_fwd(y2, self._p(p + "ln2.g"), self._p(p + "ln2.b"), cfg.eps)
        sv[li] = (x, qkv, attn, lse, y1, m1, r1, h1, y2, m2, r2) + ((x_full, x1_full) if tp is not None else (None, None))
        return out

    def _layer_bwd(self, li, dout, B, S, kv_len, sv):
        cfg, p, tp = self.cfg, f"l.{li}.", self.tp
        Hl, D = cfg.heads // self.tp_size, cfg.head_dim
        x, qkv, attn, lse, y1, m1, r1, h1, y2, m2, r2, x_full, x1_full = sv.pop(li)
        dy2, dg, db = K.layer_norm_bwd(dout, y2, self._p(p + "ln2.g"), m2, r2)
        self._lngrad(p + "ln2.g", p + "ln2.b", dg, db)
        a = K.bias_act_fwd(h1, None, G.ACT_GELU)
        self._bgrad(p + "b2", dy2)
        if tp is None:
            self._wgrad(p + "w2", dy2, a)
            dh1 = G.gemm(dy2, self._p(p + "w2"), b_layout="kn", aux_in=h1, act=G.ACT_GELU)
        else:
            dy2_full, dh1 = tp.ag_gemm(dy2, self._p(p + "w2"), b_layout="kn", aux_in=h1, act=G.ACT_GELU, return_gathered=True)
            self._wgrad(p + "w2", dy2_full, a)
        del a, h1
        self._bgrad(p + "b1", dh1)
        if tp is None:
            x1, _, _ = K.layer_norm_fwd(y1, self._p(p + "ln1.g"), self._p(p + "ln1.b"), cfg.eps)
            self._wgrad(p + "w1", dh1, x1)
            dx1 = G.gemm(dh1, self._p(p + "w1"), b_layout="kn", residual=dy2)
            del x1
        else:
            self._wgrad(p + "w1", dh1, x1_full)
            dx1 = tp.gemm_rs(dh1, self._p(p + "w1"), b_layout="kn", residual=dy2)
            del x1_full
        del dh1
        dy1, dg, db = K.layer_norm_bwd(dx1, y1, self._p(p + "ln1.g"), m1, r1)
        self._lngrad(p + "ln1.g", p + "ln1.b", dg, db)
        a2 = attn.view(B * S, Hl * D)
        self._bgrad(p + "bo", dy1)
        if tp is None:
            self._wgrad(p + "wo", dy1, a2)
            dattn = G.gemm(dy1, self._p(p + "wo"), b_layout="kn")
        else:
            dy1_full, dattn = tp.ag_gemm(dy1, self._p(p + "wo"), b_layout="kn", return_gathered=True)
            self._wgrad(p + "wo", dy1_full, a2)
        q5 = qkv.view(B, S, 3, Hl, D)
        dqkv5 = torch.empty((B, S, 3, Hl, D), dtype=qkv.dtype, device=qkv.device)
        K.fmha_bwd(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], attn, dattn.view(B, S, Hl, D), lse, causal=False, kv_len=kv_len,
                   dqkv=dqkv5)
        dqkv = dqkv5.view(B * S, 3 * Hl * D)
        self._bgrad(p + "bqkv", dqkv)
        if tp is None:
            self._wgrad(p + "wqkv", dqkv, x)
            dx = G.gemm(dqkv, self._p(p + "wqkv"), b_layout="kn", residual=dy1)
        else:
            self._wgrad(p + "wqkv", dqkv, x_full)
            dx = tp.gemm_rs(dqkv, self._p(p + "wqkv"), b_layout="kn", residual=dy1)
        return dx

    # ------------------------------------------------------------------ stage API (same contract as GPTStage)
    def _fields(self, batch):
        S, P = self.cfg.seq_len, self.cfg.max_predictions
        return (batch[:, :S].contiguous(), batch[:, S:2 * S].contiguous(), batch[:, 2 * S:2 * S + P].contiguous(),
                batch[:, 2 * S + P:2 * S + 2 * P].contiguous(), batch[:, 2 * S + 2 * P].contiguous(),
                batch[:, 2 * S + 2 * P + 1].contiguous())

    def forward(self, mb, inp, labels=None, loss_scale=1.0, bs=None):
        cfg, tp = self.cfg, self.tp
        batch = inp if self.first else labels
        ids, types, mpos, mlab, nsp, lens = self._fields(batch) if batch is not None else (None,) * 6
        B, S = (ids.shape if ids is not None else (bs[0], cfg.seq_len))
        kv_len = lens.to(torch.int32) if lens is not None and bool((lens < S).any()) else None
        sv = {"bs": (B, S), "kv_len": kv_len}
        if self.first:
            e = E.embedding_fwd(ids, self._p("wte"), self._p("wpe"), seq=S, vocab_start=self.tp_rank * self.vocab_local)
            if tp is not None:
                # word embeddings are partial sums over the vocabulary shards; add positions / types once
                e = tp.all_reduce(e) - (self.tp_size - 1) * self._p("wpe")[torch.arange(B * S, device=e.device) % S]
            e = e + self._p("wtt")[types.reshape(-1)]
            if tp is not None:
                Tl = B * S // self.tp_size
                e = e[self.tp_rank * Tl:(self.tp_rank + 1) * Tl].contiguous()
            x, me, re_ = K.layer_norm_fwd(e, self._p("emb_ln.g"), self._p("emb_ln.b"), cfg.eps)
            sv["emb"] = (ids, types, e, me, re_)
        else:
            x = inp
        for li in range(self.l0, self.l1):
            x = self._layer_fwd(li, x, B, S, kv_len, sv)
        out = x
        if self.last:
            full = tp.all_gather_rows(x) if tp is not None else x
            rows = (torch.arange(B, device=full.device)[:, None] * S + mpos).reshape(-1)
            hm = full[rows].contiguous()                                        # [B*P, h]
            t, t_pre = G.gemm(hm, self._p("mlm.w"), bias=self._p("mlm.b"), act=G.ACT_GELU, want_aux=True)
            tn, mt, rt = K.layer_norm_fwd(t, self._p("mlm.ln.g"), self._p("mlm.ln.b"), cfg.eps)
            logits = G.gemm(tn, self._p("wte"), bias=self._p("mlm.bias"))
            lab = mlab.reshape(-1)
            n_pred = lab.numel()
            stats = K.xent_stats(logits, lab, vocab_start=self.tp_rank * self.vocab_local)
            if tp is not None:
                stats = tp.merge_xent_stats(stats)
            mlm_rows, dlogits = K.xent_grad(logits, lab, stats, grad_scale=loss_scale / n_pred,
                                            vocab_start=self.tp_rank * self.vocab_local, inplace=True)
            cls = full[torch.arange(B, device=full.device) * S].contiguous()    # [B, h]
            pooled_pre = G.gemm(cls, self._p("pool.w"), bias=self._p("pool.b"))
            pooled = torch.tanh(pooled_pre.float()).to(pooled_pre.dtype)
            nsp_logits = G.gemm(pooled, self._p("nsp.w"), bias=self._p("nsp.b"))[:, :2].float()
            nsp_logp = torch.log_softmax(nsp_logits, -1)
            nsp_loss = -nsp_logp.gather(1, nsp[:, None]).mean()
            dnsp = (torch.exp(nsp_logp) - torch.nn.functional.one_hot(nsp, 2).float()) * (loss_scale / B)
            sv["head"] = (x, full.shape, rows, hm, t_pre, t, mt, rt, tn, dlogits, cls, pooled, dnsp)
            out = (mlm_rows.sum() / n_pred + nsp_loss) * loss_scale
        self.saved[mb] = sv
        return out

    def backward(self, mb, dout=None):
        cfg, tp = self.cfg, self.tp
        sv = self.saved.pop(mb)
        B, S = sv["bs"]
        kv_len = sv["kv_len"]
        if self.last:
            x, full_shape, rows, hm, t_pre, t, mt, rt, tn, dlogits, cls, pooled, dnsp = sv.pop("head")
            # MLM head
            self._wgrad("wte", dlogits, tn)
            self._bgrad("mlm.bias", dlogits)
            if tp is None:
                dtn = G.gemm(dlogits, self._p("wte"), b_layout="kn")
            else:
                dtn = tp.all_reduce(G.gemm(dlogits, self._p("wte"), b_layout="kn"))
            dt, dg, db = K.layer_norm_bwd(dtn, t, self._p("mlm.ln.g"), mt, rt)
            self._lngrad("mlm.ln.g", "mlm.ln.b", dg, db)
            dpre = K.bias_act_bwd(t_pre, None, dt, G.ACT_GELU)
            self._wgrad("mlm.w", dpre, hm)
            self._bgrad("mlm.b", dpre)
            dhm = G.gemm(dpre, self._p("mlm.w"), b_layout="kn")
            # NSP head
            dn = torch.zeros((B, 8), dtype=torch.bfloat16, device=dnsp.device)
            dn[:, :2] = dnsp.to(torch.bfloat16)
            self._wgrad("nsp.w", dn, pooled)
            self._bgrad("nsp.b", dn)
            dpooled = G.gemm(dn, self._p("nsp.w"), b_layout="kn")
            dpp = (dpooled.float() * (1 - pooled.float() ** 2)).to(torch.bfloat16)
            self._wgrad("pool.w", dpp, cls)
            self._bgrad("pool.b", dpp)
            dcls = G.gemm(dpp, self._p("pool.w"), b_layout="kn")
            dfull = torch.zeros(full_shape, dtype=torch.bfloat16, device=dhm.device)
            dfull.index_add_(0, rows, dhm)
            dfull.index_add_(0, torch.arange(B, device=dfull.device) * S, dcls)
            if tp is not None:
                Tl = B * S // self.tp_size
                dy = dfull[self.tp_rank * Tl:(self.tp_rank + 1) * Tl].contiguous()
            else:
                dy = dfull
        else:
            dy = dout
        for li in range(self.l1 - 1, self.l0 - 1, -1):
            dy = self._layer_bwd(li, dy, B, S, kv_len, sv)
        if self.first:
            ids, types, e, me, re_ = sv.pop("emb")
            de, dg, db = K.layer_norm_bwd(dy, e, self._p("emb_ln.g"), me, re_)
            self._lngrad("emb_ln.g", "emb_ln.b", dg, db)
            if tp is not None:
                de = tp.all_gather_rows(de)
            for nme in ("wte", "wpe", "wtt"):
                if not self.store.acc_flag(nme):
                    self.store.g[nme].zero_()
            E.embedding_bwd(ids, de, self.store.g["wte"], self.store.g["wpe"], seq=S, vocab_start=self.tp_rank * self.vocab_local)
            self.store.g["wtt"].index_add_(0, types.reshape(-1), de.float())
            return None
        return dy


from .gpt import GPTStage as _GPTStage  # noqa: E402

BertStage.sync_replicated_grads = _GPTStage.sync_replicated_grads
