"""Stand-in baseline: the benchmark's GPT in stock PyTorch, none of this package's kernels or engines.

Used by ``bench.py --impl torch_proxy`` because the reference framework cannot be built offline. It is what a user
of PyTorch would write for the same job: fp32 parameters under ``torch.autocast(bfloat16)`` (cuBLAS GEMMs),
``flash_attn`` for the causal attention, ``torch.nn.functional`` LayerNorm / GELU / cross entropy, Megatron-style tensor
parallelism (column- and row-parallel linears with an all-reduce in forward or backward, vocabulary-parallel embedding
and cross entropy) and 1F1B pipeline parallelism over ``torch.distributed`` (NCCL), gradient accumulation over the
micro-batches, gradient-norm clipping and ``torch.optim.AdamW(fused=True)``. Rank layout as in the other arms:
``rank = (dp_idx * pp + pp_idx) * tp + tp_idx``.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F


class _Copy(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _Reduce(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _Layer(torch.nn.Module):
    def __init__(self, cfg, tp, group, device):
        super().__init__()
        h, f = cfg.hidden, cfg.ffn
        self.cfg, self.tp, self.group = cfg, tp, group
        std, std_out = cfg.init_std, cfg.init_std / math.sqrt(2.0 * cfg.layers)
        mk = lambda *s, sd=std: torch.nn.Parameter(torch.randn(*s, device=device) * sd)  # noqa: E731
        zeros = lambda *s: torch.nn.Parameter(torch.zeros(*s, device=device))  # noqa: E731
        self.ln1, self.ln2 = torch.nn.LayerNorm(h, eps=cfg.eps, device=device), torch.nn.LayerNorm(h, eps=cfg.eps, device=device)
        self.wqkv, self.bqkv = mk(3 * h // tp, h), zeros(3 * h // tp)
        self.wo, self.bo = mk(h, h // tp, sd=std_out), zeros(h)
        self.w1, self.b1 = mk(f // tp, h), zeros(f // tp)
        self.w2, self.b2 = mk(h, f // tp, sd=std_out), zeros(h)

    def forward(self, x, batch, seq):
        from flash_attn import flash_attn_qkvpacked_func
        cfg, tp = self.cfg, self.tp
        hl = cfg.heads // tp
        h = self.ln1(x)
        if tp > 1:
            h = _Copy.apply(h, self.group)
        qkv = F.linear(h, self.wqkv, self.bqkv).view(batch, seq, 3, hl, cfg.head_dim)
        a = flash_attn_qkvpacked_func(qkv, causal=cfg.causal).reshape(batch * seq, hl * cfg.head_dim)
        o = F.linear(a, self.wo)
        if tp > 1:
            o = _Reduce.apply(o, self.group)
        x = x + o + self.bo
        h = self.ln2(x)
        if tp > 1:
            h = _Copy.apply(h, self.group)
        m = F.gelu(F.linear(h, self.w1, self.b1), approximate="tanh" if cfg.act == "gelu_tanh" else "none")
        o = F.linear(m, self.w2)
        if tp > 1:
            o = _Reduce.apply(o, self.group)
        return x + o + self.b2


def _vocab_parallel_xent(logits, labels, vocab_start, group):
    """Mean cross entropy over vocabulary-split logits [T, V/tp] (fp32), Megatron's formulation."""
    logits = logits.float()
    mx = logits.max(-1).values
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    logits = logits - mx[:, None]
    local = labels - vocab_start
    inside = (local >= 0) & (local < logits.shape[1])
    tgt = torch.where(inside, logits.gather(1, local.clamp(0, logits.shape[1] - 1)[:, None])[:, 0], torch.zeros_like(mx))
    tgt = _Reduce.apply(tgt, group)
    se = _Reduce.apply(torch.exp(logits).sum(-1), group)
    return (torch.log(se) - tgt).mean()


class _Stage(torch.nn.Module):
    def __init__(self, cfg, l0, l1, first, last, tp, tp_rank, group, device):
        super().__init__()
        self.cfg, self.first, self.last, self.tp, self.tp_rank, self.group = cfg, first, last, tp, tp_rank, group
        vl = cfg.vocab_size // tp
        self.vocab_start = tp_rank * vl
        if first:
            self.wte = torch.nn.Parameter(torch.randn(vl, cfg.hidden, device=device) * cfg.init_std)
            self.wpe = torch.nn.Parameter(torch.randn(cfg.seq_len, cfg.hidden, device=device) * cfg.init_std)
        self.layers = torch.nn.ModuleList([_Layer(cfg, tp, group, device) for _ in range(l0, l1)])
        if last:
            self.lnf = torch.nn.LayerNorm(cfg.hidden, eps=cfg.eps, device=device)
            self.head = torch.nn.Parameter(torch.randn(vl, cfg.hidden, device=device) * cfg.init_std)

    def forward(self, inp, labels, batch, seq):
        cfg = self.cfg
        if self.first:
            ids = inp.reshape(-1)
            local = ids - self.vocab_start
            inside = (local >= 0) & (local < self.wte.shape[0])
            x = F.embedding(local.clamp(0, self.wte.shape[0] - 1), self.wte) * inside[:, None].to(self.wte.dtype)
            if self.tp > 1:
                x = _Reduce.apply(x, self.group)
            x = x + self.wpe[torch.arange(batch * seq, device=ids.device) % seq]
        else:
            x = inp
        for layer in self.layers:
            x = layer(x, batch, seq)
        if not self.last:
            return x
        h = self.lnf(x)
        if self.tp > 1:
            h = _Copy.apply(h, self.group)
        logits = F.linear(h, self.head)
        if self.tp > 1:
            return _vocab_parallel_xent(logits, labels.reshape(-1), self.vocab_start, self.group)
        return F.cross_entropy(logits.float(), labels.reshape(-1))


class GPTProxy:
    """``train_step(tokens)``: one optimizer step over ``n_micro`` micro-batches of this rank's share of the batch
    (tokens: int64 [n_micro * micro_batch, seq + 1] on the device). Returns the mean loss (on ranks where ``has_loss``)."""

    def __init__(self, cfg, tp=1, pp=1, dp=1, micro_batch=4, n_micro=16, device="cuda", lr=1e-4, weight_decay=0.1, clip_grad=1.0):
        self.cfg, self.tp, self.pp, self.dp, self.n_micro, self.micro = cfg, tp, pp, dp, n_micro, micro_batch
        self.device = torch.device(device)
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        assert tp * pp * dp == world
        self.tp_idx, self.pp_idx, self.dp_idx = rank % tp, (rank // tp) % pp, rank // (tp * pp)
        self.tp_group = self.dp_group = None
        self.mp_group = None
        if world > 1:
            for d in range(dp):
                for p in range(pp):
                    ranks = [(d * pp + p) * tp + t for t in range(tp)]
                    g = dist.new_group(ranks) if tp > 1 else None
                    if rank in ranks:
                        self.tp_group = g
            for p in range(pp):
                for t in range(tp):
                    ranks = [(d * pp + p) * tp + t for d in range(dp)]
                    g = dist.new_group(ranks) if dp > 1 else None
                    if rank in ranks:
                        self.dp_group = g
            for d in range(dp):
                ranks = [(d * pp + p) * tp + t for p in range(pp) for t in range(tp)]
                g = dist.new_group(ranks) if pp * tp > 1 else None
                if rank in ranks:
                    self.mp_group = g
        per = cfg.layers // pp
        l0 = self.pp_idx * per
        l1 = cfg.layers if self.pp_idx == pp - 1 else l0 + per
        self.first, self.last = self.pp_idx == 0, self.pp_idx == pp - 1
        self.has_loss = self.last
        torch.manual_seed(1234 + rank)
        self.stage = _Stage(cfg, l0, l1, self.first, self.last, tp, self.tp_idx, self.tp_group, self.device)
        decay = [p for p in self.stage.parameters() if p.dim() >= 2]
        rest = [p for p in self.stage.parameters() if p.dim() < 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": weight_decay}, {"params": rest, "weight_decay": 0.0}],
                                     lr=lr, betas=(0.9, 0.95), eps=1e-8, fused=True)
        self.clip = clip_grad
        self.prev = rank - tp if self.pp_idx > 0 else None
        self.next = rank + tp if self.pp_idx < pp - 1 else None
        self.act_shape = (micro_batch * cfg.seq_len, cfg.hidden)

    # ---- pipeline p2p (batched so that neighbours never wait on each other)
    def _p2p(self, send_next=None, send_prev=None, recv_prev=False, recv_next=False):
        ops, rp, rn = [], None, None
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev, self.prev))
        if recv_prev:
            rp = torch.empty(self.act_shape, dtype=torch.bfloat16, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rp, self.prev))
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next, self.next))
        if recv_next:
            rn = torch.empty(self.act_shape, dtype=torch.bfloat16, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rn, self.next))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return rp, rn

    def _fwd(self, m, inputs, labels, recv):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            inp = inputs[m] if self.first else recv.requires_grad_(True)
            out = self.stage(inp, labels[m] if self.last else None, self.micro, self.cfg.seq_len)
        if self.last:
            out = out / self.n_micro
        elif out.dtype != torch.bfloat16:
            out = out.to(torch.bfloat16)
        return inp, out

    def train_step(self, tokens):
        n, mb = self.n_micro, self.micro
        inputs = [tokens[i * mb:(i + 1) * mb, :-1] for i in range(n)]
        labels = [tokens[i * mb:(i + 1) * mb, 1:] for i in range(n)]
        loss = torch.zeros((), device=self.device)
        if self.pp == 1:
            for m in range(n):
                _, out = self._fwd(m, inputs, labels, None)
                out.backward()
                loss += out.detach()
        else:
            warm = min(self.pp - self.pp_idx - 1, n)
            saved = []
            recv, _ = self._p2p(recv_prev=not self.first)
            fm = 0
            for _ in range(warm):
                inp, out = self._fwd(fm, inputs, labels, recv)
                fm += 1
                saved.append((inp, out))
                recv, _ = self._p2p(send_next=None if self.last else out.detach(), recv_prev=(not self.first) and fm < n)
            for i in range(n - warm):
                inp, out = self._fwd(fm, inputs, labels, recv)
                fm += 1
                saved.append((inp, out))
                if self.last:
                    loss += out.detach()
                    grad = None
                else:
                    _, grad = self._p2p(send_next=out.detach(), recv_next=True)
                inp0, out0 = saved.pop(0)
                out0.backward(grad)
                dprev = None if self.first else inp0.grad
                recv, _ = self._p2p(send_prev=dprev, recv_prev=(not self.first) and fm < n)
            for _ in range(warm):
                _, grad = self._p2p(recv_next=True)
                inp0, out0 = saved.pop(0)
                out0.backward(grad)
                self._p2p(send_prev=None if self.first else inp0.grad)
        params = [p for p in self.stage.parameters() if p.grad is not None]
        if self.dp > 1:
            for p in params:
                dist.all_reduce(p.grad, group=self.dp_group)
                p.grad.div_(self.dp)
        if self.clip:
            # replicated tensors (vectors and the position table under tensor parallelism) count once
            sq_rep = torch.zeros((), device=self.device)
            sq = torch.zeros((), device=self.device)
            for p in params:
                s = p.grad.float().pow(2).sum()
                if self.tp > 1 and (p.dim() < 2 or (self.first and p is self.stage.wpe)):
                    sq_rep += s
                else:
                    sq += s
            tot = sq + sq_rep / self.tp
            if self.mp_group is not None:
                dist.all_reduce(tot, group=self.mp_group)
            coef = torch.clamp(self.clip / (tot.sqrt() + 1e-6), max=1.0)
            torch._foreach_mul_([p.grad for p in params], coef)
        self.opt.step()
        self.opt.zero_grad(set_to_none=False)
        return loss
