"""Step time of the native graph runtime on a small GPT, as a training step and as a forward pass, beside stock PyTorch.

    python -m oneflow_b200.utils.bench_graph_runtime [--layers 4 --hidden 1024 --heads 8 --seq 1024 --batch 4 --vocab 8192]

Prints one JSON line per measurement. The native numbers go through the public binding (``TrainingGraph.step`` /
``InferenceGraph.run``): every call copies its inputs from host memory and reads its result back, as a serving or training
loop written against the C ABI would. The PyTorch numbers are eager bf16 autocast with the fused AdamW, inputs already on
the device (the most favourable setting for it). Synthetic token ids, random weights."""
from __future__ import annotations

import argparse
import json
import tempfile
import time

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from oneflow_b200.utils import export as E


class Layer(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.ln1, self.qkv, self.proj = nn.LayerNorm(d), nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.ln2, self.fc1, self.fc2 = nn.LayerNorm(d), nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.heads = heads

    def forward(self, x):
        B, S, _ = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.heads, -1).unbind(2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, S, -1))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class GPT(nn.Module):
    def __init__(self, layers, d, heads, vocab, seq):
        super().__init__()
        self.emb, self.pos = nn.Embedding(vocab, d), nn.Embedding(seq, d)
        self.layers = nn.ModuleList([Layer(d, heads) for _ in range(layers)])
        self.ln = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.head.weight = self.emb.weight

    def hidden(self, ids):
        x = self.emb(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))
        for layer in self.layers:
            x = layer(x)
        return self.ln(x)

    def logits(self, ids):
        return self.head(self.hidden(ids))

    def forward(self, ids, targets):
        logits = self.logits(ids)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]), targets.view(-1))


class NextToken(nn.Module):
    """What a serving step returns: the logits of the last position only."""

    def __init__(self, gpt):
        super().__init__()
        self.gpt = gpt

    def forward(self, ids):
        return self.gpt.head(self.gpt.hidden(ids)[:, -1])


def _time(fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t = time.perf_counter()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t) / steps * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--vocab", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--only", default="all", choices=["all", "train", "forward", "torch"], help="run one group of measurements")
    a = ap.parse_args()
    torch.manual_seed(0)
    model = GPT(a.layers, a.hidden, a.heads, a.vocab, a.seq)
    for p in model.parameters():
        p.data = p.data.bfloat16().float()
    ids = torch.randint(0, a.vocab, (a.batch, a.seq))
    tgt = torch.randint(0, a.vocab, (a.batch, a.seq))
    cfg = {"layers": a.layers, "hidden": a.hidden, "heads": a.heads, "seq": a.seq, "batch": a.batch, "vocab": a.vocab}
    tokens = a.batch * a.seq

    d_train = E.export_graph(model, (ids, tgt), tempfile.mkdtemp(), fuse=False)
    d_infer = E.export_graph(NextToken(model), (ids,), tempfile.mkdtemp())
    for opt in ("adamw", "sgd") if a.only in ("all", "train") else ():
        g = E.TrainingGraph(d_train, device=0, optimizer=opt, lr=1e-4)
        first = g.step(ids.numpy(), tgt.numpy())
        ms = _time(lambda: g.step(ids.numpy(), tgt.numpy()), a.warmup, a.steps)
        print(json.dumps({"what": f"native training step ({opt})", "ms": ms, "tokens_per_s": tokens / ms * 1e3, "first_loss": first,
                          "plan": g.stats(), "config": cfg}), flush=True)
        g.close()
    if a.only in ("all", "forward"):
        g = E.InferenceGraph(d_infer, device=0)
        ms = _time(lambda: g.run(ids.numpy()), a.warmup, a.steps)
        print(json.dumps({"what": "native forward (prefill, next-token logits to host)", "ms": ms, "tokens_per_s": tokens / ms * 1e3, "plan": g.stats()}), flush=True)
        g.close()
    if a.only not in ("all", "torch"):
        return

    dev = torch.device("cuda:0")
    tm = model.to(dev)
    opt = torch.optim.AdamW(tm.parameters(), lr=1e-4, fused=True)
    ids_d, tgt_d = ids.to(dev), tgt.to(dev)

    def torch_step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = tm(ids_d, tgt_d)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return float(loss.detach())

    ms = _time(torch_step, a.warmup, a.steps)
    print(json.dumps({"what": "torch eager training step (bf16 autocast, fused AdamW)", "ms": ms, "tokens_per_s": tokens / ms * 1e3}), flush=True)

    def torch_fwd():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            return tm.head(tm.hidden(ids_d)[:, -1]).float().cpu()

    ms = _time(torch_fwd, a.warmup, a.steps)
    print(json.dumps({"what": "torch eager forward (prefill, next-token logits to host)", "ms": ms, "tokens_per_s": tokens / ms * 1e3}), flush=True)


if __name__ == "__main__":
    main()
