"""The hand-written GPT forward/backward against a PyTorch autograd statement of the same network."""
import math

import pytest
import torch
import torch.nn.functional as F

from oneflow_b200.models.gpt import GPTConfig, GPTStage
from oneflow_b200.parallel.engine import FlatAdamW, StagedTrainer

CFG = GPTConfig(vocab_size=256, hidden=64, layers=2, heads=2, ffn=256, seq_len=32, act="gelu_tanh")


def torch_gpt_loss(params, cfg, inp, lab):
    """fp32 autograd reference built from the stage's own parameter tensors."""
    P = {k: v.detach().float().requires_grad_(True) for k, v in params.items()}
    B, S = inp.shape
    x = P["wte"][inp] + P["wpe"][torch.arange(S)][None]
    x = x.reshape(B * S, cfg.hidden)
    H, D = cfg.heads, cfg.head_dim
    for li in range(cfg.layers):
        p = f"h.{li}."
        ln1 = F.layer_norm(x, (cfg.hidden,), P[p + "ln1.g"], P[p + "ln1.b"], cfg.eps)
        qkv = (ln1 @ P[p + "attn.wqkv"].t() + P[p + "attn.bqkv"]).view(B, S, 3, H, D)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).permute(0, 2, 1, 3).reshape(B * S, H * D)
        x = x + a @ P[p + "attn.wo"].t() + P[p + "attn.bo"]
        ln2 = F.layer_norm(x, (cfg.hidden,), P[p + "ln2.g"], P[p + "ln2.b"], cfg.eps)
        h1 = F.gelu(ln2 @ P[p + "mlp.w1"].t() + P[p + "mlp.b1"], approximate="tanh")
        x = x + h1 @ P[p + "mlp.w2"].t() + P[p + "mlp.b2"]
    x = F.layer_norm(x, (cfg.hidden,), P["lnf.g"], P["lnf.b"], cfg.eps)
    logits = x @ P["wte"].t()
    loss = F.cross_entropy(logits, lab.reshape(-1))
    loss.backward()
    return loss.detach(), {k: v.grad for k, v in P.items()}


def _check_stage(device, CFG=CFG):
    torch.manual_seed(0)
    st = GPTStage(CFG, device=device, seed=3)
    # make LayerNorm / bias parameters non-trivial
    for n, p in st.store.named_parameters():
        if n.endswith(".b") or n.endswith("bqkv") or n.endswith("bo") or n.endswith("b1") or n.endswith("b2"):
            p.copy_(torch.randn(p.shape) * 0.05)
        if n.endswith(".g"):
            p.copy_(1 + torch.randn(p.shape) * 0.05)
    B, S = 2, CFG.seq_len
    tok = torch.randint(0, CFG.vocab_size, (B, S + 1), device=device)
    inp, lab = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    st.store.start_accumulation()
    loss = st.forward(0, inp, lab)
    st.backward(0)
    ref_loss, ref_g = torch_gpt_loss({k: v.cpu() for k, v in st.store.p.items()}, CFG, inp.cpu(), lab.cpu())
    assert abs(loss.item() - ref_loss.item()) < 0.05 * max(1.0, abs(ref_loss.item()))
    bad = []
    for name, g in st.store.g.items():
        r = ref_g[name]
        denom = r.abs().max().item() + 1e-6
        err = (g.float().cpu() - r).abs().max().item() / denom
        if err > 0.08:
            bad.append((name, err))
    assert not bad, bad
    return st, tok


def test_gpt_stage_matches_autograd_cpu():
    _check_stage("cpu")


def test_gpt_grad_accumulation_and_adamw_cpu():
    torch.manual_seed(1)
    st = GPTStage(CFG, device="cpu", seed=5)
    opt = FlatAdamW(st.store, lr=1e-2, weight_decay=0.1, clip_grad=1.0)
    tr = StagedTrainer(st, opt, n_micro=2)
    tok = torch.randint(0, CFG.vocab_size, (4, CFG.seq_len + 1))
    losses = [tr.train_step(tok).item() for _ in range(8)]
    assert losses[-1] < losses[0] - 0.3, losses
    # two micro-batches of 2 == one micro-batch of 4 (same gradients)
    st2 = GPTStage(CFG, device="cpu", seed=5)
    st3 = GPTStage(CFG, device="cpu", seed=5)
    for s, n in ((st2, 2), (st3, 1)):
        s.store.start_accumulation()
        mb = 4 // n
        for m in range(n):
            t = tok[m * mb:(m + 1) * mb]
            s.forward(m, t[:, :-1].contiguous(), t[:, 1:].contiguous(), loss_scale=1.0 / n)
            s.backward(m)
    d = (st2.store.grad - st3.store.grad).abs().max().item()
    assert d < 2e-2 * st3.store.grad.abs().max().item() + 1e-4


@pytest.mark.gpu
def test_gpt_stage_matches_autograd_gpu():
    from oneflow_b200.ops import _native
    cfg = GPTConfig(vocab_size=256, hidden=128, layers=2, heads=2, ffn=512, seq_len=128, act="gelu_tanh")
    _check_stage("cuda", cfg)
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)


@pytest.mark.gpu
def test_gpt_training_step_gpu_loss_decreases():
    torch.manual_seed(2)
    cfg = GPTConfig(vocab_size=1024, hidden=256, layers=2, heads=2, ffn=1024, seq_len=256)
    st = GPTStage(cfg, device="cuda", seed=1)
    opt = FlatAdamW(st.store, lr=3e-3, weight_decay=0.01)
    tr = StagedTrainer(st, opt, n_micro=2)
    tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), device="cuda")
    losses = [tr.train_step(tok).item() for _ in range(10)]
    assert losses[-1] < losses[0] - 0.5, losses
