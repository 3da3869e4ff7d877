"""The hand-written BERT forward/backward against a PyTorch autograd statement of the same network."""
import pytest
import torch
import torch.nn.functional as F

from oneflow_b200.models.bert import BertConfig, BertStage, make_batch
from oneflow_b200.parallel.engine import FlatAdamW, StagedTrainer


def torch_bert_loss(params, cfg, batch):
    P = {k: v.detach().float().requires_grad_(True) for k, v in params.items()}
    S, NP = cfg.seq_len, cfg.max_predictions
    ids, types = batch[:, :S], batch[:, S:2 * S]
    mpos, mlab = batch[:, 2 * S:2 * S + NP], batch[:, 2 * S + NP:2 * S + 2 * NP]
    nsp, lens = batch[:, 2 * S + 2 * NP], batch[:, 2 * S + 2 * NP + 1]
    B = ids.shape[0]
    H, D, h = cfg.heads, cfg.head_dim, cfg.hidden
    x = P["wte"][ids] + P["wpe"][torch.arange(S)][None] + P["wtt"][types]
    x = F.layer_norm(x.reshape(B * S, h), (h,), P["emb_ln.g"], P["emb_ln.b"], cfg.eps)
    key_mask = (torch.arange(S)[None, :] < lens[:, None])[:, None, None, :]
    for li in range(cfg.layers):
        p = f"l.{li}."
        qkv = (x @ P[p + "wqkv"].t() + P[p + "bqkv"]).view(B, S, 3, H, D)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=key_mask).permute(0, 2, 1, 3).reshape(B * S, h)
        x = F.layer_norm(x + a @ P[p + "wo"].t() + P[p + "bo"], (h,), P[p + "ln1.g"], P[p + "ln1.b"], cfg.eps)
        f = F.gelu(x @ P[p + "w1"].t() + P[p + "b1"])
        x = F.layer_norm(x + f @ P[p + "w2"].t() + P[p + "b2"], (h,), P[p + "ln2.g"], P[p + "ln2.b"], cfg.eps)
    rows = (torch.arange(B)[:, None] * S + mpos).reshape(-1)
    t = F.gelu(x[rows] @ P["mlm.w"].t() + P["mlm.b"])
    t = F.layer_norm(t, (h,), P["mlm.ln.g"], P["mlm.ln.b"], cfg.eps)
    mlm = F.cross_entropy(t @ P["wte"].t() + P["mlm.bias"], mlab.reshape(-1))
    pooled = torch.tanh(x[torch.arange(B) * S] @ P["pool.w"].t() + P["pool.b"])
    nsp_loss = F.cross_entropy((pooled @ P["nsp.w"].t() + P["nsp.b"])[:, :2], nsp)
    loss = mlm + nsp_loss
    loss.backward()
    return loss.detach(), {k: v.grad for k, v in P.items()}


def _check(device, cfg, pad):
    torch.manual_seed(0)
    st = BertStage(cfg, device=device, seed=2)
    for n, p in st.store.named_parameters():
        if p.dim() == 1:
            p.copy_(torch.randn(p.shape) * 0.05 + (1.0 if n.endswith(".g") else 0.0))
    batch = make_batch(cfg, 3, generator=torch.Generator().manual_seed(1), pad_fraction=pad)
    st.store.start_accumulation()
    loss = st.forward(0, batch.to(device), batch.to(device))
    st.backward(0)
    ref_loss, ref_g = torch_bert_loss({k: v.cpu() for k, v in st.store.p.items()}, cfg, batch)
    assert abs(loss.item() - ref_loss.item()) < 0.05 * max(1.0, abs(ref_loss.item())), (loss.item(), ref_loss.item())
    bad = []
    for name, g in st.store.g.items():
        r = ref_g[name]
        if r is None:
            continue
        err = (g.float().cpu() - r).abs().max().item() / (r.abs().max().item() + 1e-6)
        if err > 0.1:
            bad.append((name, err))
    assert not bad, bad


def test_bert_stage_matches_autograd_cpu():
    _check("cpu", BertConfig(vocab_size=256, hidden=64, layers=2, heads=2, ffn=128, seq_len=32, max_predictions=4, eps=1e-5), 0.0)


def test_bert_stage_with_padding_cpu():
    _check("cpu", BertConfig(vocab_size=256, hidden=64, layers=1, heads=2, ffn=128, seq_len=32, max_predictions=4, eps=1e-5), 0.4)


def test_bert_trains_cpu():
    cfg = BertConfig(vocab_size=256, hidden=64, layers=2, heads=2, ffn=128, seq_len=32, max_predictions=4, eps=1e-5)
    st = BertStage(cfg, device="cpu", seed=4)
    tr = StagedTrainer(st, FlatAdamW(st.store, lr=5e-3, weight_decay=0.01), n_micro=2)
    batch = make_batch(cfg, 4, generator=torch.Generator().manual_seed(3))
    losses = [tr.train_step(batch).item() for _ in range(12)]
    assert losses[-1] < losses[0] - 0.3, losses


@pytest.mark.gpu
def test_bert_stage_matches_autograd_gpu():
    from oneflow_b200.ops import _native
    _check("cuda", BertConfig(vocab_size=256, hidden=128, layers=2, heads=2, ffn=256, seq_len=128, max_predictions=8, eps=1e-5), 0.3)
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)
