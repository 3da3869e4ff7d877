"""DLRM training engine against an fp32 autograd statement of the same network (CPU here, CUDA kernels on a GPU)."""
import pytest
import torch

from oneflow_b200.models import dlrm as M
from oneflow_b200.ops.interaction import dot_feature_interaction_reference


def _round(x):
    """bf16 rounding of an activation as the engine stores it, transparent to autograd."""
    return x + (x.bfloat16().float() - x).detach()


def _reference_grads(tr, dense, labels, emb):
    cfg = tr.cfg
    params = {n: p.detach().float().clone().requires_grad_() for n, p in tr.store.p.items()}
    emb32 = emb.detach().float().clone().requires_grad_()
    x = dense.float()
    x = x.bfloat16().float()
    for i in range(len(tr.bottom_dims) - 1):
        x = _round(torch.relu(x @ params[f"bottom.{i}.w"].t() + params[f"bottom.{i}.b"]))
    pad = cfg.interaction_dim - (cfg.embedding_dim + (cfg.num_tables + 1) * cfg.num_tables // 2)
    z = _round(dot_feature_interaction_reference([x, emb32], x, False, pad))
    nt = len(tr.top_dims) - 1
    for i in range(nt):
        z = z @ params[f"top.{i}.w"].t() + params[f"top.{i}.b"]
        if i < nt - 1:
            z = torch.relu(z)
        z = _round(z)
    loss = torch.nn.functional.binary_cross_entropy_with_logits(z[:, 0], labels.float())
    loss.backward()
    return loss.detach(), {n: p.grad for n, p in params.items()}, emb32.grad


def _check(device):
    torch.manual_seed(0)
    cfg = M.tiny_config()
    tr = M.DLRMTrainer(cfg, device, seed=1)
    tr.keep_trace = True
    dense, ids, labels = (t.to(device) for t in M.make_batch(cfg, cfg.global_batch, seed=5))
    before = tr.store.flat.clone()
    loss = tr.train_step(dense, ids, labels)
    # gradients of the step that just ran, against autograd on the weights the step started from
    tr.store.flat.copy_(before)
    ref_loss, ref_g, ref_demb = _reference_grads(tr, dense, labels, tr.trace["emb"])
    assert abs(float(loss) - float(ref_loss)) < 2e-2 * max(1.0, float(ref_loss))
    for name, g in ref_g.items():
        got = tr.store.g[name].float()
        assert (got - g).norm().item() <= 0.015 * g.norm().item() + 1e-7, (name, (got - g).norm().item(), g.norm().item())
    d = tr.trace["d_sparse"].float()
    assert (d - ref_demb).norm().item() <= 0.02 * ref_demb.norm().item(), ((d - ref_demb).norm().item(), ref_demb.norm().item())
    # a few more steps on the same batch: the loss must go down (embedding SGD + MLP Adam both act)
    first = float(loss)
    for _ in range(12):
        loss = tr.train_step(dense, ids, labels)
    assert float(loss) < first - 1e-3, (first, float(loss))
    prob = tr.forward(dense, ids)
    assert prob.shape == (cfg.global_batch,) and float(prob.min()) >= 0 and float(prob.max()) <= 1


def test_dlrm_trainer_cpu():
    _check("cpu")


@pytest.mark.gpu
def test_dlrm_trainer_gpu():
    from oneflow_b200.ops import _native
    _check("cuda")
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)


def test_dlrm_module_trains_with_public_api():
    import oneflow_b200 as flow
    from oneflow_b200 import one_embedding as oe
    cfg = M.tiny_config()
    torch.manual_seed(0)
    model = M.DLRMModule(cfg)
    opt = torch.optim.Adam([p for n, p in model.named_parameters() if "shadow" not in n], lr=3e-3)
    sparse_opt = oe.Optimizer(model.embedding, torch.optim.SGD, lr=0.05)
    dense, ids, labels = M.make_batch(cfg, 128, seed=2)
    losses = []
    for _ in range(8):
        logit = model(dense, ids)
        loss = torch.nn.functional.binary_cross_entropy_with_logits(logit, labels)
        opt.zero_grad()
        loss.backward()
        opt.step()
        sparse_opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0]


def test_make_batch_statistics():
    cfg = M.DLRMConfig()
    dense, ids, labels = M.make_batch(cfg, 4096, seed=0)
    assert dense.shape == (4096, 16) and ids.shape == (4096, 26) and labels.shape == (4096,)
    assert torch.all(dense[:, 13:] == 0) and abs(float(dense[:, :13].mean()) - 0.596) < 0.03   # E[log(1 + Exp(1))]
    for t in range(4):
        assert int(ids[:, t].max()) < cfg.rows_of(t) and int(ids[:, t].min()) >= 0
    # heavy head: a large share of the lookups of the biggest table falls on few rows
    assert ids[:, 0].unique().numel() < 3500
    assert abs(float(labels.mean()) - 0.25) < 0.03
