"""Device OneEmbedding engine on one GPU: lookup / initialisation, segment-summed gradients, row optimizers,
snapshots, and the MultiTableEmbedding module routed through it."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

INITS = [{"type": "uniform", "low": -0.1, "high": 0.1}, {"type": "normal", "mean": 0.0, "std": 0.05},
         {"type": "constant", "value": 0.25}]


def _engine(line_factor=1, **kw):
    from oneflow_b200.one_embedding.native import NativeEmbeddingEngine
    return NativeEmbeddingEngine("cuda", 1 << 15, 128, 128 * line_factor, INITS, 1 << 16, seed=3, **kw)


def _rows_of(eng, ids):
    T = ids.shape[-1]
    keys = ids.reshape(-1) * eng.num_tables + torch.arange(T, device=ids.device).repeat(ids.shape[0]) % eng.num_tables
    rows = eng.find(keys).long()
    assert (rows >= 0).all()
    return keys, rows


def test_lookup_initialisation_and_dedup():
    from oneflow_b200.ops import _native
    eng = _engine()
    torch.manual_seed(0)
    ids = torch.randint(0, 2000, (4096, 3), device="cuda")
    out = eng.forward(ids)
    assert out.shape == (4096, 3, 128) and out.dtype == torch.bfloat16
    keys, rows = _rows_of(eng, ids)
    assert eng.size == torch.unique(keys).numel()
    torch.testing.assert_close(out.view(-1, 128).float(), eng.rows[rows].bfloat16().float(), atol=0, rtol=0)
    u, n, c = out[:, 0].float(), out[:, 1].float(), out[:, 2].float()
    assert u.abs().max() <= 0.1 + 1e-3 and abs(u.mean()) < 2e-3 and abs(u.std() - 0.2 / math.sqrt(12)) < 3e-3
    assert abs(n.mean()) < 2e-3 and abs(n.std() - 0.05) < 3e-3
    assert torch.all(c == 0.25)
    again = eng.forward(ids)            # second lookup: no new rows, identical values
    assert torch.equal(out, again) and eng.size == torch.unique(keys).numel()
    miss = eng.forward(ids + 100000, insert=False)
    assert torch.all(miss == 0) and eng.size == torch.unique(keys).numel()
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)


@pytest.mark.parametrize("kind,factor", [("sgd", 1), ("momentum", 2), ("adam", 3), ("adagrad", 2), ("ftrl", 3), ("smart_decay_adam", 4)])
def test_row_optimizers_match_reference_update(kind, factor):
    from oneflow_b200.one_embedding.embedding import _row_update
    hyper = {"sgd": {"lr": 0.3}, "momentum": {"lr": 0.3, "momentum": 0.9},
             "adam": {"lr": 0.01, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "weight_decay": 0.01},
             "smart_decay_adam": {"lr": 0.01, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8},
             "adagrad": {"lr": 0.1, "lr_decay": 0.01, "eps": 1e-10},
             "ftrl": {"lr": 0.1, "lr_power": -0.5, "lambda1": 0.001, "lambda2": 0.01, "beta": 0.1}}[kind]
    eng = _engine(factor, state_init=0.1 if kind in ("adagrad", "ftrl") else 0.0)
    torch.manual_seed(1)
    for step in ((1, 2, 5) if kind == "smart_decay_adam" else (1, 2)):     # the jump to step 5 leaves rows untouched for a while
        ids = torch.randint(0, 500, (2048, 3), device="cuda")
        out = eng.forward(ids)
        keys, rows = _rows_of(eng, ids)
        grad = (torch.randn(2048, 3, 128, device="cuda") * 0.1).bfloat16()
        uk, inverse = torch.unique(keys, return_inverse=True)
        seg = torch.zeros(uk.numel(), 128, device="cuda").index_add_(0, inverse, grad.view(-1, 128).float())
        seg = seg.bfloat16().float()                      # 16-bit on the wire between requester and owner
        urows = eng.find(uk).long()
        before = eng.rows[urows].clone()
        _row_update(kind, before, seg, 128, hyper, step)
        eng.backward(grad, kind, hyper, step)
        torch.testing.assert_close(eng.rows[urows], before, atol=2e-5, rtol=2e-4)


def test_snapshot_roundtrip_and_module_path(tmp_path):
    import oneflow_b200 as flow
    from oneflow_b200 import one_embedding as oe
    tables = [oe.make_table_options(oe.make_uniform_initializer(-0.05, 0.05)) for _ in range(4)]
    opts = oe.make_device_mem_store_options(str(tmp_path), capacity=1 << 16)
    emb = oe.MultiTableEmbedding("sparse", 64, torch.bfloat16, torch.int64, tables, opts).cuda()
    opt = oe.Optimizer(emb, torch.optim.SGD, lr=1.0)
    ids = torch.randint(0, 1000, (512, 4), device="cuda")
    out = emb(ids)
    assert emb.engine is not None, "CUDA batches must run on the device engine"
    assert out.shape == (512, 4, 64)
    first = out.detach().clone()
    out.float().sum().backward()
    opt.step()
    second = emb(ids).detach()
    keys = ids * 4 + torch.arange(4, device="cuda")
    _, inverse, counts = torch.unique(keys.reshape(-1), return_inverse=True, return_counts=True)
    expect = first.float() - counts[inverse].view(512, 4, 1).float()
    torch.testing.assert_close(second.float(), expect, atol=0.05, rtol=0.02)
    sd = emb.state_dict()
    emb2 = oe.MultiTableEmbedding("sparse", 64, torch.bfloat16, torch.int64, tables, opts).cuda()
    emb2(ids[:1])                                         # brings the engine up
    emb2.load_state_dict(sd)
    torch.testing.assert_close(emb2(ids).float(), second.float(), atol=1e-6, rtol=0)
