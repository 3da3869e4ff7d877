"""Device OneEmbedding engine on one GPU: lookup / initialisation, segment-summed gradients, row optimizers,
snapshots, and the MultiTableEmbedding module routed through it."""
import math

import pytest
import torch

from oneflow_b200.ops import _native

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


def test_device_lru_cache_against_a_bookkeeping_model():
    """The set-associative LRU kernels (32 ways per set, set = mix64(key) % n_sets) against host bookkeeping: a key is a
    hit exactly while it is resident (put and not reported evicted since), hits and evicted rows carry the latest values,
    no set ever holds more than 32 keys, a row is only pushed out of a set that would overflow, and the victim was not
    used more recently than a key that stays (except its siblings of the same put call)."""
    from oneflow_b200.one_embedding.cached_store import DeviceLruCache
    line = 16
    cache = DeviceLruCache(capacity_rows=8 * 32, line=line, device="cuda")     # 8 sets
    n_sets = cache.n_sets

    def set_of(k):
        x = k & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 30; x = (x * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 27; x = (x * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 31
        return x % n_sets
    truth, last_use, resident = {}, {}, set()
    g = torch.Generator().manual_seed(5)
    clock = 0
    for rnd in range(40):
        keys = torch.unique(torch.randint(0, 600, (96,), generator=g))
        klist = keys.tolist()
        rows, hit, miss = cache.get(keys.cuda())
        clock += 1
        assert hit.cpu().tolist() == [k in resident for k in klist], rnd
        assert sorted(miss.cpu().tolist()) == [i for i, k in enumerate(klist) if k not in resident]
        for i, k in enumerate(klist):
            if k in resident:
                assert torch.equal(rows[i].cpu(), truth[k]), (rnd, k)
                last_use[k] = clock
        new_rows = torch.randn(len(klist), line, generator=g)
        before = {s: sum(1 for k in resident if set_of(k) == s) for s in range(n_sets)}
        incoming = {s: sum(1 for k in klist if k not in resident and set_of(k) == s) for s in range(n_sets)}
        ek, er = cache.put(keys.cuda(), new_rows.cuda())
        clock += 1
        for i, k in enumerate(klist):
            truth[k] = new_rows[i]
            resident.add(k)
            last_use[k] = clock
        out_per_set = {}
        for j, k in enumerate(ek.tolist()):
            assert k in resident, (rnd, k)
            assert torch.equal(er[j].cpu(), truth[k]), (rnd, k)          # the pushed-out row is the latest value of its key
            resident.discard(k)
            out_per_set[set_of(k)] = out_per_set.get(set_of(k), 0) + 1
        for s in range(n_sets):
            assert out_per_set.get(s, 0) == max(0, before[s] + incoming[s] - 32), (rnd, s)
            assert sum(1 for k in resident if set_of(k) == s) <= 32
        for k in ek.tolist():
            stay = [last_use[r] for r in resident if set_of(r) == set_of(k) and last_use[r] < clock]
            assert not stay or last_use[k] <= max(stay) or last_use[k] == clock, (rnd, k)
    dk, dr = cache.dump()
    assert sorted(dk.cpu().tolist()) == sorted(resident)
    for j, k in enumerate(dk.tolist()):
        assert torch.equal(dr[j].cpu(), truth[k])
    assert _native.read_status() == (0, 0)


def test_cached_store_on_cuda_follows_the_full_store(tmp_path):
    import oneflow_b200 as flow
    oe = flow.one_embedding
    tables = [oe.make_table_options(oe.make_uniform_initializer(-0.1, 0.1))]

    def build(opts, name):
        emb = oe.MultiTableEmbedding(name, embedding_dim=8, dtype=torch.float32, key_type=torch.int64, tables=tables, store_options=opts)
        return emb, oe.Optimizer(emb, flow.optim.SGD, lr=0.1)
    full, fopt = build(oe.make_device_mem_store_options(str(tmp_path / "f"), capacity=4096, size_factor=1), "gfull")
    cached, copt = build(oe.make_cached_host_mem_store_options(64 * 8 * 4 / (1 << 20), str(tmp_path / "c"), capacity=4096, size_factor=1), "gcached")
    g = torch.Generator().manual_seed(9)
    for step in range(10):
        ids = torch.randint(0, 300, (128, 1), generator=g).cuda()
        outs = []
        for emb, opt in ((full, fopt), (cached, copt)):
            y = emb(ids)
            ((y - 0.5) ** 2).sum().backward()
            opt.step()
            opt.zero_grad()
            outs.append(y.detach())
        assert torch.allclose(outs[0], outs[1], atol=1e-6), step
    assert cached.store.stats["evicted"] > 0
    from oneflow_b200.one_embedding.cached_store import DeviceLruCache
    assert isinstance(cached.store.cache, DeviceLruCache)
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)
