"""Worker for the multi-process tests of the flow API (global tensors, boxing, nn.Graph, checkpoints):
    python -m oneflow.distributed.launch --nproc_per_node N tests/flow_worker.py <case> [tmpdir]"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch

import oneflow as flow
import oneflow.nn as nn


def mlp_config1(tmp):
    """Two-rank CPU training check: 2-layer MLP 784->512->10 fp32 ReLU, params broadcast on cpu[0,1], input split(0),
    nn.Graph + SGD lr 0.1 + cross-entropy, seed 0, 20 steps, then save/load round trip."""
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    torch.manual_seed(0)
    P = flow.placement("cpu", list(range(world)))
    model = nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 10))
    ref = nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 10))
    ref.load_state_dict(model.state_dict())
    model.to_global(P, flow.sbp.broadcast)
    g = torch.Generator().manual_seed(0)
    x_full = torch.randn(64, 784, generator=g)
    y_full = torch.randint(0, 10, (64,), generator=g)
    x = flow.tensor(x_full, placement=P, sbp=flow.sbp.split(0))
    y = flow.tensor(y_full, placement=P, sbp=flow.sbp.split(0))
    assert x.to_local().shape == (64 // world, 784)
    opt = flow.optim.SGD(model.parameters(), lr=0.1)
    loss_fn = nn.CrossEntropyLoss()

    class TrainGraph(nn.Graph):
        def __init__(self):
            super().__init__()
            self.model = model
            self.loss_fn = loss_fn
            self.add_optimizer(opt)

        def build(self, x, y):
            loss = self.loss_fn(self.model(x), y)
            loss.backward()
            return loss

    graph = TrainGraph()
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    losses, ref_losses = [], []
    for step in range(20):
        loss = graph(x, y)
        losses.append(float(loss.numpy()))
        ref_opt.zero_grad()
        rl = torch.nn.functional.cross_entropy(ref(x_full), y_full)
        rl.backward()
        ref_opt.step()
        ref_losses.append(rl.item())
    assert np.allclose(losses, ref_losses, rtol=1e-4, atol=1e-5), (losses[:3], ref_losses[:3], losses[-1], ref_losses[-1])
    assert losses[-1] < losses[0]
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert p.sbp == (flow.sbp.broadcast,), p.sbp
        assert np.allclose(p.numpy(), q.detach().numpy(), rtol=1e-4, atol=1e-5), n
    # save / load round trip of the graph state (directory format, written by rank 0)
    path = os.path.join(tmp, "ckpt")
    flow.save(graph.state_dict(), path, global_dst_rank=0, save_as_external_data=True)
    flow.comm.barrier()
    loaded = flow.load(path, global_src_rank=0)
    w = loaded["model"]["0.weight"]
    assert w.is_global and w.placement == flow.placement("cpu", [0])
    w2 = w.to_global(P, flow.sbp.broadcast)
    assert np.allclose(w2.numpy(), model[0].weight.numpy())
    assert int(loaded["System-Train-TrainStep"].to_global(P, flow.sbp.broadcast).numpy()[0]) == 20
    model2 = nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 10)).to_global(P, flow.sbp.broadcast)
    sd = flow.utils.global_view.to_global(loaded["model"], P, flow.sbp.broadcast)
    model2.load_state_dict(sd)
    out1, out2 = model(x), model2(x)
    assert np.allclose(out1.numpy(), out2.numpy(), atol=1e-6)
    if rank == 0:
        print("LOSSES", losses[0], losses[-1])


def boxing_exhaustive(tmp):
    """Every 1-D sbp pair on odd shapes, and 2-D pairs on [[0,1],[2,3]] when 4 ranks are available."""
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    S, B, Pm = flow.sbp.split, flow.sbp.broadcast, flow.sbp.partial_sum
    g = torch.Generator().manual_seed(3)
    base = torch.randn(5, 7, 4, generator=g)
    P1 = flow.placement("cpu", list(range(world)))
    one_d = [S(0), S(1), S(2), B, Pm]
    for a in one_d:
        for b in one_d:
            x = flow.tensor(base, placement=P1, sbp=B).to_global(P1, a)
            y = x.to_global(P1, b)
            assert y.sbp == (b,)
            assert np.allclose(y.numpy(), base.numpy(), atol=1e-5), (str(a), str(b))
    if world >= 4:
        P2 = flow.placement("cpu", [[0, 1], [2, 3]])
        base2 = torch.randn(8, 6, generator=g)
        kinds = [S(0), S(1), B, Pm]
        for a0 in kinds:
            for a1 in kinds:
                for b0 in kinds:
                    for b1 in kinds:
                        x = flow.tensor(base2, placement=P2, sbp=(B, B)).to_global(P2, (a0, a1))
                        y = x.to_global(P2, (b0, b1))
                        assert np.allclose(y.numpy(), base2.numpy(), atol=1e-5), (str(a0), str(a1), str(b0), str(b1))
        # placement change: [0,1] -> [2,3] and 1-D -> 2-D
        Pa, Pb = flow.placement("cpu", [0, 1]), flow.placement("cpu", [2, 3])
        x = flow.tensor(base2, placement=Pa, sbp=S(0))
        y = x.to_global(Pb, S(1))
        z = y.to_global(P2, (S(0), B))
        assert np.allclose(z.numpy(), base2.numpy(), atol=1e-6)
        if rank in (0, 1):
            assert y.to_local().numel() == 0
    if rank == 0:
        print("BOXING OK")


def global_ops(tmp):
    """SBP signatures of matmul (all five), reductions, layer norm, embedding; autograd through to_global."""
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    S, B, Pm = flow.sbp.split, flow.sbp.broadcast, flow.sbp.partial_sum
    P = flow.placement("cpu", list(range(world)))
    g = torch.Generator().manual_seed(4)
    a, b = torch.randn(6, 8, generator=g), torch.randn(8, 4, generator=g)
    ref = a @ b
    cases = [((S(0), B), S(0)), ((B, S(1)), S(1)), ((S(1), S(0)), Pm), ((B, B), B)]
    for (sa, sb), so in cases:
        x = flow.tensor(a, placement=P, sbp=B).to_global(P, sa)
        y = flow.tensor(b, placement=P, sbp=B).to_global(P, sb)
        z = flow.matmul(x, y)
        assert z.sbp == (so,), (str(sa), str(sb), z.sbp)
        assert np.allclose(z.numpy(), ref.numpy(), atol=1e-5)
    x = flow.tensor(a, placement=P, sbp=S(0))
    assert x.sum(0).sbp == (Pm,) and np.allclose(x.sum(0).numpy(), a.sum(0).numpy(), atol=1e-5)
    assert x.sum(1).sbp == (S(0),)
    assert np.allclose(x.mean().numpy(), a.mean().numpy(), atol=1e-6)
    ln = torch.nn.LayerNorm(8)
    assert np.allclose(torch.nn.functional.layer_norm(x, (8,)).numpy(), torch.nn.functional.layer_norm(a, (8,)).numpy(), atol=1e-5)
    # tensor-parallel MLP: column-parallel then row-parallel gives a partial-sum output
    w1, w2 = torch.randn(16, 8, generator=g), torch.randn(4, 16, generator=g)
    xg = flow.tensor(a, placement=P, sbp=B).requires_grad_(True)
    W1 = flow.tensor(w1, placement=P, sbp=S(0)).requires_grad_(True)
    W2 = flow.tensor(w2, placement=P, sbp=S(1)).requires_grad_(True)
    h = torch.relu(torch.nn.functional.linear(xg, W1))
    assert h.sbp == (S(1),)
    o = torch.nn.functional.linear(h, W2)
    assert o.sbp == (Pm,)
    o.to_global(P, B).sum().backward()
    at = a.clone().requires_grad_(True); w1t = w1.clone().requires_grad_(True); w2t = w2.clone().requires_grad_(True)
    torch.nn.functional.linear(torch.relu(torch.nn.functional.linear(at, w1t)), w2t).sum().backward()
    assert np.allclose(W1.grad.numpy(), w1t.grad.numpy(), atol=1e-4)
    assert np.allclose(W2.grad.numpy(), w2t.grad.numpy(), atol=1e-4)
    assert np.allclose(xg.grad.numpy(), at.grad.numpy(), atol=1e-4)
    # vocabulary-parallel embedding
    table = torch.randn(10 * world, 6, generator=g)
    idx = torch.randint(0, 10 * world, (4, 3), generator=g)
    E = flow.tensor(table, placement=P, sbp=S(0))
    I = flow.tensor(idx, placement=P, sbp=B)
    e = torch.nn.functional.embedding(I, E)
    assert e.sbp == (Pm,) and np.allclose(e.numpy(), table[idx].numpy(), atol=1e-6)
    # dimension-preserving ops keep a split that is not on the dimension they work along (no gather happens)
    t4 = torch.randn(2 * world, 4, 6, 6, generator=g)
    X = flow.tensor(t4, placement=P, sbp=S(0))
    F = torch.nn.functional

    def same(got, want, sbp):
        assert got.sbp == (sbp,), (got.sbp, sbp)
        assert np.allclose(got.numpy(), want.numpy(), atol=1e-5)
    same(X[:, 1], t4[:, 1], S(0))                                   # select on another dimension
    same(X[:, 1:3], t4[:, 1:3], S(0))                               # slice on another dimension
    same(X.select(0, 1), t4.select(0, 1), B)                        # select on the split dimension: gathered
    same(torch.cat([X, X * 2], 1), torch.cat([t4, t4 * 2], 1), S(0))
    same(torch.stack([X, X + 1], 0), torch.stack([t4, t4 + 1], 0), S(1))
    for got, want in zip(X.split(2, dim=1), t4.split(2, dim=1)):
        same(got, want, S(0))
    for got, want in zip(X.unbind(1), t4.unbind(1)):
        same(got, want, S(0))
    ii = torch.tensor([2, 0])
    same(X.index_select(1, flow.tensor(ii, placement=P, sbp=B)), t4.index_select(1, ii), S(0))
    same(F.max_pool2d(X, 2), F.max_pool2d(t4, 2), S(0))
    same(F.avg_pool2d(X, 2), F.avg_pool2d(t4, 2), S(0))
    same(F.adaptive_avg_pool2d(X, 1), F.adaptive_avg_pool2d(t4, 1), S(0))
    same(F.dropout(X, 0.0, True), t4, S(0))
    rm, rv = torch.zeros(4), torch.ones(4)
    Bn = lambda t: flow.tensor(t, placement=P, sbp=B)  # noqa: E731
    same(F.batch_norm(X, Bn(rm), Bn(rv), training=False), F.batch_norm(t4, rm, rv, training=False), S(0))
    got = F.batch_norm(X, Bn(rm.clone()), Bn(rv.clone()), training=True)  # training: statistics of the whole batch
    assert np.allclose(got.numpy(), F.batch_norm(t4, rm.clone(), rv.clone(), training=True).numpy(), atol=1e-5)
    q = torch.randn(2 * world, 2, 5, 8, generator=g)
    Q = flow.tensor(q, placement=P, sbp=S(0))
    same(F.scaled_dot_product_attention(Q, Q, Q, is_causal=True), F.scaled_dot_product_attention(q, q, q, is_causal=True), S(0))
    Xr = flow.tensor(t4, placement=P, sbp=S(0)).requires_grad_(True)
    tr = t4.clone().requires_grad_(True)
    (F.max_pool2d(torch.cat([Xr[:, :2], Xr[:, 2:] * 3], 1), 2).sum()).backward()
    (F.max_pool2d(torch.cat([tr[:, :2], tr[:, 2:] * 3], 1), 2).sum()).backward()
    assert np.allclose(Xr.grad.numpy(), tr.grad.numpy(), atol=1e-5)
    if rank == 0:
        print("GLOBAL OPS OK")


def graph_features(tmp):
    """Gradient accumulation == big batch, ZeRO turns B params into S(0), pipeline stages on different
    placements, grad scaler, lr scheduler, activation checkpointing."""
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    S, B = flow.sbp.split, flow.sbp.broadcast
    P = flow.placement("cpu", list(range(world)))
    torch.manual_seed(1)

    def make():
        torch.manual_seed(1)
        return nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))
    g = torch.Generator().manual_seed(2)
    xf, yf = torch.randn(16 * world, 16, generator=g), torch.randint(0, 4, (16 * world,), generator=g)

    def run(acc, zero, ckpt=False, sched=False, scaler=None):
        m = make().to_global(P, B)
        opt = flow.optim.SGD(m.parameters(), lr=0.05, momentum=0.9)
        lr_sch = flow.optim.lr_scheduler.StepLR(opt, step_size=2, gamma=0.5) if sched else None

        class G(nn.Graph):
            def __init__(self):
                super().__init__()
                self.m = m
                self.add_optimizer(opt, lr_sch=lr_sch)
                if acc > 1:
                    self.config.set_gradient_accumulation_steps(acc)
                if zero:
                    self.config.enable_zero(True, stage=zero, shard_min_size=1)
                if ckpt:
                    self.m.to(nn.graph.GraphModule).activation_checkpointing = True
                if scaler is not None:
                    self.set_grad_scaler(scaler)

            def build(self, x, y):
                loss = torch.nn.functional.cross_entropy(self.m(x), y)
                loss.backward()
                return loss
        gr = G()
        x = flow.tensor(xf, placement=P, sbp=S(0))
        y = flow.tensor(yf, placement=P, sbp=S(0))
        out = [gr(x, y) for _ in range(4)]
        return m, out, gr
    m1, o1, _ = run(1, 0)
    m2, o2, _ = run(2, 0)
    assert o2[0].shape == (2,)
    for p, q in zip(m1.parameters(), m2.parameters()):
        assert np.allclose(p.numpy(), q.numpy(), atol=1e-5)
    m3, o3, g3 = run(1, 2)
    assert m3[0].weight.sbp == (S(0),), m3[0].weight.sbp
    for p, q in zip(m1.parameters(), m3.parameters()):
        assert np.allclose(p.numpy(), q.numpy(), atol=1e-5)
    m4, o4, _ = run(1, 0, ckpt=True, sched=True, scaler=flow.amp.StaticGradScaler(128.0))
    assert all(np.isfinite(float(o.numpy())) for o in o4)
    sd = g3.state_dict()
    assert "System-Train-TrainStep" in sd and "m" in sd
    # pipeline: two stages on disjoint placements
    if world >= 2:
        P0, P1 = flow.placement("cpu", [0]), flow.placement("cpu", [1])
        torch.manual_seed(5)
        s0, s1 = nn.Linear(16, 32), nn.Linear(32, 4)
        r0, r1 = nn.Linear(16, 32), nn.Linear(32, 4)
        r0.load_state_dict(s0.state_dict()); r1.load_state_dict(s1.state_dict())
        s0.to_global(P0, B); s1.to_global(P1, B)
        opt = flow.optim.SGD(list(s0.parameters()) + list(s1.parameters()), lr=0.1)

        class PG(nn.Graph):
            def __init__(self):
                super().__init__()
                self.s0, self.s1 = s0, s1
                self.s0.to(nn.graph.GraphModule).set_stage(0, P0)
                self.s1.to(nn.graph.GraphModule).set_stage(1, P1)
                self.config.set_gradient_accumulation_steps(2)
                self.add_optimizer(opt)

            def build(self, x, y):
                h = torch.relu(self.s0(x))
                out = self.s1(h)
                y = y.to_global(P1, B)
                loss = torch.nn.functional.cross_entropy(out, y)
                loss.backward()
                return loss
        pg = PG()
        x = flow.tensor(xf[:8], placement=P0, sbp=B)
        y = flow.tensor(yf[:8], placement=P0, sbp=B)
        for _ in range(3):
            loss = pg(x, y)
        ro = torch.optim.SGD(list(r0.parameters()) + list(r1.parameters()), lr=0.1)
        for _ in range(3):
            ro.zero_grad()
            (torch.nn.functional.cross_entropy(r1(torch.relu(r0(xf[:4]))), yf[:4]) / 2).backward()
            (torch.nn.functional.cross_entropy(r1(torch.relu(r0(xf[4:8]))), yf[4:8]) / 2).backward()
            ro.step()
        if rank == 0:
            assert np.allclose(s0.weight.to_local().detach().numpy(), r0.weight.detach().numpy(), atol=1e-5)
            assert loss.to_local().numel() == 0     # loss lives on the last stage only
        if rank == 1:
            assert np.allclose(s1.weight.to_local().detach().numpy(), r1.weight.detach().numpy(), atol=1e-5)
    if rank == 0:
        print("GRAPH FEATURES OK")


def ddp_and_comm(tmp):
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    t = torch.full((4,), float(rank + 1))
    flow.comm.all_reduce(t)
    assert t[0].item() == sum(range(1, world + 1))
    outs = [torch.zeros(2) for _ in range(world)]
    flow.comm.all_gather(outs, torch.full((2,), float(rank)))
    assert [o[0].item() for o in outs] == list(range(world))
    rs = torch.zeros(3)
    flow.comm.reduce_scatter(rs, [torch.full((3,), float(rank + r)) for r in range(world)])
    assert rs[0].item() == sum(r2 + rank for r2 in range(world))
    if world >= 2:
        if rank == 0:
            flow.comm.send(torch.arange(6.0).view(2, 3), 1)
        elif rank == 1:
            got = flow.comm.recv(0)
            assert got.shape == (2, 3) and got[1, 2].item() == 5.0
    torch.manual_seed(7 + rank)   # different init per rank: DDP must broadcast rank 0's
    m = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2), nn.Linear(2, 2))
    ddp = nn.parallel.DistributedDataParallel(m, bucket_size=2)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(5, 8, generator=g)
    ddp(x).sum().backward()
    ddp.finish_pending()
    grads = [p.grad.clone() for p in m.parameters()]
    for gr in grads:
        ref = gr.clone()
        flow.comm.all_reduce(ref)
        assert torch.allclose(ref / world, gr, atol=1e-6)   # already averaged and identical on every rank
    if rank == 0:
        print("DDP COMM OK")


def auto_parallel_graph(tmp):
    """nn.Graph with config.enable_auto_parallel: the solver shards the big Linear layers, losses match the
    fully replicated run."""
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    P = flow.placement("cpu", list(range(world)))

    def run(auto):
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(256, 2048), nn.ReLU(), nn.Linear(2048, 256))
        model.to_global(P, flow.sbp.broadcast)
        opt = flow.optim.SGD(model.parameters(), lr=0.05)
        g = torch.Generator().manual_seed(1)
        x = flow.tensor(torch.randn(16, 256, generator=g), placement=P, sbp=flow.sbp.broadcast)
        y = flow.tensor(torch.randn(16, 256, generator=g), placement=P, sbp=flow.sbp.broadcast)

        class G(nn.Graph):
            def __init__(self):
                super().__init__()
                self.model = model
                self.add_optimizer(opt)
                if auto:
                    self.config.enable_auto_parallel(True)
                    self.config.set_auto_parallel_computation_cost_ratio(1e-4)   # tiny test layers: make compute matter

            def build(self, a, b):
                loss = ((self.model(a) - b) ** 2).mean()
                loss.backward()
                return loss

        graph = G()
        out = []
        for _ in range(4):
            l = graph(x, y)
            l = l.to_global(P, flow.sbp.broadcast).to_local() if hasattr(l, "to_global") else l
            out.append(float(l))
        return out, getattr(graph, "_auto_parallel_choices", None), model

    base, _, _ = run(False)
    auto, choices, model = run(True)
    assert choices is not None and any(k != "data" for _, k in choices), choices
    w0 = model[0].weight
    assert any(s.kind == "S" for s in w0.sbp) or any(s.kind == "S" for s in model[2].weight.sbp)
    for a, b in zip(base, auto):
        assert abs(a - b) < 1e-4 * max(1.0, abs(a)), (base, auto, choices)
    assert auto[-1] < auto[0]
    if rank == 0:
        print("AUTO PARALLEL", choices, auto)

    # general form: any module, traced; the plan of a residual MLP at a small token count is column -> row parallel, and
    # the module distributed by it computes what the replicated module computes
    from oneflow_b200.framework import auto_parallel as AP

    class Res(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln, self.fc1, self.fc2 = nn.LayerNorm(64), nn.Linear(64, 256), nn.Linear(256, 64)

        def forward(self, x):
            return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.ln(x))))

    torch.manual_seed(3)
    ref_m = Res()
    xs = torch.randn(8, 64)
    want = ref_m(xs)
    plan, _ = AP.plan_module(ref_m, xs, world, input_sbp=flow.sbp.broadcast)
    assert plan["fc1"].kind == "column" and plan["fc2"].kind == "row", {k: v.kind for k, v in plan.items()}
    m2 = Res()
    m2.load_state_dict(ref_m.state_dict())
    m2.to_global(P, flow.sbp.broadcast)
    AP.apply_plan(m2, plan, P)
    assert m2.fc1.weight.sbp[0] == flow.sbp.split(0) and m2.fc2.weight.sbp[0] == flow.sbp.split(1)
    assert tuple(m2.fc1.weight.to_local().shape) == (256 // world, 64)
    got = m2(flow.tensor(xs, placement=P, sbp=flow.sbp.broadcast)).to_global(P, flow.sbp.broadcast).to_local()
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()


def data_readers(tmp):
    """Sharded readers: every rank reads its own part files / batch slice; dense outputs are global split(0) tensors;
    the torch.distributed-shaped wrappers of flow.distributed forward to flow.comm."""
    import numpy as np
    from oneflow_b200.utils.ofrecord import write_ofrecord_file
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    d = os.path.join(tmp, "rec")
    if rank == 0:
        os.makedirs(d, exist_ok=True)
        for part in range(2 * world):
            write_ofrecord_file(os.path.join(d, f"part-{part:03d}"),
                                [{"label": np.array([part * 100 + i], np.int32), "x": np.full(4, part * 100 + i, np.float32)} for i in range(6)])
        np.arange(40 * 3, dtype=np.float32).reshape(40, 3).tofile(os.path.join(tmp, "raw.bin"))
    flow.comm.barrier()
    pl = flow.placement("cpu", list(range(world)))
    r = flow.nn.OFRecordReader(d, batch_size=4 * world, data_part_num=2 * world, part_name_suffix_length=3, placement=pl, sbp=flow.sbp.split(0))
    lab = flow.nn.OFRecordRawDecoder("label", shape=(1,), dtype=flow.int32)
    xs = flow.nn.OFRecordRawDecoder("x", shape=(4,), dtype=flow.float32)
    b = r()
    la, x = lab(b), xs(b)
    assert la.is_global and tuple(la.shape) == (4 * world, 1) and tuple(x.shape) == (4 * world, 4)
    mine = la.to_local().reshape(-1).tolist()
    assert len(mine) == 4 and all((v // 100) % world == rank for v in mine), mine      # parts dealt round robin
    full = la.to_global(pl, flow.sbp.broadcast).to_local().reshape(-1).tolist()
    assert len(set(full)) == 4 * world
    assert torch.equal(x.to_local()[:, 0], la.to_local().reshape(-1).float())
    rr = flow.nn.RawReader([os.path.join(tmp, "raw.bin")], shape=(3,), dtype=flow.float32, batch_size=2 * world, random_shuffle=False,
                           placement=pl, sbp=flow.sbp.split(0))
    y = rr()
    assert tuple(y.shape) == (2 * world, 3) and y.to_local()[0, 0].item() == rank * 2 * 3
    cf = flow.nn.CoinFlip(batch_size=2 * world, random_seed=1, placement=pl, sbp=flow.sbp.split(0))()
    assert tuple(cf.shape) == (2 * world,)
    # flow.distributed wrappers
    D = flow.distributed
    t = torch.full((3,), float(rank + 1))
    D.all_reduce(t, D.ReduceOp.SUM)
    assert t[0].item() == sum(range(1, world + 1))
    outs = [torch.zeros(2) for _ in range(world)]
    D.all_gather(outs, torch.full((2,), float(rank)))
    assert [o[0].item() for o in outs] == list(range(world))
    bt = torch.full((2,), float(rank))
    D.broadcast(bt, 0)
    assert bt[0].item() == 0.0
    assert D.get_rank() == rank and D.get_world_size() == world and D.is_initialized() and D.is_available()
    if rank == 0:
        D.send(torch.arange(4.0), 1)
    elif rank == 1:
        got = torch.zeros(4)
        D.recv(got, 0)
        assert got[3].item() == 3.0
    D.barrier()


def embedding_stages(tmp):
    """The OneEmbedding stage ops across ranks: id shuffle -> lookup -> embedding shuffle equals the fused forward, and the
    gradient shuffle delivers every rank's gradient rows, summed per key, to the key's owner."""
    C = flow._C
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    opts = flow.one_embedding.make_table_options(flow.one_embedding.make_uniform_initializer(-0.1, 0.1))
    store = flow.one_embedding.make_device_mem_store_options(persistent_path=os.path.join(tmp, "emb"), capacity=4096, size_factor=1)
    emb = flow.one_embedding.MultiTableEmbedding("stages", embedding_dim=4, dtype=flow.float32, key_type=flow.int64,
                                                 tables=[opts], store_options=store)
    g = torch.Generator().manual_seed(5 + rank)
    ids = torch.randint(0, 20, (12,), generator=g)
    mat, inv_part, n_cur, cur_ids, cur_tids, cur_inv = C.one_embedding_id_shuffle(ids, None, 1, "stages")
    assert mat.numel() == world * world and int(mat.reshape(world, world)[rank].sum()) == torch.unique(ids).numel()
    lines = C.one_embedding_lookup(n_cur, cur_ids, cur_tids, flow.float32, flow.float32, 4, 4, "stages", "", "", 0)
    out = C.one_embedding_embedding_shuffle(lines, mat, cur_inv, inv_part, "stages")
    assert torch.allclose(out, emb(ids).reshape(-1, 4))
    # a key held by two ranks resolves to the same row on both
    gathered = [torch.zeros(12, 5) for _ in range(world)]
    flow.comm.all_gather(gathered, torch.cat([ids.float().unsqueeze(1), out], 1))
    table = {}
    for t in gathered:
        for row in t.tolist():
            assert table.setdefault(row[0], row[1:]) == row[1:]
    grad = torch.full((12, 4), float(rank + 1))
    ug = C.one_embedding_embedding_gradient_shuffle(grad, mat, cur_inv, inv_part, "stages")
    assert ug.shape == (int(n_cur), 4)
    total = ug.sum().reshape(1)
    flow.comm.all_reduce(total)
    assert abs(total.item() - sum(12 * 4 * (r + 1) for r in range(world))) < 1e-3


def rank_divergence(tmp):
    """A rank that skips a global-tensor operation makes its peers raise within ONEFLOW_TIMEOUT_SECONDS instead of
    hanging in the collective; ranks that run DIFFERENT operations are told so; heartbeats name a rank that is gone.
    (The reference's check: python/oneflow/test/exceptions/test_global_branch_error_local_to_global_with_split_sbp.py.)"""
    import time
    from oneflow_b200.framework import control_plane as CP
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    assert CP.client() is not None, "the process group must have been created over the in-tree control store"
    P = flow.placement("cpu", list(range(world)))
    os.environ["ONEFLOW_TIMEOUT_SECONDS"] = "2"
    # 1. everybody agrees: the check is transparent
    x = flow.tensor(torch.arange(8.0).reshape(4, 2), placement=P, sbp=flow.sbp.split(0))
    assert np.allclose(x.to_global(P, flow.sbp.broadcast).numpy(), np.arange(8.0).reshape(4, 2))
    # 2. rank 1 takes another branch and never calls to_global
    t0 = time.time()
    if rank == 0:
        try:
            flow.rand(2).to_global(placement=P, sbp=flow.sbp.split(0))
            raise SystemExit("the missing rank was not noticed")
        except RuntimeError as e:
            assert "Maybe executing different code in different ranks" in str(e), str(e)
            assert "did not reach" in str(e)
        assert 1.5 < time.time() - t0 < 20
    else:
        time.sleep(3)
    os.environ["ONEFLOW_TIMEOUT_SECONDS"] = "30"
    CP.barrier("after-skip", world, 30)
    CP.resync()
    # 3. the ranks run different boxing steps on the same group
    os.environ["ONEFLOW_TIMEOUT_SECONDS"] = "5"
    y = flow.tensor(torch.ones(4, 4), placement=P, sbp=flow.sbp.split(0))
    try:
        y.to_global(P, flow.sbp.broadcast if rank == 0 else flow.sbp.split(1))
        raise SystemExit("the differing operation was not noticed")
    except RuntimeError as e:
        assert "differs between ranks" in str(e) and "Maybe executing different code" in str(e), str(e)
    os.environ.pop("ONEFLOW_TIMEOUT_SECONDS")
    CP.barrier("after-mismatch", world, 30)
    CP.resync()
    # 4. heartbeats: every rank is alive now
    assert flow.env.lost_ranks(5.0) == []
    if rank == 0:
        print("RANK DIVERGENCE OK")
    CP.barrier("end", world, 30)


def native_data_parallel(tmp):
    """The native graph compiler under data parallelism: every rank runs forward and backward of its shard of the batch in
    its own compiled plan, the fp32 gradients are averaged over the ranks by one collective outside the graph, every rank
    applies the same update. The result equals one plan over the whole batch."""
    import numpy as np
    import torch.nn.functional as F
    from oneflow_b200.utils import export as E
    rank, world = flow.env.get_rank(), flow.env.get_world_size()

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.ln, self.fc2 = torch.nn.Linear(32, 64), torch.nn.LayerNorm(64), torch.nn.Linear(64, 16)

        def forward(self, x, y):
            return F.cross_entropy(self.fc2(self.ln(F.gelu(self.fc1(x)))), y)

    torch.manual_seed(0)
    m = Net()
    for prm in m.parameters():
        prm.data = prm.data.bfloat16().float()
    x, y = torch.randn(16 * world, 32).bfloat16().float(), torch.randint(0, 16, (16 * world,))
    lo, hi = 16 * rank, 16 * (rank + 1)
    shard = E.export_graph(m, (x[lo:hi], y[lo:hi]), os.path.join(tmp, f"shard{rank}"), fuse=False)
    whole = E.export_graph(m, (x, y), os.path.join(tmp, f"whole{rank}"), fuse=False)
    kw = dict(device=-1, optimizer="adamw", lr=1e-2, clip_grad_norm=1.0)
    g = E.TrainingGraph(shard, external_gradient_reduction=True, **kw)
    ref = E.TrainingGraph(whole, **kw)
    for _ in range(4):
        g.step(x[lo:hi].numpy(), y[lo:hi].numpy())
        g.all_reduce_gradients()
        g.apply_update()
        ref.step(x.numpy(), y.numpy())
    mine, want = g.parameters(), ref.parameters()
    for k in want:
        assert np.abs(mine[k] - want[k]).max() < 1e-2, (k, float(np.abs(mine[k] - want[k]).max()))
    # every rank holds the same weights, bit for bit
    flat = torch.from_numpy(np.concatenate([mine[k] for k in sorted(mine)]))
    gathered = [torch.empty_like(flat) for _ in range(world)]
    torch.distributed.all_gather(gathered, flat)
    assert all(torch.equal(gathered[0], t) for t in gathered)
    assert g.evaluate(x[lo:hi].numpy(), y[lo:hi].numpy()) > 0


if __name__ == "__main__":
    case = sys.argv[1]
    tmp = sys.argv[2] if len(sys.argv) > 2 else "/tmp"
    {"mlp_config1": mlp_config1, "boxing": boxing_exhaustive, "global_ops": global_ops, "graph_features": graph_features,
     "ddp_comm": ddp_and_comm, "auto_parallel": auto_parallel_graph, "data_readers": data_readers, "embedding_stages": embedding_stages, "rank_divergence": rank_divergence, "native_dp": native_data_parallel}[case](tmp)
    if case != "rank_divergence":
        flow.comm.barrier()
    if flow.env.get_rank() == 0:
        print(f"CASE {case} OK")
