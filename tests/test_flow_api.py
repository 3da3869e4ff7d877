"""The flow API on CPU ranks: global tensors, exhaustive boxing, SBP signatures, nn.Graph (the two-rank MLP training check,
gradient accumulation, ZeRO, pipeline stages), DDP, flow.comm — each case runs as real processes under the
launcher (gloo), the way the reference runs its multi-rank tests."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_PORT = [29800]


def launch(case, nproc, timeout=900):
    _PORT[0] += 1
    tmp = tempfile.mkdtemp()
    cmd = [sys.executable, "-m", "oneflow_b200.distributed.launch", "--nproc_per_node", str(nproc), "--master_port",
           str(_PORT[0]), os.path.join(ROOT, "tests", "flow_worker.py"), case, tmp]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, cwd=ROOT, env=env)
    assert p.returncode == 0 and f"CASE {case} OK" in p.stdout, p.stdout[-4000:]


def test_mlp_graph_sgd_two_cpu_ranks():
    launch("mlp_config1", 2)


@pytest.mark.parametrize("n", [2, 4])
def test_boxing_exhaustive(n):
    launch("boxing", n)


def test_global_op_sbp_signatures():
    launch("global_ops", 2)


def test_graph_features():
    launch("graph_features", 2)


def test_ddp_and_comm():
    launch("ddp_comm", 2)


def test_graph_auto_parallel():
    launch("auto_parallel", 2)


def test_sharded_data_readers_and_distributed_wrappers():
    launch("data_readers", 2)


def test_rank_divergence_is_reported_not_waited_for():
    launch("rank_divergence", 2, timeout=180)


def test_one_embedding_stage_ops_two_ranks():
    launch("embedding_stages", 2)


def test_launcher_kills_group_on_failure(tmp_path):
    script = tmp_path / "boom.py"
    script.write_text("import os, sys, time\nif os.environ['RANK']=='1': sys.exit(3)\ntime.sleep(60)\n")
    cmd = [sys.executable, "-m", "oneflow_b200.distributed.launch", "--nproc_per_node", "2", "--master_port", "29899", str(script)]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=40, cwd=ROOT)
    assert p.returncode != 0


# ---------------------------------------------------------------------------------------------- single process
def test_placement_and_sbp_basics():
    import oneflow as flow
    p = flow.placement("cuda", [[0, 1], [2, 3]])
    assert p.hierarchy == (2, 2) and p.ranks.tolist() == [[0, 1], [2, 3]]
    assert p.coords(2) == (1, 0) and p.axis_ranks(0, 1) == [1, 3] and p.axis_ranks(1, 2) == [2, 3]
    assert flow.sbp.split(1) is flow.sbp.split(1) and str(flow.sbp.split(1)) == "S(1)"
    assert flow.sbp.broadcast.is_broadcast() and flow.sbp.partial_sum.is_partial_sum()
    with pytest.raises(ValueError):
        flow.placement("cpu", [0, 0])


def test_balanced_splitter_and_slice_views():
    from oneflow_b200.framework.balanced_splitter import BalancedSplitter
    from oneflow_b200.framework.nd_sbp import local_shape, slice_view
    import oneflow as flow
    bs = BalancedSplitter(10, 4)
    assert [bs.at(i) for i in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [bs.owner(e) for e in range(10)] == [0, 0, 0, 1, 1, 1, 2, 2, 3, 3]
    S, B = flow.sbp.split, flow.sbp.broadcast
    assert slice_view((8, 6), (2, 2), (S(0), S(0)), (1, 0)) == [(4, 6), (0, 6)]
    assert local_shape((7, 5), (2, 2), (S(1), S(0)), (0, 1)) == (3, 3)
    assert local_shape((7, 5), (2, 2), (B, B), (1, 1)) == (7, 5)


def test_checkpoint_formats_single_process(tmp_path):
    import pickletools

    import oneflow as flow
    sd = {"w": torch.nn.Parameter(torch.randn(3, 2)), "b": torch.arange(5), "h": torch.randn(2, 2).bfloat16(), "step": 3,
          "nested": [torch.ones(2), {"k": torch.zeros(1, dtype=torch.int8)}], "dtype": torch.float16}
    f = tmp_path / "single.pt"
    flow.save(sd, f)
    names = [a for op, a, _ in pickletools.genops(f.read_bytes()) if op.name == "GLOBAL"]
    assert "oneflow Tensor" in names and "oneflow.nn Parameter" in names and "oneflow._oneflow_internal dtype" in names
    assert not any(n.startswith("torch") or n.startswith("oneflow_b200") or n.startswith("numpy._core") for n in names), names
    back = flow.load(f)
    assert isinstance(back["w"], torch.nn.Parameter) and torch.equal(back["w"], sd["w"]) and back["dtype"] == torch.float16
    assert torch.equal(back["h"], sd["h"]) and torch.equal(back["nested"][1]["k"], sd["nested"][1]["k"])
    d = tmp_path / "dir"
    flow.save(sd, d, save_as_external_data=True)
    sub = [p for p in d.iterdir() if p.is_dir()]
    assert (d / "pickled_data").exists() and len(sub) == 5
    meta = (sub[0] / "meta").read_text()
    assert meta.startswith("shape {") and "data_type: k" in meta
    back = flow.load(d)
    assert torch.equal(back["b"], sd["b"]) and torch.equal(back["h"], sd["h"])
    # legacy variable directory
    legacy = tmp_path / "legacy"
    from oneflow_b200.framework.check_point import save_tensor_dir
    save_tensor_dir(torch.arange(6.0).view(2, 3), legacy / "fc.weight")
    (legacy / "broken").mkdir()
    (legacy / "snapshot_done").write_text("")
    out = flow.load(legacy)
    assert list(out) == ["fc.weight"] and out["fc.weight"].shape == (2, 3)
    # a torch.save file loads as well
    tf = tmp_path / "t.pt"
    torch.save({"x": torch.ones(3)}, tf)
    assert torch.equal(flow.load(tf)["x"], torch.ones(3))
    # golden meta text as written by the reference for an 8x3 float tensor
    g = tmp_path / "golden"
    g.mkdir()
    (g / "meta").write_text("shape {\n  dim: 8\n  dim: 3\n}\ndata_type: kFloat\n")
    (g / "out").write_bytes(np.arange(24, dtype=np.float32).tobytes())
    from oneflow_b200.framework.check_point import load_tensor_dir
    assert torch.equal(load_tensor_dir(g), torch.arange(24.0).view(8, 3))


def test_optimizers_match_reference_math():
    import oneflow as flow
    torch.manual_seed(0)
    w0, g0 = torch.randn(50), torch.randn(50)
    # AdamW with do_bias_correction: w -= lr/bc1 * m / (sqrt(v)/sqrt(bc2) + eps) + lr*wd*w
    p = torch.nn.Parameter(w0.clone())
    opt = flow.optim.AdamW([p], lr=0.1, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    p.grad = g0.clone()
    opt.step()
    m, v = 0.1 * g0, 0.01 * g0 * g0
    exp = w0 - (0.1 / 0.1) * m / (v.sqrt() / (0.01 ** 0.5) + 1e-8) - 0.1 * 0.1 * w0
    assert torch.allclose(p.detach(), exp, atol=1e-5)
    # momentum SGD with clip_grad_max_norm in the param group
    p = torch.nn.Parameter(w0.clone())
    opt = flow.optim.SGD([{"params": [p], "clip_grad_max_norm": 1.0, "clip_grad_norm_type": 2.0}], lr=0.5, momentum=0.9)
    p.grad = g0.clone()
    opt.clip_grad()
    assert abs(p.grad.norm().item() - 1.0) < 1e-4
    opt.step()
    assert torch.allclose(p.detach(), w0 - 0.5 * g0 / g0.norm(), atol=1e-4)
    lamb = flow.optim.LAMB([torch.nn.Parameter(w0.clone())], lr=0.01)
    lamb.param_groups[0]["params"][0].grad = g0.clone()
    lamb.step()
    sch = flow.optim.lr_scheduler.CosineDecayLR(flow.optim.SGD([torch.nn.Parameter(w0.clone())], lr=1.0), decay_steps=10, alpha=0.1)
    lrs = []
    for _ in range(12):
        lrs.append(sch.get_last_lr()[0])
        sch.optimizer.step()
        sch.step()
    assert abs(lrs[0] - 1.0) < 1e-6 and abs(lrs[10] - 0.1) < 1e-6 and abs(lrs[11] - 0.1) < 1e-6
    w = flow.optim.lr_scheduler.WarmupLR(flow.optim.SGD([torch.nn.Parameter(w0.clone())], lr=1.0), warmup_factor=0.5, warmup_iters=4)
    assert abs(w.get_last_lr()[0] - 0.5) < 1e-6


def test_one_embedding_single_rank_sgd_and_adam(tmp_path):
    import oneflow as flow
    oe = flow.one_embedding
    tables = [oe.make_table_options(oe.make_uniform_initializer(-0.1, 0.1)) for _ in range(3)]
    emb = oe.MultiTableEmbedding("t", embedding_dim=8, dtype=torch.float32, key_type=torch.int64, tables=tables,
                                 store_options=oe.make_device_mem_store_options(str(tmp_path), capacity=1000, size_factor=3))
    opt = oe.Optimizer(emb, flow.optim.Adam, lr=0.1)
    ids = torch.tensor([[1, 2, 3], [1, 5, 3], [7, 2, 9]])
    y0 = emb(ids).detach().clone()
    assert y0.shape == (3, 3, 8) and torch.equal(y0[0, 0], y0[1, 0]) and not torch.equal(y0[0, 0], y0[0, 1])
    target = torch.zeros_like(y0)
    for _ in range(30):
        loss = ((emb(ids) - target) ** 2).sum()
        loss.backward()
        opt.step()
        opt.zero_grad()
    assert emb(ids).abs().max().item() < y0.abs().max().item() * 0.5
    sd = emb.state_dict()
    emb2 = oe.MultiTableEmbedding("t", embedding_dim=8, dtype=torch.float32, key_type=torch.int64, tables=tables,
                                  store_options=oe.make_device_mem_store_options(str(tmp_path), capacity=1000, size_factor=3))
    emb2.load_state_dict(sd)
    assert torch.allclose(emb2(ids), emb(ids))
    with pytest.raises(ValueError):
        oe.Optimizer(oe.MultiTableEmbedding("u", 8, torch.float32, torch.int64, tables,
                                            oe.make_device_mem_store_options(str(tmp_path), 10, size_factor=1)), flow.optim.Adam)


@pytest.mark.parametrize("kind", ["host", "ssd"])
def test_cached_embedding_store_matches_full_store(tmp_path, kind):
    """An LRU cache far smaller than the working set in front of a host-memory / SSD table: training must follow the
    run with the whole table resident, rows must survive being evicted and fetched again, and a snapshot must hold
    every row."""
    import oneflow as flow
    oe = flow.one_embedding
    tables = [oe.make_table_options(oe.make_uniform_initializer(-0.1, 0.1)) for _ in range(2)]

    def build(opts, name):
        emb = oe.MultiTableEmbedding(name, embedding_dim=8, dtype=torch.float32, key_type=torch.int64, tables=tables, store_options=opts)
        return emb, oe.Optimizer(emb, flow.optim.Adam, lr=0.05)
    full, fopt = build(oe.make_device_mem_store_options(str(tmp_path / "full"), capacity=4096, size_factor=3), "full_" + kind)
    budget_mb = 64 * 24 * 4 / (1 << 20)                      # room for 64 rows of 24 floats: the steps touch ~400 distinct rows
    if kind == "host":
        opts = oe.make_cached_host_mem_store_options(budget_mb, str(tmp_path / "h"), capacity=4096, size_factor=3)
    else:
        opts = oe.make_cached_ssd_store_options(budget_mb, str(tmp_path / "s"), capacity=4096, size_factor=3)
    cached, copt = build(opts, "cached_" + kind)
    g = torch.Generator().manual_seed(3)
    for step in range(12):
        ids = torch.randint(0, 200, (64, 2), generator=g)
        outs = []
        for emb, opt in ((full, fopt), (cached, copt)):
            y = emb(ids)
            ((y - 0.5) ** 2).sum().backward()
            opt.step()
            opt.zero_grad()
            outs.append(y.detach())
        assert torch.allclose(outs[0], outs[1], atol=1e-6), step
    st = cached.store
    assert st.stats["evicted"] > 0 and st.stats["misses"] > st.stats["created"] > 0, st.stats   # rows went out and came back
    probe = torch.arange(0, 200).reshape(100, 2)
    assert torch.allclose(full(probe), cached(probe), atol=1e-6)
    snap = st.snapshot()
    assert snap["keys"].numel() == st.size == full.store.size


def test_smart_decay_adam_catches_up_rows_that_skipped_steps(tmp_path):
    """A row that was not touched for some steps decays its moments by beta^skipped and catches the skipped moves up, as
    the reference's sparse kernel does; a row touched every step follows the plain recurrences."""
    import oneflow as flow
    oe = flow.one_embedding
    tables = [oe.make_table_options(oe.make_constant_initializer(1.0))]
    emb = oe.MultiTableEmbedding("sd", embedding_dim=4, dtype=torch.float32, key_type=torch.int64, tables=tables,
                                 store_options=oe.make_device_mem_store_options(str(tmp_path), capacity=100, size_factor=4))
    lr, b1, b2, eps = 0.1, 0.9, 0.999, 1e-8
    opt = oe.Optimizer(emb, oe.SmartDecayAdam, lr=lr, betas=(b1, b2), eps=eps)
    # id 1 is looked up every step, id 2 only at steps 1 and 4
    sched = [[1, 2], [1], [1], [1, 2]]
    w = {1: np.ones(4), 2: np.ones(4)}
    m = {1: np.zeros(4), 2: np.zeros(4)}
    v = {1: np.zeros(4), 2: np.zeros(4)}
    last = {1: 0, 2: 0}
    for step, ids in enumerate(sched, 1):
        x = torch.tensor([ids])
        y = emb(x)
        (y * torch.arange(1.0, 5.0)).sum().backward()       # gradient of every looked-up row: [1, 2, 3, 4]
        opt.step()
        opt.zero_grad()
        g = np.arange(1.0, 5.0)
        for i in ids:
            skip = step - last[i]
            catch = m[i] * b1 * (1 - b1 ** (skip - 1)) / (1 - b1) if skip > 1 else 0.0
            m[i] = b1 ** skip * m[i] + (1 - b1) * g
            v[i] = b2 ** skip * v[i] + (1 - b2) * g * g
            w[i] = w[i] - lr * (m[i] + catch) / (np.sqrt(v[i]) + eps)
            last[i] = step
    got = emb(torch.tensor([[1, 2]])).detach().numpy()[0]
    assert np.allclose(got[0], w[1], atol=1e-5) and np.allclose(got[1], w[2], atol=1e-5), (got, w)
    with pytest.raises(ValueError):    # the step slot needs a fourth block in the stored line
        oe.Optimizer(oe.MultiTableEmbedding("sd3", 4, torch.float32, torch.int64, tables,
                                            oe.make_device_mem_store_options(str(tmp_path), 10, size_factor=3)), oe.SmartDecayAdam)


def test_load_variable_directory_written_by_the_reference():
    """The reference ships a saved model of its C++ API tests: a legacy variable directory (one folder per variable with
    the raw bytes in ``out`` and a text-proto ``meta``). ``flow.load`` must read it as it is (read-only, in place)."""
    import struct
    import oneflow as flow
    # the reference checkout sits beside this repository (or where ONEFLOW_REFERENCE_ROOT points)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("ONEFLOW_REFERENCE_ROOT", os.path.join(os.path.dirname(repo), "reference"))
    root = os.path.join(ref, "oneflow", "api", "cpp", "tests", "graph_test_model", "affine_with_parameter")
    if not os.path.isdir(os.path.join(root, "model.a")):
        pytest.skip("the reference tree is not mounted")
    sd = flow.load(root)
    assert set(sd) >= {"model.a", "model.b"}
    a = sd["model.a"]
    assert tuple(a.shape) == (3, 4) and a.dtype == flow.float32
    raw = open(os.path.join(root, "model.a", "out"), "rb").read()
    assert np.allclose(a.numpy().reshape(-1), np.array(struct.unpack("<12f", raw), dtype=np.float32))
    one = flow.load(os.path.join(root, "model.a"))          # a single tensor directory loads as the tensor
    assert np.array_equal(np.asarray(one.numpy()), a.numpy())


def test_doctor_entry_point():
    p = subprocess.run([sys.executable, "-m", "oneflow", "--doctor"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       cwd=ROOT, timeout=300)
    assert p.returncode == 0 and "version:" in p.stdout and "native kernel library" in p.stdout, p.stdout


def test_sdpa_grouped_heads_unequal_lengths_on_cpu():
    """The CPU path of flow.nn.functional.scaled_dot_product_attention: grouped key/value heads are repeated, and with Sq != Sk
    the causal diagonal sits at the bottom-right corner (query row r sees key columns <= r + Sk - Sq)."""
    import oneflow_b200 as flow
    from oneflow_b200.ops import kernels as K
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 4, 5, 8), torch.randn(2, 2, 7, 8), torch.randn(2, 2, 7, 8)
    y = flow.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    o, lse = K.fmha_reference(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), True, 1 / 8 ** 0.5)
    assert torch.allclose(y, o.transpose(1, 2), atol=1e-5)
    # more queries than keys: the first Sq - Sk rows see nothing and come back as zeros with zero gradient
    q2 = torch.randn(1, 2, 6, 8, requires_grad=True)
    k2, v2 = torch.randn(1, 2, 3, 8, requires_grad=True), torch.randn(1, 2, 3, 8)
    o2, lse2 = K.fmha_reference(q2.transpose(1, 2), k2.transpose(1, 2), v2.transpose(1, 2), True, 0.3)
    assert torch.equal(o2[0, :3], torch.zeros_like(o2[0, :3])) and torch.isinf(lse2[0, :, :3]).all()
    o2.sum().backward()
    assert torch.isfinite(q2.grad).all() and torch.isfinite(k2.grad).all() and q2.grad[0, :, :3].abs().sum() == 0


def test_profiler_key_averages_table_on_cpu():
    """flow.profiler.profile records ATen operators and record_function ranges; key_averages groups them (optionally by input
    shape) and prints the reference's columns."""
    import oneflow_b200 as flow
    x = torch.randn(32, 16)
    w = torch.randn(16, 16)
    with flow.profiler.profile(activities=[flow.profiler.ProfilerActivity.CPU], record_shapes=True) as prof:
        with flow.profiler.record_function("block"):
            for _ in range(3):
                y = torch.mm(x, w)
            z = torch.relu(y)
        torch.mm(z.t(), z)
    evs = prof.events()
    assert [e.name for e in evs][0] == "block" and evs[0].kind == "custom" and len(evs[0].children) >= 4
    avg = prof.key_averages()
    by_name = {e.name: e for e in avg}
    assert by_name["aten::mm"].count == 4 and by_name["aten::relu"].count == 1 and by_name["block"].count == 1
    assert by_name["aten::mm"].cpu_time_total > 0 and by_name["aten::mm"].cuda_time is None
    shaped = prof.key_averages(group_by_input_shape=True)
    mm = sorted((e.input_shapes, e.count) for e in shaped if e.name == "aten::mm")
    assert mm == [("[(16,32), (32,16)]", 1), ("[(32,16), (16,16)]", 3)]
    table = shaped.table()
    head = table.splitlines()[0]
    for col in ("Name", "CPU time total", "CPU time", "GPU time total", "GPU time", "Number of calls", "Input shapes"):
        assert col in head
    assert "Bandwidth" not in head
    with pytest.raises(AssertionError, match="only work with cuda"):
        flow.profiler.profile(activities=[flow.profiler.ProfilerActivity.CPU], record_bandwidth_for_cuda=True)
    with pytest.raises(RuntimeError, match="didn't finish"):
        flow.profiler.profile().key_averages()


def test_remat_evicts_under_a_budget_and_recomputes_for_backward():
    """flow.remat.scope: activations beyond the budget are evicted in forward (their storage is released), recomputed from
    their producers when backward needs them, and the gradients equal the ones of a run without a budget."""
    import oneflow_b200 as flow

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList([torch.nn.Linear(128, 128) for _ in range(8)])

        def forward(self, x):
            for l in self.layers:
                x = torch.tanh(l(x)) + x
            return x

    torch.manual_seed(0)
    m, x = Net(), torch.randn(256, 128)
    ref = m(x).pow(2).mean()
    ref.backward()
    g_ref = [p.grad.clone() for p in m.parameters()]
    for p in m.parameters():
        p.grad = None
    act = 256 * 128 * 4
    old = flow.remat.is_small_pieces_optimization_enabled()
    flow.remat.set_small_pieces_optimization(False)
    try:
        with flow.remat.scope(budget=12 * act) as r:          # forward alone would hold 8 layers x 3 tensors
            y = m(x)
            assert r.stats["forced_eviction_num"] > 0 and flow.remat.allocated_memory("cpu") <= 12 * act
            loss = y.pow(2).mean()
            loss.backward()
            assert r.stats["recomputation_num"] > 0
        st = flow.remat.stats()
        g_remat = [q.grad.clone() for q in m.parameters()]
        for q in m.parameters():
            q.grad = None
        with flow.remat.scope() as free:                      # no budget: nothing is evicted, everything is held
            m(x).pow(2).mean().backward()
        assert free.stats["forced_eviction_num"] == 0
        # a recomputation chain holds its inputs while it runs, so the peak may pass the budget, but stays below holding all
        assert st["peak_bytes"] < free.stats["peak_bytes"]
        assert torch.equal(loss.detach(), ref.detach())
        for a, b in zip(g_ref, g_remat):
            assert torch.equal(a, b)
        assert torch.isfinite(y).all()                        # the result tensor is in memory after the scope
        # explicit eviction and the in-memory query
        with flow.remat.scope() as r:
            a = torch.randn(64, 64)
            b = a @ a
            c = torch.relu(b)
            assert flow.remat.is_in_memory(b)
            flow.remat.evict(b)
            assert not flow.remat.is_in_memory(b) and b.untyped_storage().nbytes() == 0
            d = b + 1                                         # touching it brings it back
            assert flow.remat.is_in_memory(b) and torch.equal(d, a @ a + 1)
            with pytest.raises(RuntimeError, match="cannot be evicted"):
                flow.remat.evict(a)                           # an input has no producer
            flow.remat.disable_eviction(c)
            with pytest.raises(RuntimeError, match="cannot be evicted"):
                flow.remat.evict(c)
            assert flow.remat.stats()["eager_eviction_num"] == 1 and flow.remat.stats()["recomputation_num"] == 1
    finally:
        flow.remat.set_small_pieces_optimization(old)
    assert flow.remat.parse_size("1.5GB") == int(1.5 * 2 ** 30)


def test_autoprof_profiles_a_script_into_a_csv(tmp_path):
    """python -m oneflow.autoprof script.py: one CSV row per operator and input shape, a summary table on stdout; the alias
    package keeps real packages as packages so that ``python -m oneflow.<package>`` finds their __main__."""
    script = tmp_path / "work.py"
    script.write_text("import oneflow as flow\nx = flow.randn(64, 128)\nw = flow.randn(128, 256)\n"
                      "for _ in range(3):\n    y = flow.nn.functional.gelu(flow.matmul(x, w))\nprint('ran', tuple(y.shape))\n")
    env = dict(os.environ, ONEFLOW_PROFILE_CSV=str(tmp_path / "ops"), PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-m", "oneflow.autoprof", str(script)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=300, cwd=str(tmp_path), env=env)
    assert p.returncode == 0 and "ran (64, 256)" in p.stdout and "aten::mm" in p.stdout, p.stdout[-3000:]
    import csv
    rows = list(csv.DictReader(open(str(tmp_path / "ops.csv"))))
    mm = [r for r in rows if r["op"] == "aten::mm"]
    assert len(mm) == 1 and mm[0]["count"] == "3" and "(64,128)" in mm[0]["input_shapes"].replace(" ", "")
    import oneflow as flow
    assert flow.support.env_var_util.parse_boolean_from_env("ONEFLOW_SURELY_UNSET_VARIABLE", True) is True
    os.environ["ONEFLOW_TEST_BOOL"] = "off"
    assert flow.support.env_var_util.parse_boolean_from_env("ONEFLOW_TEST_BOOL", True) is False
    os.environ.pop("ONEFLOW_TEST_BOOL")
    t = torch.arange(6.0)
    assert torch.equal(flow.utils.dlpack.from_dlpack(flow.utils.dlpack.to_dlpack(t)), t)


def test_model_fit_runs_training_validation_checkpoints_and_callbacks(tmp_path):
    import numpy as np
    import oneflow as flow

    class Data(flow.model.NumpyDataModule):
        def forward(self, step_idx=0, optimizer_idx=0):
            rng = np.random.default_rng(step_idx % 4)
            x = rng.standard_normal((16, 8)).astype(np.float32)
            return x, (x.sum(1, keepdims=True) > 0).astype(np.float32)

    class Net(flow.model.Model):
        def __init__(self):
            super().__init__()
            self.fc = flow.nn.Linear(8, 1)

        def forward(self, x):
            return self.fc(x)

        def training_step(self, batch, optimizer_idx=0):
            x, y = batch
            return flow.nn.functional.binary_cross_entropy_with_logits(self(x), y), "extra"

        def validation_step(self, batch):
            x, y = batch
            return ((self(x) > 0).float() == y).float().mean()

        def configure_optimizers(self):
            return flow.optim.SGD(self.parameters(), lr=0.5)

    class Log(flow.model.Callback):
        def __init__(self):
            self.train, self.val = [], []

        def on_training_step_end(self, outputs, step_idx=0, optimizer_idx=0):
            self.train.append(float(outputs[0].detach()))

        def on_validation_step_end(self, outputs, step_idx=0):
            self.val.append((step_idx, float(outputs)))

    flow.manual_seed(0)
    net, log = Net(), Log()
    train, val, ckpt = flow.model.TrainingConfig(), flow.model.ValidationConfig(), flow.model.CheckpointConfig()
    train.config_data(Data())
    val.config_data(Data())
    val.config_step_interval(10)
    ckpt.config_save(str(tmp_path), step_interval=20)
    net.fit(training_config=train, validation_config=val, checkpoint_config=ckpt, callbacks=log, max_steps=40)
    assert len(log.train) == 40 and log.train[-1] < 0.6 * log.train[0]
    assert [s for s, _ in log.val] == [9, 19, 29, 39] and log.val[-1][1] > 0.85
    assert sorted(os.listdir(str(tmp_path))) == ["step_20", "step_40"]
    again, load = Net(), flow.model.CheckpointConfig()
    load.config_load(str(tmp_path / "step_40"))
    again.fit(checkpoint_config=load, max_steps=0)
    assert torch.equal(again.fc.weight, net.fc.weight)
    with pytest.raises(ValueError, match="DataModule"):
        bad = flow.model.TrainingConfig()
        Net().fit(training_config=bad, max_steps=1)

    class NoStep(flow.model.Model):
        def configure_optimizers(self):
            return None

    with pytest.raises(NotImplementedError, match="training_step"):
        NoStep().fit(training_config=train, max_steps=1)


def test_load_mnist_reads_local_idx_files(tmp_path):
    import gzip
    import struct
    import numpy as np
    import oneflow as flow
    rng = np.random.default_rng(0)
    for stem, n in (("train", 250), ("t10k", 120)):
        images = rng.integers(0, 256, (n, 28, 28), dtype=np.uint8)
        labels = rng.integers(0, 10, (n,), dtype=np.uint8)
        with gzip.open(str(tmp_path / f"{stem}-images-idx3-ubyte.gz"), "wb") as f:
            f.write(struct.pack(">HBBIII", 0, 8, 3, n, 28, 28) + images.tobytes())
        with open(str(tmp_path / f"{stem}-labels-idx1-ubyte"), "wb") as f:
            f.write(struct.pack(">HBBI", 0, 8, 1, n) + labels.tobytes())
    (xtr, ytr), (xte, yte) = flow.data.load_mnist(100, 50, data_dir=str(tmp_path))
    assert len(xtr) == 2 and xtr[0].shape == (100, 1, 28, 28) and xtr[0].dtype == np.float32 and 0.0 <= xtr[0].min() and xtr[0].max() <= 1.0
    assert len(yte) == 2 and yte[0].shape == (50,) and yte[0].dtype == np.int32
    with pytest.raises(FileNotFoundError, match="nothing is downloaded"):
        flow.data.load_mnist(data_dir=str(tmp_path / "empty"))
