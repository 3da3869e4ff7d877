"""Multi-process (gloo, CPU) checks of tensor / pipeline / data parallel training logic."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_PORT = [29620]


def run_case(case, nproc, dev="cpu", timeout=600):
    _PORT[0] += 1
    env = dict(os.environ, OMP_NUM_THREADS="2", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_PORT[0]), os.path.join(ROOT, "tests", "mp_worker.py"),
           case, dev]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert p.returncode == 0 and f"CASE {case} OK" in p.stdout, p.stdout[-4000:]
    return p.stdout


def test_tensor_parallel_matches_unsharded_cpu():
    run_case("tp_matches_single", 2)


@pytest.mark.parametrize("case,n", [("gpt_2_1_1", 2), ("gpt_1_2_1", 2), ("gpt_1_1_2", 2), ("gpt_2_2_1", 4)])
def test_gpt_parallel_training_cpu(case, n):
    run_case(case, n)


def _dlrm_losses(out):
    line = [l for l in out.splitlines() if l.startswith("DLRM_LOSSES ")][-1]
    return [float(v) for v in line.split()[1].split(",")]


def test_dlrm_two_ranks_match_one_rank_cpu():
    one = _dlrm_losses(run_case("dlrm_parallel", 1))
    two = _dlrm_losses(run_case("dlrm_parallel", 2))
    assert len(one) == len(two) == 4
    for a, b in zip(one, two):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (one, two)


def test_resnet_data_parallel_cpu():
    run_case("resnet_parallel", 2)


def test_sync_batchnorm_and_partial_fc_cpu():
    run_case("sync_bn_partial_fc", 2)


def test_auto_parallel_chain():
    from oneflow_b200.framework import auto_parallel as ap
    # a transformer MLP block with many tokens: the classic answer is column-parallel then row-parallel
    big = [ap.LinearSpec("w1", 4096, 16384, tokens=8192), ap.LinearSpec("w2", 16384, 4096, tokens=8192)]
    choices = ap.solve_chain(big, world=4, mem_bytes_per_rank=1.2e9)
    assert [c.kind for c in choices] == ["column", "row"], [c.kind for c in choices]
    # small weights, huge batch: plain data parallelism is cheapest
    small = [ap.LinearSpec("a", 256, 256, tokens=1 << 20), ap.LinearSpec("b", 256, 256, tokens=1 << 20)]
    assert [c.kind for c in ap.solve_chain(small, world=8)] == ["data", "data"]
    # one rank: nothing to decide, no communication
    assert all(c.kind == "data" for c in ap.solve_chain(big, world=1))


def test_bert_tensor_parallel_cpu():
    run_case("bert_tp", 2)


def test_sbp_graph_solver_is_exact_and_plans_modules():
    """The SBP-graph solver (node / edge elimination + node merging) finds the brute-force optimum on random graphs,
    including ones where every node has three or more neighbours; plan_module picks Megatron-style column -> row parallel
    layers when the activations are small against the weights and data parallel when they are large."""
    import itertools
    import random

    import torch
    from oneflow_b200.framework import auto_parallel as ap
    random.seed(0)
    merged = 0
    for trial in range(200):
        n = random.randint(2, 7)
        g = ap.SbpGraph()
        k = [random.randint(1, 3) for _ in range(n)]
        for i in range(n):
            g.add_node(i, [random.random() for _ in range(k[i])])
        dense = trial % 4 == 0
        for i in range(n):
            for j in range(i + 1, n):
                if dense or random.random() < 0.5:
                    g.add_edge(i, j, [[random.random() for _ in range(k[j])] for _ in range(k[i])])
        merged += dense and n >= 4
        choice, total = g.solve()
        best = min(g.cost_of(dict(enumerate(c))) for c in itertools.product(*[range(x) for x in k]))
        assert abs(total - best) < 1e-9 and abs(g.cost_of(choice) - best) < 1e-9
    assert merged > 10          # complete graphs on >= 4 nodes need the merging step

    class Block(torch.nn.Module):
        def __init__(self, h=512):
            super().__init__()
            self.ln, self.fc1, self.fc2 = torch.nn.LayerNorm(h), torch.nn.Linear(h, 4 * h), torch.nn.Linear(4 * h, h)

        def forward(self, x):
            return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.ln(x))))

    m = Block()
    small, _ = ap.plan_module(m, torch.randn(8, 512), 4)
    assert (small["fc1"].kind, small["gelu"].kind, small["fc2"].kind) == ("column", "split_last", "row")
    assert small.param_sbp["fc1.weight"] == ap._sbp.split(0) and small.param_sbp["fc2.weight"] == ap._sbp.split(1)
    large, _ = ap.plan_module(m, torch.randn(65536, 512), 4)
    assert (large["fc1"].kind, large["fc2"].kind) == ("data", "data")
