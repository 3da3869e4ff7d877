"""The flow-API GPT (flow.nn modules, global tensors, nn.Graph with set_stage and gradient accumulation, flow.optim.AdamW)
must follow the loss curve of a plain PyTorch statement of the same network, for every parallel layout. CPU ranks run
over gloo; the GPU cases run one process per GPU with the fused tensor-parallel kernels and keep their output in
``tests/logs`` when ``OFB_KEEP_TEST_LOGS`` is set."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_PORT = [29900]


def run(tp, pp, dp, device, timeout=900, extra_env=None):
    _PORT[0] += 1
    n = tp * pp * dp
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(_PORT[0]), os.path.join(ROOT, "tests", "gpt_flow_worker.py"), str(tp), str(pp), str(dp), device]
    env = dict(os.environ, OMP_NUM_THREADS="2", MASTER_ADDR="127.0.0.1", OFB_TEST_DUMP_AFTER=str(timeout - 60), **(extra_env or {}))
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, env=env, cwd=ROOT)
    keep = os.environ.get("OFB_KEEP_TEST_LOGS")
    if keep:
        os.makedirs(keep, exist_ok=True)
        with open(os.path.join(keep, f"gpt_flow_tp{tp}_pp{pp}_dp{dp}_{device}.log"), "w") as f:
            f.write(p.stdout)
    assert p.returncode == 0 and f"GPT FLOW tp{tp} pp{pp} dp{dp} {device} OK" in p.stdout, p.stdout[-4000:]


@pytest.mark.parametrize("tp,pp,dp", [(1, 1, 1), (2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 1)])
def test_gpt_flow_graph_matches_pytorch_cpu(tp, pp, dp):
    run(tp, pp, dp, "cpu")


@pytest.mark.gpu
def test_gpt_flow_graph_matches_pytorch_one_gpu():
    run(1, 1, 1, "cuda")


@pytest.mark.gpu
def test_gpt_flow_graph_with_captured_micro_batch_one_gpu():
    """``config.enable_cuda_graph``: the forward + backward of a micro-batch is captured once and replayed; the loss curve
    must be the one of the eager run (and of the PyTorch statement)."""
    run(1, 1, 1, "cuda", extra_env={"OFB_TEST_CUDA_GRAPH": "1"})


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("tp,pp,dp", [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 1), (4, 1, 1), (2, 1, 2)])
def test_gpt_flow_graph_matches_pytorch_multi_gpu(tp, pp, dp):
    if torch.cuda.device_count() < tp * pp * dp:
        pytest.skip(f"needs {tp * pp * dp} GPUs")
    run(tp, pp, dp, "cuda")
