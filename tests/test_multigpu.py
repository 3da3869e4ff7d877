"""Multi-GPU checks (one process per GPU): in-kernel collectives over symmetric memory, the GEMM fused with
reduce-scatter / all-gather, and tensor / pipeline parallel GPT training."""
import pytest
import torch

from test_parallel_cpu import run_case

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _n(want):
    have = torch.cuda.device_count()
    if have < want:
        pytest.skip(f"needs {want} GPUs")
    return want


def test_collectives_2gpu():
    run_case("collectives", _n(2), "cuda")


@pytest.mark.parametrize("n", [2, 4])
def test_fused_gemm_collectives(n):
    run_case("fused_gemm", _n(n), "cuda")


def test_tensor_parallel_matches_unsharded_2gpu():
    run_case("tp_matches_single", _n(2), "cuda")


@pytest.mark.parametrize("case,n", [("gpt_2_1_1", 2), ("gpt_1_2_1", 2), ("gpt_1_1_2", 2), ("gpt_2_2_1", 4)])
def test_gpt_parallel_training_gpu(case, n):
    run_case(case, _n(n), "cuda")


@pytest.mark.parametrize("n", [2, 4])
def test_embedding_engine_matches_single_rank(n):
    run_case("embedding_engine", _n(n), "cuda")


def test_dlrm_two_gpus_match_one_gpu():
    from test_parallel_cpu import _dlrm_losses
    _n(2)
    one = _dlrm_losses(run_case("dlrm_parallel", 1, "cuda"))
    two = _dlrm_losses(run_case("dlrm_parallel", 2, "cuda"))
    for a, b in zip(one, two):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (one, two)


def test_resnet_data_parallel_2gpu():
    run_case("resnet_parallel", _n(2), "cuda")


def test_bert_tensor_parallel_2gpu():
    run_case("bert_tp", _n(2), "cuda")
