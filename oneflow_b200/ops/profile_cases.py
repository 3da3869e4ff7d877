"""Small stand-alone cases of the hot kernels for profiling one kernel at a time:

    python -m oneflow_b200.ops.profile_cases <case> [--reps N]

Every case allocates a few hundred MB at most (inputs larger than the 126 MB L2 where DRAM figures matter), runs
the kernel ``reps`` times after two warm-up calls and prints the CUDA-event time per call.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import gemm as G
from . import kernels as K


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def case_gemm_2cta():
    a, b = _bf(8192, 4096), _bf(8192, 4096, scale=0.02)
    return (lambda: G.gemm(a, b)), 2 * 8192 * 8192 * 4096, 0


def case_gemm_bias_relu():
    a, b, bias = _bf(55296, 480), _bf(1024, 480, scale=0.05), _bf(1024)
    return (lambda: G.gemm(a, b, bias=bias, act="relu")), 2 * 55296 * 1024 * 480, (55296 * 480 + 55296 * 1024) * 2


def case_gemm_wgrad_splitk():
    dy, x = _bf(55296, 1024), _bf(55296, 512)
    out = torch.empty(1024, 512, dtype=torch.float32, device="cuda")
    return (lambda: G.gemm(dy, x, a_layout="km", b_layout="kn", out=out, out_dtype=torch.float32)), 2 * 55296 * 1024 * 512, 0


def _qkv():
    return [_bf(4, 2048, 32, 128, scale=0.5) for _ in range(3)]


def case_fmha_fwd():
    q, k, v = _qkv()
    fl = 4 * 4 * 32 * 2048 * 2048 * 128 / 2
    return (lambda: K.fmha_fwd(q, k, v, causal=True)), fl, 0


def case_fmha_bwd():
    q, k, v = _qkv()
    o, lse = K.fmha_fwd(q, k, v, causal=True)
    d_o = torch.randn_like(o)
    fl = 10 * 4 * 32 * 2048 * 2048 * 128 / 2
    return (lambda: K.fmha_bwd(q, k, v, o, d_o, lse, causal=True)), fl, 0


def _single_rank_tp(tokens, hidden):
    """A one-rank tensor-parallel context: the fused GEMM+collective kernels run with their exchange logic compiled in but
    nothing to exchange, which isolates their main loop and epilogue for a single-GPU capture."""
    import torch.distributed as dist
    from ..parallel.tensor_parallel import TPContext
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29655", rank=0, world_size=1, device_id=dev)
    return TPContext(None, [0], dev, max_tokens=tokens, max_cols=hidden, hidden=hidden)


def case_gemm_rs_single_rank():
    tp = _single_rank_tp(8192, 4096)
    a, w = _bf(8192, 4096), _bf(4096, 4096, scale=0.02)
    return (lambda: tp.gemm_rs(a, w)), 2 * 8192 * 4096 * 4096, 0


def case_ag_gemm_single_rank():
    tp = _single_rank_tp(8192, 4096)
    x, w = _bf(8192, 4096), _bf(4096, 4096, scale=0.02)
    return (lambda: tp.ag_gemm(x, w)), 2 * 8192 * 4096 * 4096, 0


def _conv_case(mode):
    from . import conv as C
    n, h, w, cin, cout = 64, 56, 56, 64, 64
    x, wt, dy = _bf(n, h, w, cin), _bf(cout, 3, 3, cin, scale=0.05), _bf(n, h, w, cout)
    fl = 2 * n * h * w * 9 * cin * cout
    by = (n * h * w * (cin + cout)) * 2
    if mode == "fprop":
        return (lambda: C.conv_fprop(x, wt)), fl, by
    if mode == "dgrad":
        return (lambda: C.conv_dgrad(dy, wt)), fl, by
    return (lambda: C.conv_wgrad(x, dy, (3, 3))), fl, by


def case_conv_fprop():
    return _conv_case("fprop")


def case_conv_dgrad():
    return _conv_case("dgrad")


def case_conv_wgrad():
    return _conv_case("wgrad")


def _interaction_inputs():
    b = 55296
    return _bf(b, 128, scale=0.5), _bf(b, 26, 128, scale=0.5)


def case_interaction_fwd():
    dense, sparse = _interaction_inputs()
    by = (dense.numel() + sparse.numel() + dense.shape[0] * 480) * 2
    return (lambda: K.interaction_fwd(dense, sparse, False, 480)), 2 * dense.shape[0] * 351 * 128, by


def case_interaction_bwd():
    dense, sparse = _interaction_inputs()
    dout = _bf(dense.shape[0], 480, scale=0.1)
    by = (2 * dense.numel() + 2 * sparse.numel() + dout.numel()) * 2
    return (lambda: K.interaction_bwd(dense, sparse, dout, False)), 4 * dense.shape[0] * 351 * 128, by


def case_embedding_step():
    from ..models import dlrm as M
    from ..one_embedding.native import NativeEmbeddingEngine
    cfg = M.DLRMConfig()
    inits = [{"type": "uniform", "low": -0.01, "high": 0.01}] * 26
    eng = NativeEmbeddingEngine("cuda", 55296 * 26, 128, 128, inits, 1 << 22, seed=1)
    ids = M.make_batch(cfg, 55296, seed=3)[1].cuda()
    grad = _bf(55296, 26, 128, scale=0.01)
    hyper = {"lr": 0.05}

    def step():
        eng.forward(ids)
        eng.backward(grad, "sgd", hyper, 1)
    return step, 0, 55296 * 26 * 128 * 2 * 2


def case_batchnorm_relu():
    from . import cnn as N
    x = _bf(256, 56, 56, 64)
    gamma, beta = torch.ones(64, device="cuda"), torch.zeros(64, device="cuda")
    return (lambda: N.bn_train_fwd(x, gamma, beta, None, True)), 0, 3 * x.numel() * 2


def _ln_inputs():
    rows, cols = 32768, 4096         # 256 MiB per tensor: every pass streams from HBM
    return _bf(rows, cols), torch.ones(cols, device="cuda", dtype=torch.bfloat16), torch.zeros(cols, device="cuda", dtype=torch.bfloat16)


def case_layer_norm_fwd():
    x, g, b = _ln_inputs()
    return (lambda: K.layer_norm_fwd(x, g, b)), 0, 2 * x.numel() * 2


def case_layer_norm_bwd():
    x, g, b = _ln_inputs()
    y, mean, rstd = K.layer_norm_fwd(x, g, b)
    dy = _bf(*x.shape, scale=0.1)
    del y
    return (lambda: K.layer_norm_bwd(dy, x, g, mean, rstd)), 0, 3 * x.numel() * 2


def case_adamw():
    n = 64 << 20
    g = torch.randn(n, device="cuda")
    w, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    c = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    return (lambda: K.multi_tensor_adamw([g], [w], [c], [m], [v], lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1)), 0, n * 30


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    torch.manual_seed(0)
    fn, flops, nbytes = CASES[args.case]()
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.reps
    msg = f"{args.case}: {ms * 1e3:.1f} us per call"
    if flops:
        msg += f", {flops / ms / 1e9:.0f} TFLOP/s"
    if nbytes:
        msg += f", {nbytes / ms / 1e6:.0f} GB/s (algorithmic bytes)"
    print(msg)


if __name__ == "__main__":
    main()
