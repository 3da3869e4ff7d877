"""Micro-benchmarks of the native kernels with roofline fractions.

    python -m oneflow_b200.ops.bench_kernels gemm --m 8192 --n 4096 --k 4096 [--layout mk,nk] [--iters 20]
    python -m oneflow_b200.ops.bench_kernels fmha --batch 4 --seq 2048 --heads 32 --dim 128 --causal
    python -m oneflow_b200.ops.bench_kernels layer_norm --rows 8192 --cols 4096
    python -m oneflow_b200.ops.bench_kernels adamw --numel 268435456
    python -m oneflow_b200.ops.bench_kernels all

Timing: CUDA events on the launching stream after 3 warm-up launches; operands are cycled through a set
larger than the 126 MB L2 so that every timed launch reads from HBM. The denominators are the measured
copy bandwidth / cuBLAS bf16 throughput in MEASURED_PEAKS.json at the repository root when present
(fallback 6650 GB/s and 1590 TFLOP/s). One JSON line per kernel.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import gemm as G
from . import kernels as K

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def time_ms(fn, iters, warmup=3):
    for _ in range(warmup):
        fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _copies(nbytes_per_set):
    """How many operand sets to rotate through so that the working set exceeds L2 comfortably."""
    return max(2, math.ceil((256 << 20) / max(nbytes_per_set, 1)))


def bench_gemm(m, n, k, layout="mk,nk", iters=20, bn=0, bias=False, act=0, out_f32=False, accumulate=False):
    al, bl = layout.split(",")
    dev, dt = "cuda", torch.bfloat16
    nset = min(_copies((m * k + n * k + m * n) * 2), 8)
    As = [torch.randn((m, k) if al == "mk" else (k, m), device=dev, dtype=dt) for _ in range(nset)]
    Bs = [torch.randn((n, k) if bl == "nk" else (k, n), device=dev, dtype=dt) for _ in range(nset)]
    odt = torch.float32 if out_f32 else dt
    outs = [torch.zeros(m, n, device=dev, dtype=odt) for _ in range(nset if accumulate else 1)]   # accumulation reads the output too
    b = torch.randn(n, device=dev, dtype=dt) if bias else None
    ms = time_ms(lambda i: G.gemm(As[i % nset], Bs[i % nset], a_layout=al, b_layout=bl, out=outs[i % len(outs)], out_dtype=odt, bn=bn, bias=b,
                                  act=act, accumulate=accumulate), iters)
    tf = 2.0 * m * n * k / ms / 1e9
    pk = peaks()
    return {"kernel": "gemm_bf16_tcgen05", "m": m, "n": n, "k": k, "layout": layout, "bn": bn, "out": "f32" if out_f32 else "bf16",
            "accumulate": bool(accumulate), "ms": ms, "tflops": tf,
            "frac_of_" + pk["source"] + "_cublas_burst": tf / pk["bf16_tflops"]}


def bench_fmha(batch, seq, heads, dim, causal, iters=10):
    qkv = [torch.randn(batch, seq, 3, heads, dim, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    outs = {}

    def fwd(i):
        t = qkv[i % 4]
        outs["o"], outs["lse"] = K.fmha_fwd(t[:, :, 0], t[:, :, 1], t[:, :, 2], causal=causal)
    ms_f = time_ms(fwd, iters)
    d_o = torch.randn_like(outs["o"])

    def bwd(i):
        t = qkv[0]
        K.fmha_bwd(t[:, :, 0], t[:, :, 1], t[:, :, 2], outs["o"], d_o, outs["lse"], causal=causal)
    fwd(0)
    ms_b = time_ms(bwd, iters)
    fl = 4.0 * batch * heads * seq * seq * dim * (0.5 if causal else 1.0)
    pk = peaks()
    res = {"kernel": "fmha_fwd/bwd", "batch": batch, "seq": seq, "heads": heads, "dim": dim, "causal": causal,
           "fwd_ms": ms_f, "fwd_tflops": fl / ms_f / 1e9, "bwd_ms": ms_b, "bwd_tflops": 2.5 * fl / ms_b / 1e9,
           "fwd_frac_of_" + pk["source"] + "_cublas_burst": fl / ms_f / 1e9 / pk["bf16_tflops"]}
    # the library kernel on the same box, same inputs, same timing loop (right after ours, so the clocks are comparable)
    try:
        from flash_attn import flash_attn_func
    except Exception:
        return res

    def fa_fwd(i):
        t = qkv[i % 4]
        return flash_attn_func(t[:, :, 0], t[:, :, 1], t[:, :, 2], causal=causal)
    res["flash_attn_fwd_ms"] = time_ms(fa_fwd, iters)
    leaf = qkv[0].clone().requires_grad_()
    o = flash_attn_func(leaf[:, :, 0], leaf[:, :, 1], leaf[:, :, 2], causal=causal)

    def fa_bwd(i):
        leaf.grad = None
        o.backward(d_o, retain_graph=True)
    res["flash_attn_bwd_ms"] = time_ms(fa_bwd, iters)
    return res


def bench_layer_norm(rows, cols, iters=20):
    nset = _copies(rows * cols * 2)
    xs = [torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(nset)]
    g = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(cols, device="cuda", dtype=torch.bfloat16)
    st = {}

    def fwd(i):
        st["y"], st["m"], st["r"] = K.layer_norm_fwd(xs[i % nset], g, b)
    ms_f = time_ms(fwd, iters)
    dy = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    ms_b = time_ms(lambda i: K.layer_norm_bwd(dy, xs[i % nset], g, st["m"], st["r"]), iters)
    pk = peaks()
    gb_f = rows * cols * 4 / 1e9
    gb_b = rows * cols * 6 / 1e9
    return {"kernel": "layer_norm", "rows": rows, "cols": cols, "fwd_ms": ms_f, "fwd_gbs": gb_f / ms_f * 1e3,
            "fwd_frac_of_" + pk["source"] + "_hbm": gb_f / ms_f * 1e3 / pk["hbm_gbs"], "bwd_ms": ms_b, "bwd_gbs": gb_b / ms_b * 1e3,
            "bwd_frac_of_" + pk["source"] + "_hbm": gb_b / ms_b * 1e3 / pk["hbm_gbs"]}


def bench_adamw(numel, iters=10):
    w = torch.randn(numel, device="cuda")
    g = torch.randn(numel, device="cuda")
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    c = torch.empty(numel, device="cuda", dtype=torch.bfloat16)
    ms = time_ms(lambda i: K.multi_tensor_adamw([g], [w], [c], [m], [v], lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                               weight_decay=0.1, step=i + 1), iters)
    gb = numel * (4 * 4 + 3 * 4 + 2) / 1e9   # read g,w,m,v ; write w,m,v,bf16 copy
    pk = peaks()
    return {"kernel": "multi_tensor_adamw", "numel": numel, "ms": ms, "gbs": gb / ms * 1e3,
            "frac_of_" + pk["source"] + "_hbm": gb / ms * 1e3 / pk["hbm_gbs"]}


def bench_xent(rows, vocab, iters=10):
    nset = _copies(rows * vocab * 2)
    xs = [torch.randn(rows, vocab, device="cuda", dtype=torch.bfloat16) for _ in range(min(nset, 3))]
    lab = torch.randint(0, vocab, (rows,), device="cuda")

    def run(i):
        x = xs[i % len(xs)]
        st = K.xent_stats(x, lab)
        K.xent_grad(x, lab, st, inplace=True)
    ms = time_ms(run, iters)
    gb = rows * vocab * 2 * 4 / 1e9  # two reads for the statistics pass, read + write for the gradient pass
    pk = peaks()
    return {"kernel": "softmax_xent stats+grad", "rows": rows, "vocab": vocab, "ms": ms, "gbs": gb / ms * 1e3,
            "frac_of_" + pk["source"] + "_hbm": gb / ms * 1e3 / pk["hbm_gbs"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "fmha", "layer_norm", "adamw", "xent", "all"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="mk,nk")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--out-f32", action="store_true", help="gemm: fp32 output (weight-gradient form)")
    ap.add_argument("--accumulate", action="store_true", help="gemm: C += A B (read-add-write epilogue)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--vocab", type=int, default=50304)
    a = ap.parse_args()
    out = []
    if a.kernel in ("gemm",):
        out.append(bench_gemm(a.m, a.n, a.k, a.layout, a.iters, a.bn, out_f32=a.out_f32, accumulate=a.accumulate))
    if a.kernel in ("fmha",):
        out.append(bench_fmha(a.batch, a.seq, a.heads, a.dim, a.causal, a.iters))
    if a.kernel in ("layer_norm",):
        out.append(bench_layer_norm(a.rows, a.cols, a.iters))
    if a.kernel in ("adamw",):
        out.append(bench_adamw(a.numel, a.iters))
    if a.kernel in ("xent",):
        out.append(bench_xent(a.rows, a.vocab, a.iters))
    if a.kernel == "all":
        for (m, n, k, lay) in [(8192, 12288, 4096, "mk,nk"), (8192, 4096, 4096, "mk,nk"), (8192, 16384, 4096, "mk,nk"),
                               (8192, 4096, 16384, "mk,nk"), (8192, 4096, 16384, "mk,kn"), (4096, 16384, 8192, "km,kn"),
                               (8192, 50304, 4096, "mk,nk"), (8192, 8192, 8192, "mk,nk")]:
            out.append(bench_gemm(m, n, k, lay, 10))
        out.append(bench_fmha(4, 2048, 32, 128, True))
        out.append(bench_fmha(32, 512, 16, 64, False))
        out.append(bench_layer_norm(8192, 4096))
        out.append(bench_layer_norm(16384, 1024))
        out.append(bench_adamw(1 << 28))
        out.append(bench_xent(8192, 50304))
    for o in out:
        print(json.dumps(o))


if __name__ == "__main__":
    main()
