"""Micro-benchmark of the fused GEMM+collective kernels and of raw NVLink accesses, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m oneflow_b200.ops.bench_gemm_comm [--tokens 8192] [--hidden 4096] [--ffn 16384] [--no-p2p]

For the four tensor-parallel products of a GPT layer (attention output and MLP down projection as GEMM -> reduce-scatter,
QKV and MLP up projection as all-gather -> GEMM) it prints the CUDA-event time of the fused kernel and of the plain GEMM of
the same shape (max over ranks, microseconds), and, per access pattern, the bandwidth of SM loads / stores to the next
rank's symmetric arena (GB/s). ``OFB_GEMM_COMM_2CTA=0`` selects the one-SM kernels."""
import argparse
import ctypes
import json
import os
from ctypes import c_int, c_longlong

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=16384)
    ap.add_argument("--no-p2p", action="store_true")
    ap.add_argument("--collectives", action="store_true",
                    help="also time the device collectives (all-reduce, reduce-scatter, all-gather, all-to-all, NVLS all-reduce) "
                         "against NCCL's at 8 / 64 MB and print bus bandwidths")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    from oneflow_b200.comm.symmetric import SymmetricArena
    from oneflow_b200.ops import _native
    from oneflow_b200.ops import gemm as G
    from oneflow_b200.parallel.tensor_parallel import TPContext
    T, H, F, n = args.tokens, args.hidden, args.ffn, world
    tp = TPContext(None, list(range(world)), dev, max_tokens=T, max_cols=H, hidden=H)
    bf = torch.bfloat16

    def timeit(fn, iters=20, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    res = {}
    x_sh = torch.randn(T // n, H, device=dev, dtype=bf)
    x_full = torch.randn(T, H, device=dev, dtype=bf)
    for name, (N, K) in {"attn_out": (H, H // n), "mlp_down": (H, F // n)}.items():
        a = torch.randn(T, K, device=dev, dtype=bf)
        w = torch.randn(N, K, device=dev, dtype=bf) * 0.02
        res[f"gemm_rs_{name}"] = timeit(lambda: tp.gemm_rs(a, w))
        res[f"plain_{name}"] = timeit(lambda: G.gemm(a, w))
    for name, N in {"qkv": 3 * H // n, "mlp_up": F // n}.items():
        w = torch.randn(N, H, device=dev, dtype=bf) * 0.02
        res[f"ag_gemm_{name}"] = timeit(lambda: tp.ag_gemm(x_sh, w))
        res[f"plain_{name}"] = timeit(lambda: G.gemm(x_full, w))
    bw = {}
    if not args.no_p2p and world > 1:
        ar = SymmetricArena(None, list(range(world)), dev, 2 * (256 << 20) + (1 << 22))
        o_a, o_b = ar.region(256 << 20), ar.region(256 << 20)
        lib = _native.kernels()
        nbytes = 128 << 20
        for mode, nm in ((0, "pull_wide"), (1, "push_wide"), (2, "push_seg64"), (3, "push_seg256")):
            for ctas in (37, 148, 296):
                def f():
                    _native.check(lib.ofb_comm_p2p_bandwidth(ctypes.byref(ar.ctx), c_int((rank + 1) % world), c_int(mode), c_longlong(o_a),
                                                             c_longlong(o_b), c_longlong(nbytes), c_longlong(8192), c_int(ctas),
                                                             _native.stream_ptr()), "p2p_bandwidth")
                us = timeit(f, iters=10, warm=3)
                bw[f"{nm}_{ctas}ctas"] = round(nbytes / us / 1e3, 1)
    if rank == 0:
        print("GEMM_COMM_US", json.dumps({"ranks": world, "tokens": T, "hidden": H, "ffn": F, **{k: round(v, 1) for k, v in res.items()}}), flush=True)
        if bw:
            print("P2P_GBS", json.dumps({"ranks": world, **bw}), flush=True)
    coll = {}
    if args.collectives and world > 1:
        from oneflow_b200.comm.symmetric import DeviceCollectives, MultimemAllReduce
        arena2 = SymmetricArena(None, list(range(world)), dev, 4 * (64 << 20) + (1 << 22))
        dc = DeviceCollectives(arena2, io_bytes=64 << 20, ctas=128)
        mm = MultimemAllReduce(None, list(range(world)), dev, nbytes=64 << 20)
        for mb in (8, 64):
            nel = (mb << 20) // 2
            xfull = torch.randn(nel, device=dev, dtype=bf)
            xshard = torch.randn(nel // n, device=dev, dtype=bf)
            out_full = torch.empty_like(xfull)
            out_shard = torch.empty_like(xshard)
            nbytes = nel * 2
            # bus bandwidth as NCCL's tests define it: algorithm bytes x (2(n-1)/n for all-reduce, (n-1)/n for the others)
            f_ar, f_1 = 2.0 * (n - 1) / n, (n - 1.0) / n

            def gbs(us, f):
                return round(nbytes * f / us / 1e3, 1)
            coll[f"all_reduce_{mb}MB_ours"] = gbs(timeit(lambda: dc.all_reduce(xfull), 10, 3), f_ar)
            coll[f"all_reduce_{mb}MB_nccl"] = gbs(timeit(lambda: dist.all_reduce(xfull), 10, 3), f_ar)
            if mm.available:
                coll[f"all_reduce_{mb}MB_nvls"] = gbs(timeit(lambda: mm.all_reduce(xfull), 10, 3), f_ar)
            coll[f"reduce_scatter_{mb}MB_ours"] = gbs(timeit(lambda: dc.reduce_scatter(xfull.view(n, -1)), 10, 3), f_1)
            coll[f"reduce_scatter_{mb}MB_nccl"] = gbs(timeit(lambda: dist.reduce_scatter_tensor(out_shard, xfull), 10, 3), f_1)
            coll[f"all_gather_{mb}MB_ours"] = gbs(timeit(lambda: dc.all_gather(xshard.view(1, -1)), 10, 3), f_1)
            coll[f"all_gather_{mb}MB_nccl"] = gbs(timeit(lambda: dist.all_gather_into_tensor(out_full, xshard), 10, 3), f_1)
            rows = 4096
            cols = nel // rows
            # this rank's row shard of a [rows, cols / 64, 64] tensor, re-split along the middle axis
            xa = xfull.view(rows, cols // 64, 64)[:rows // n].contiguous()
            coll[f"all_to_all_{mb}MB_ours"] = gbs(timeit(lambda: dc.all_to_all(xa, 0, 1, (rows, cols // 64, 64)), 10, 3), f_1 / n)
            coll[f"all_to_all_{mb}MB_nccl"] = gbs(timeit(lambda: dist.all_to_all_single(out_full, xfull), 10, 3), f_1)
    status = _native.read_status()
    if rank == 0 and coll:
        print("COLLECTIVES_BUS_GBS", json.dumps({"ranks": world, **coll}))
    if rank == 0:
        print("KERNEL_STATUS", list(status))
    dist.barrier()


if __name__ == "__main__":
    main()
