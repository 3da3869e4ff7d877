"""Worker for the flow-API GPT tests: the model of models/gpt_flow.py (flow.nn + global tensors + nn.Graph with
set_stage) trained for a few steps on N ranks must reproduce the loss curve of a plain PyTorch statement of the same
network on one process. Usage:
    python -m oneflow.distributed.launch --nproc_per_node N tests/gpt_flow_worker.py <tp> <pp> <dp> <device> [steps]"""
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch

import oneflow as flow
from oneflow_b200.framework import global_tensor as GT
from oneflow_b200.models import gpt_flow as GF
from oneflow_b200.models.gpt import GPTConfig


def full(p):
    """The logical value of a parameter (gathered to every rank of its placement)."""
    g = GT.to_global(p.detach(), p.placement, (flow.sbp.broadcast,) * p.placement.ndim)
    return g._local.float().cpu()


def reference_curve(cfg, params, batches, n_micro, steps, lr, wd, clip):
    """fp32 PyTorch training of the same GPT from the same initial values: returns the loss of every micro-batch."""
    P = {k: v.clone().requires_grad_(True) for k, v in params.items()}
    decay = [v for k, v in P.items() if v.dim() >= 2]
    rest = [v for k, v in P.items() if v.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": wd}, {"params": rest, "weight_decay": 0.0}], lr=lr,
                            betas=(0.9, 0.95), eps=1e-8)
    H, heads, D = cfg.hidden, cfg.heads, cfg.head_dim
    F = torch.nn.functional

    def forward(tok):
        inp, lab = tok[:, :-1], tok[:, 1:]
        Bq, Sq = inp.shape
        x = P["embedding.wte"][inp.reshape(-1)] + P["embedding.wpe"][torch.arange(Bq * Sq) % Sq]
        for i in range(cfg.layers):
            p = f"layers.{i}."
            h = F.layer_norm(x, (H,), P[p + "ln1_w"], P[p + "ln1_b"], cfg.eps)
            qkv = h @ P[p + "wqkv"].reshape(3 * H, H).t() + P[p + "bqkv"].reshape(-1)
            q, k, v = (t.reshape(Bq, Sq, heads, D).transpose(1, 2) for t in qkv.reshape(Bq * Sq, 3, H).unbind(1))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=cfg.causal).transpose(1, 2).reshape(Bq * Sq, H)
            x = a @ P[p + "wo"].t() + P[p + "bo"] + x
            h = F.layer_norm(x, (H,), P[p + "ln2_w"], P[p + "ln2_b"], cfg.eps)
            m = F.gelu(h @ P[p + "w1"].t() + P[p + "b1"], approximate="tanh" if cfg.act == "gelu_tanh" else "none")
            x = m @ P[p + "w2"].t() + P[p + "b2"] + x
        h = F.layer_norm(x, (H,), P["head.lnf_w"], P["head.lnf_b"], cfg.eps)
        return F.cross_entropy(h @ P["head.lm_head"].t(), lab.reshape(-1))
    out = []
    for s in range(steps):
        opt.zero_grad()
        mb = batches[s].shape[0] // n_micro
        for m in range(n_micro):
            loss = forward(batches[s][m * mb:(m + 1) * mb])
            (loss / n_micro).backward()
            out.append(loss.item())
        if clip:
            torch.nn.utils.clip_grad_norm_(list(P.values()), clip)
        opt.step()
    return out


def main():
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("OFB_TEST_DUMP_AFTER", "600")), exit=True)
    tp, pp, dp, device = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    steps = int(sys.argv[5]) if len(sys.argv) > 5 else 3
    rank, world = flow.env.get_rank(), flow.env.get_world_size()
    assert world == tp * pp * dp
    cuda = device == "cuda"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    # sizes that let the fused tensor-parallel kernels run on CUDA: tokens per micro-batch a multiple of 128 * tp * dp
    cfg = GPTConfig(vocab_size=512, hidden=128, layers=2 * pp, heads=2 * max(tp, 1), ffn=512, seq_len=128) if cuda else \
        GPTConfig(vocab_size=64, hidden=32, layers=2 * pp, heads=2 * max(tp, 1), ffn=64, seq_len=16)
    if cuda:
        cfg.heads = max(2, tp)
        cfg.hidden = 64 * cfg.heads
    dtype = torch.bfloat16 if cuda else torch.float32
    n_micro, micro = 2, (4 * dp if cuda else 2 * dp)
    lr, wd, clip = 1e-3, 0.1, 1.0
    graph, model, lay = GF.build_gpt_graph(cfg, tp=tp, pp=pp, dp=dp, grad_acc=n_micro, device_type=device, lr=lr,
                                           weight_decay=wd, clip_grad=clip, zero_stage=1, seed=3, dtype=dtype)
    graph.config.enable_multi_tensor_update(True)
    captured = os.environ.get("OFB_TEST_CUDA_GRAPH") == "1"
    if captured:
        graph.config.enable_cuda_graph(True)      # micro-batches after the first call replay a captured CUDA graph
    params = {}
    for name, p in model.named_parameters():
        pl = p.placement
        # every rank takes part in the gather of every parameter's own placement; only members get values
        v = full(p) if pl.contains(rank) else None
        params[name] = v
    # collect the logical parameters on rank 0 (they live on different stages)
    gathered = [None] * world
    torch.distributed.all_gather_object(gathered, {k: v for k, v in params.items() if v is not None}) if world > 1 else None
    if world > 1:
        params = {}
        for d in gathered:
            params.update(d)
    g = torch.Generator().manual_seed(11)
    batches = [torch.randint(0, cfg.vocab_size, (n_micro * micro, cfg.seq_len + 1), generator=g)] * steps   # one batch, repeated
    dp_idx = rank // (pp * tp)
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    losses = []
    for s in range(steps):
        # micro-batch m of the reference = rows [m*micro, (m+1)*micro): this data-parallel slice holds its share of each
        per = micro // dp
        rows = torch.cat([batches[s][m * micro + dp_idx * per: m * micro + (dp_idx + 1) * per] for m in range(n_micro)])
        x, y = GF.make_inputs(lay, rows.to(dev))
        loss = graph(x, y)
        lg = GT.to_global(loss.detach().float(), flow.placement(device, list(range(world))), flow.sbp.broadcast)
        losses += [float(v) for v in lg._local.reshape(-1).cpu()]
    from oneflow_b200.ops import _native
    if cuda:
        assert _native.read_status() == (0, 0), _native.read_status(False)
    if rank == 0:
        ref = reference_curve(cfg, params, batches, n_micro, steps, lr, wd, clip)
        tol = 3e-2 if cuda else 2e-4
        assert len(ref) == len(losses)
        assert np.allclose(losses, ref, rtol=tol, atol=tol), (losses, ref)
        assert ref[-1] < ref[0]
        plan = graph._plan
        ops = [o["op"] for o in plan["fused_ops_per_micro_batch"]]
        if cuda and tp > 1:
            assert "all_gather_gemm" in ops and "gemm_reduce_scatter" in ops, ops
        if pp > 1:
            assert plan["schedule"] == "1F1B" and plan["stages"] == pp
        if captured:
            assert plan.get("captured_micro_batch") is True, "the micro-batch was not captured"
        print(f"GPT FLOW tp{tp} pp{pp} dp{dp} {device} OK", [round(v, 4) for v in losses[:4]])
    flow.comm.barrier()


if __name__ == "__main__":
    main()
