"""Data-parallel gradient paths.

``ZeroShard`` (ZeRO stage 1/2): every data-parallel rank owns a contiguous slice of the flat parameter
buffer; gradients are reduce-scattered straight into that slice (``P -> S(0)``, fused with the 1/dp scale
and the cast to fp32), the owner updates its slice of the fp32 master weights and moments, and the
updated bf16 parameters are all-gathered (``S(0) -> B``). This is what the reference's
``optimizer_placement_optimization_pass.cpp`` (mode distributed_split) arranges with SBP rewrites.

``GradAllReduce``: plain data parallelism (``P -> B``), bucketed so that a bucket's all-reduce (fused with
cast and scale) can be launched while the backward of earlier layers still runs — the job of the
reference's DDP hooks (python/oneflow/nn/parallel/distributed.py:26-67) and of its fused NCCL all-reduce
(core/job/collective_boxing/nccl_executor_backend.cu:265-325).

CUDA tensors use the in-kernel collectives over symmetric memory; CPU tensors (gloo ranks in tests) use
torch.distributed.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _align_up(n, a):
    return (n + a - 1) // a * a


class _DPBase:
    def __init__(self, group, ranks, device, io_bytes=64 << 20):
        self.group, self.ranks = group, list(ranks)
        self.size = len(self.ranks)
        self.rank = self.ranks.index(dist.get_rank())
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.coll = None
        if self.cuda:
            from ..comm.symmetric import DeviceCollectives, SymmetricArena
            self.arena = SymmetricArena(group, ranks, device, 3 * io_bytes + (1 << 22))
            self.coll = DeviceCollectives(self.arena, io_bytes=io_bytes)
            # elements per chunk such that every rank's slice stays 16-byte aligned for fp32 and bf16
            self.chunk = (io_bytes // 4) // (self.size * 64) * (self.size * 64)


class ZeroShard(_DPBase):
    def range(self, n):
        """This rank's [lo, hi) slice of a flat buffer of n elements (n is padded by the store to 64)."""
        per = _align_up((n + self.size - 1) // self.size, 64)
        lo = min(n, self.rank * per)
        return lo, min(n, lo + per)

    def _per(self, n):
        return _align_up((n + self.size - 1) // self.size, 64)

    def reduce_scatter_grads(self, grad, lo, hi):
        """grad: flat gradients of the whole buffer (fp32 or bf16). Returns the fp32 mean over the
        data-parallel ranks of this rank's slice [lo, hi)."""
        n = grad.numel()
        per = self._per(n)
        scale = 1.0 / self.size
        out = torch.empty(hi - lo, dtype=torch.float32, device=grad.device)
        if not self.cuda:
            full = grad.float().clone()
            dist.all_reduce(full, group=self.group)
            out.copy_(full[lo:hi] * scale)
            return out
        # The buffer is cut into pieces of `sub` elements per rank so that each call reduces
        # [r*per + k*sub, r*per + (k+1)*sub) of every rank r in one kernel: gather those pieces into the
        # staging region as a [size, sub] matrix, whose row r then lands on rank r.
        sub_max = self.chunk // self.size
        done = 0
        while done < per:
            sub = min(sub_max, per - done)
            stage = self.coll.input_view((self.size, sub), grad.dtype)
            for r in range(self.size):
                a = min(n, r * per + done)
                b = min(n, r * per + done + sub)
                if b > a:
                    stage[r, :b - a].copy_(grad[a:b])
                if b - a < sub:
                    stage[r, b - a:].zero_()
            piece = self.coll.reduce_scatter(stage.view(self.size * sub), scale=scale, out_dtype=torch.float32, staged=True)
            a = lo + done
            b = min(hi, a + sub)
            if b > a:
                out[done:done + (b - a)].copy_(piece[:b - a])
            done += sub
        return out

    def all_gather_params(self, flat, lo, hi):
        """Every rank contributes flat[lo:hi]; afterwards the whole flat buffer is up to date everywhere."""
        n = flat.numel()
        per = self._per(n)
        if not self.cuda:
            mine = torch.zeros(per, dtype=flat.dtype)
            mine[:hi - lo] = flat[lo:hi]
            parts = [torch.empty_like(mine) for _ in range(self.size)]
            dist.all_gather(parts, mine, group=self.group)
            for r, p in enumerate(parts):
                a = min(n, r * per)
                b = min(n, a + per)
                flat[a:b].copy_(p[:b - a])
            return
        sub_max = self.chunk // self.size
        done = 0
        while done < per:
            sub = min(sub_max, per - done)
            stage = self.coll.input_view((sub,), flat.dtype)
            a = min(hi, lo + done)
            b = min(hi, lo + done + sub)
            if b > a:
                stage[:b - a].copy_(flat[a:b])
            gathered = self.coll.all_gather(stage, staged=True).view(self.size, sub)
            for r in range(self.size):
                ra = min(n, r * per + done)
                rb = min(n, r * per + done + sub)
                if rb > ra and r != self.rank:
                    flat[ra:rb].copy_(gathered[r, :rb - ra])
            done += sub


class GradAllReduce(_DPBase):
    """Mean of the gradients over the data-parallel ranks, written back in place (fp32 or bf16), chunk by
    chunk so that callers can invoke it per bucket while the backward is still producing later buckets."""

    def range(self, n):
        return 0, n

    def all_reduce_(self, grad, scale=None):
        scale = (1.0 / self.size) if scale is None else scale
        if not self.cuda:
            g = grad.float()
            dist.all_reduce(g, group=self.group)
            grad.copy_(g * scale)
            return grad
        flat = grad.view(-1)
        n = flat.numel()
        done = 0
        while done < n:
            c = min(self.chunk, n - done)
            piece = self.coll.all_reduce(flat[done:done + c], scale=scale, out_dtype=flat.dtype)
            flat[done:done + c].copy_(piece)
            done += c
        return grad

    def reduce_scatter_grads(self, grad, lo, hi):
        self.all_reduce_(grad)
        return grad[lo:hi] if grad.dtype == torch.float32 else grad[lo:hi].float()

    def all_gather_params(self, flat, lo, hi):
        return
