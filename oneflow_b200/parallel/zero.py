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


class ArenaZero:
    """ZeRO stage 1 on flat buffers that LIVE in the symmetric arena: the fp32 gradient buffer and the parameter buffer of
    a rank are peer-mapped, so the reduce-scatter reads the peers' gradients where backward accumulated them and the
    parameter all-gather writes the peers' updated slices where the modules read them. No pack, no staging copy, one
    kernel each (what the reference arranges with SBP rewrites plus NCCL calls:
    oneflow/core/job_rewriter/optimizer_placement_optimization_pass.cpp:381-467).

    ``grad`` (fp32) and ``flat`` (parameter dtype) hold ``padded = n * per`` elements; rank r owns [r * per, (r + 1) * per)."""

    def __init__(self, group, ranks, device, total, param_dtype):
        from ..comm.symmetric import SymmetricArena
        self.group, self.ranks = group, list(ranks)
        self.size = len(self.ranks)
        self.rank = self.ranks.index(dist.get_rank())
        self.device = torch.device(device)
        self.total = int(total)
        self.per = _align_up((self.total + self.size - 1) // self.size, 64)
        self.padded = self.per * self.size
        esz = torch.empty((), dtype=param_dtype).element_size()
        self.param_dtype = param_dtype
        self.arena = SymmetricArena(group, ranks, device, self.padded * (4 + esz) + (1 << 16))
        self.grad_off = self.arena.region(self.padded * 4)
        self.flat_off = self.arena.region(self.padded * esz)
        self.grad = self.arena.view(self.grad_off, (self.padded,), torch.float32)
        self.flat = self.arena.view(self.flat_off, (self.padded,), param_dtype)
        self.epoch = 0

    def range(self, n=None):
        lo = min(self.total, self.rank * self.per)
        return lo, min(self.total, lo + self.per)

    def reduce_scatter_grads(self, scale=None):
        """fp32 [per]: this rank's slice of the sum of all ranks' gradient buffers, times ``scale`` (default 1 / n)."""
        import ctypes
        from ctypes import c_float, c_int, c_longlong, c_uint
        from ..ops import _native
        from ..ops import kernels as _k
        scale = (1.0 / self.size) if scale is None else scale
        out = torch.empty(self.per, dtype=torch.float32, device=self.device)
        self.epoch += 1
        _native.check(_native.kernels().ofb_comm_collective(
            ctypes.byref(self.arena.ctx), c_int(1), c_longlong(self.grad_off), c_longlong(self.grad_off), c_int(0), _native.ptr(out),
            c_int(0), c_longlong(self.padded), c_float(scale), c_uint(self.epoch), c_int(128), _native.stream_ptr()), "zero reduce-scatter")
        _k._count()
        return out

    def all_gather_params(self):
        """Every rank's freshly updated slice of the parameter buffer lands in this rank's copy, in place."""
        import ctypes
        from ctypes import c_int, c_longlong, c_uint
        from ..ops import _native
        from ..ops import kernels as _k
        self.epoch += 1
        dt = 0 if self.param_dtype == torch.float32 else 1
        _native.check(_native.kernels().ofb_comm_all_gather_inplace(
            ctypes.byref(self.arena.ctx), c_longlong(self.flat_off), c_int(dt), _native.ptr(self.flat), c_longlong(self.padded),
            c_uint(self.epoch), c_int(128), _native.stream_ptr()), "zero all-gather")
        _k._count()
