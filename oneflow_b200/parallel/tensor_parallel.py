"""Tensor-parallel context with sequence-parallel activations.

Between the tensor-parallel regions the activations are split along the token axis (SBP ``S(0)`` on the
tp mesh axis); the column-parallel products gather them (``S(0) -> B``, fused: all-gather -> GEMM) and the
row-parallel products reduce and re-split them (``P -> S(0)``, fused: GEMM -> reduce-scatter). Both fused
products are single tcgen05 kernels that move their data through NVSwitch peer memory
(csrc/comm/gemm_comm.cu); the remaining small exchanges use the in-kernel collectives of
``comm.symmetric``. In the reference these are matmul ops followed by ``_nccl_logical_*`` boxing ops
(oneflow/core/job_rewriter/insert_nccl_logical_op_pass.cpp:192-296).

On CPU tensors (gloo ranks in the tests) the same methods run on torch.distributed collectives.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint

import torch
import torch.distributed as dist

from ..ops import _native
from ..ops import gemm as G
from ..ops import kernels as K


class TPContext:
    def __init__(self, group, ranks, device, max_tokens, max_cols, hidden=None):
        self.group, self.ranks = group, list(ranks)
        self.size = len(self.ranks)
        self.rank = self.ranks.index(dist.get_rank())
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.max_tokens = max_tokens
        self.ag_epoch = 0
        self.rs_epoch = 0
        if self.cuda:
            from ..comm.symmetric import DeviceCollectives, SymmetricArena
            hidden = hidden or max_cols
            self.stage_bytes = 2 * max_tokens * hidden * 2
            self.flag_stride = 8192
            self.flag_bytes = 2 * 8 * self.flag_stride * 4
            self.gathered_bytes = 2 * max_tokens * hidden * 2
            io = max(max_tokens * hidden * 2, 1 << 22)
            self.ag_flag_bytes = 8 * 256 * 4          # per owner, one arrival flag per CTA of the pushing rank
            total = self.stage_bytes + self.flag_bytes + self.gathered_bytes + self.ag_flag_bytes + 3 * io + (1 << 22)
            self.arena = SymmetricArena(group, ranks, device, total)
            self.stage_off = self.arena.region(self.stage_bytes)
            self.flag_off = self.arena.region(self.flag_bytes)
            self.gathered_off = self.arena.region(self.gathered_bytes)
            self.ag_flag_off = self.arena.region(self.ag_flag_bytes)
            self.coll = DeviceCollectives(self.arena, io_bytes=io)
            self.hidden_cap = hidden

    # ------------------------------------------------------------------ fused products
    def ag_gemm(self, x_shard, w, *, b_layout="nk", bias=None, act=0, aux_in=None, want_aux=False, return_gathered=False):
        """epilogue(all_gather_rows(x_shard) @ W^T). Returns out, (out, aux) and/or (gathered, out)."""
        n = self.size
        Tl, Kd = x_shard.shape
        T = Tl * n
        N = w.shape[0] if b_layout == "nk" else w.shape[1]
        if not self.cuda:
            full = self.all_gather_rows(x_shard)
            res = G.gemm(full, w, b_layout=b_layout, bias=bias, act=act, aux_in=aux_in, want_aux=want_aux)
            return self._pack(res, full, want_aux, return_gathered)
        if 2 * T * Kd * 2 > self.gathered_bytes:
            raise ValueError("ag_gemm: problem larger than the gathered buffer")
        out = torch.empty((T, N), dtype=torch.bfloat16, device=x_shard.device)
        aux = torch.empty((T, N), dtype=torch.bfloat16, device=x_shard.device) if want_aux else None
        self.ag_epoch += 1
        ld_aux = N if (aux is not None or aux_in is not None) else 0
        _native.check(_native.kernels().ofb_ag_gemm(
            ctypes.byref(self.arena.ctx), _native.ptr(x_shard), _native.ptr(w), c_longlong(w.stride(0)),
            c_int(0 if b_layout == "nk" else 1), _native.ptr(out), c_longlong(N), _native.ptr(bias), _native.ptr(aux_in),
            _native.ptr(aux), c_longlong(ld_aux), c_int(G._act_code(act)), c_int(T), c_int(N), c_int(Kd), c_float(1.0),
            c_longlong(self.gathered_off), c_longlong(self.gathered_bytes), c_longlong(self.ag_flag_off), c_uint(self.ag_epoch), c_int(8),
            _native.stream_ptr()), "ag_gemm")
        K._count()
        gathered = None
        if return_gathered:
            # parity halves sit at fixed offsets of the region, whatever the shape of the call
            gathered = self.arena.view(self.gathered_off + (self.ag_epoch & 1) * (self.gathered_bytes // 2), (T, Kd), torch.bfloat16)
        res = (out, aux) if want_aux else out
        return self._pack(res, gathered, want_aux, return_gathered)

    @staticmethod
    def _pack(res, gathered, want_aux, return_gathered):
        if return_gathered:
            return (gathered,) + (res if isinstance(res, tuple) else (res,))
        return res

    def gemm_rs(self, a, w, *, b_layout="nk", bias=None, residual=None):
        """reduce_scatter_rows(a @ W^T) + bias + residual_shard -> [T / tp, N]."""
        n = self.size
        T, Kd = a.shape
        N = w.shape[0] if b_layout == "nk" else w.shape[1]
        if not self.cuda:
            part = G.gemm(a, w, b_layout=b_layout, out_dtype=torch.float32 if a.dtype == torch.float32 else a.dtype)
            out = self.reduce_scatter_rows(part)
            o = out.float()
            if bias is not None:
                o = o + bias.float()
            if residual is not None:
                o = o + residual.float()
            return o.to(a.dtype)
        if T * N * 2 * 2 > self.stage_bytes:
            raise ValueError("gemm_rs: problem larger than the staging buffer")
        out = torch.empty((T // n, N), dtype=torch.bfloat16, device=a.device)
        self.rs_epoch += 1
        _native.check(_native.kernels().ofb_gemm_rs(
            ctypes.byref(self.arena.ctx), _native.ptr(a), c_longlong(a.stride(0)), _native.ptr(w), c_longlong(w.stride(0)),
            c_int(0 if b_layout == "nk" else 1), _native.ptr(out), c_longlong(N), _native.ptr(bias), _native.ptr(residual),
            c_longlong(residual.stride(0) if residual is not None else 0), c_int(T), c_int(N), c_int(Kd), c_float(1.0),
            c_longlong(self.stage_off), c_longlong(self.stage_bytes), c_longlong(self.flag_off), c_int(self.flag_stride),
            c_uint(self.rs_epoch),
            c_int(2), _native.stream_ptr()), "gemm_rs")
        K._count()
        return out

    # ------------------------------------------------------------------ plain exchanges
    def all_gather_rows(self, x):
        if not self.cuda:
            parts = [torch.empty_like(x) for _ in range(self.size)]
            dist.all_gather(parts, x.contiguous(), group=self.group)
            return torch.cat(parts, 0)
        return self.coll.all_gather(x.contiguous())

    def reduce_scatter_rows(self, x):
        if not self.cuda:
            y = x.float().contiguous()
            dist.all_reduce(y, group=self.group)
            m = x.shape[0] // self.size
            return y[self.rank * m:(self.rank + 1) * m].to(x.dtype)
        return self.coll.reduce_scatter(x.contiguous())

    def all_reduce(self, x, scale=1.0):
        if not self.cuda:
            y = x.float().contiguous()
            dist.all_reduce(y, group=self.group)
            return (y * scale).to(x.dtype)
        return self.coll.all_reduce(x.contiguous(), scale=scale)

    def merge_xent_stats(self, stats):
        """Combines per-shard (max, sum-exp, target-logit) rows over the vocabulary shards."""
        if not self.cuda:
            parts = [torch.empty_like(stats) for _ in range(self.size)]
            dist.all_gather(parts, stats.contiguous(), group=self.group)
            return K.xent_merge(torch.stack(parts))
        rows = stats.shape[0]
        allp = self.coll.all_gather(stats.reshape(1, -1)).view(self.size, rows, 3)
        return K.xent_merge(allp)
