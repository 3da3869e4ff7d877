"""Eager ``DistributedDataParallel`` on local tensors (reference: python/oneflow/nn/parallel/distributed.py:70-185).

Parameters are broadcast from rank 0, grouped in reverse order into buckets of ``bucket_size`` parameters
whose gradients live in one contiguous buffer per bucket; a post-accumulate-grad hook counts ready
gradients and, when a bucket is complete, launches its all-reduce fused with the 1/world scale — on CUDA
the in-kernel all-reduce over symmetric memory (comm.symmetric), on CPU gloo — while the backward of
earlier layers continues. Buffers are broadcast before every forward (``broadcast_buffers``); parameters
that received no gradient contribute zeros so every rank issues the same collectives."""
from __future__ import annotations

import torch
import torch.distributed as dist


class DistributedDataParallel(torch.nn.Module):
    _is_ddp_module = True      # the mark the reference sets on a module it has wrapped
    def __init__(self, module, *, broadcast_buffers=True, broadcast_parameters=True, bucket_size=10, use_bucket=True):
        super().__init__()
        self.module = module
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.broadcast_buffers = broadcast_buffers
        params = [p for p in module.parameters() if p.requires_grad]
        for p in params:
            if p.dtype != torch.float32:
                raise TypeError("DistributedDataParallel only supports float32 parameters")
        if self.world > 1 and broadcast_parameters:
            for p in module.parameters():
                dist.broadcast(p.data, 0)
        self._coll = None
        self._buckets = []
        if self.world > 1:
            rev = list(reversed(params))
            size = bucket_size if use_bucket else 1
            for i in range(0, len(rev), size):
                self._make_bucket(rev[i:i + size])
        self._ready = {}
        self._pending = []

    def _make_bucket(self, ps):
        n = sum((p.numel() + 7) // 8 * 8 for p in ps)
        flat = torch.zeros(n, dtype=torch.float32, device=ps[0].device)
        views, off = [], 0
        for p in ps:
            v = flat[off:off + p.numel()].view(p.shape)
            views.append(v)
            off += (p.numel() + 7) // 8 * 8
        b = {"params": ps, "flat": flat, "views": views, "count": 0}
        idx = len(self._buckets)
        self._buckets.append(b)
        for p, v in zip(ps, views):
            p.register_post_accumulate_grad_hook(self._hook(idx, v))

    def _hook(self, bucket_idx, view):
        def fn(p):
            b = self._buckets[bucket_idx]
            view.copy_(p.grad)
            p.grad = view              # the gradient now lives in the bucket's contiguous storage
            b["count"] += 1
            if b["count"] == len(b["params"]):
                self._launch(b)
        return fn

    def _launch(self, b):
        flat = b["flat"]
        if flat.is_cuda:
            coll = self._device_coll(flat.device)
            if coll is not None and flat.numel() * 4 <= coll.io_bytes:
                out = coll.all_reduce(flat, scale=1.0 / self.world)
                flat.copy_(out)
                b["count"] = 0
                return
        flat.mul_(1.0 / self.world)
        self._pending.append(dist.all_reduce(flat, async_op=True))
        b["count"] = 0

    def _device_coll(self, device):
        if self._coll is None:
            if self.world > 8:
                self._coll = False          # the peer-memory collectives address one node (8 GPUs): larger groups use NCCL
            else:
                # a missing kernel library or a failed peer mapping raises: no silent switch to another path on a GPU
                from ...comm.symmetric import DeviceCollectives, SymmetricArena
                arena = SymmetricArena(None, list(range(self.world)), device, 3 * (64 << 20) + (1 << 22))
                self._coll = DeviceCollectives(arena, io_bytes=64 << 20)
        return self._coll or None

    def finish_pending(self):
        """Flushes buckets that did not fill (unused parameters) and waits for outstanding reductions."""
        for b in self._buckets:
            if 0 < b["count"] < len(b["params"]):
                for p, v in zip(b["params"], b["views"]):
                    if p.grad is None or p.grad.data_ptr() != v.data_ptr():
                        if p.grad is None:
                            v.zero_()
                        p.grad = v
                self._launch(b)
        for w in self._pending:
            w.wait()
        self._pending = []

    def forward(self, *args, **kwargs):
        if self.world > 1 and self.broadcast_buffers:
            for buf in self.module.buffers():
                dist.broadcast(buf, 0)
        out = self.module(*args, **kwargs)
        if self.world > 1 and torch.is_grad_enabled():
            # when the backward of this forward has run, flush partially filled buckets
            torch.autograd.Variable._execution_engine.queue_callback  # noqa: B018  (presence check)
            self._arm_flush(out)
        return out

    def _arm_flush(self, out):
        outs = [o for o in (out if isinstance(out, (tuple, list)) else [out]) if isinstance(o, torch.Tensor) and o.requires_grad]
        if not outs:
            return
        ddp = self

        def hook(_grad):
            torch.autograd.Variable._execution_engine.queue_callback(ddp.finish_pending)
            return None
        outs[0].register_hook(hook)
