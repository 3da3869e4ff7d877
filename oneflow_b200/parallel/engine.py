"""Training engine for the staged models (GPT/BERT): micro-batching with gradient accumulation,
1F1B pipeline schedule over NCCL p2p, tensor-parallel context, flat fused AdamW with optional
ZeRO-1 sharding over the data-parallel group.

What the reference expresses through nn.Graph passes (gradient accumulation: repeat/acc/unpack
ops, lazy_op_interpreter.cpp:270-330; pipeline: pipeline_buffer_pass.cpp + actor back-pressure;
ZeRO: optimizer_placement_optimization_pass.cpp; fused model update: fuse_update_ops_pass.cpp,
multi_tensor_model_update.cpp; clip_grad via multi_reduce_sum_pow_abs) is an explicit
per-rank schedule here, launched on CUDA streams.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K


class FlatAdamW:
    """AdamW over a ParamStore: fp32 master weights and moments in flat buffers, the bf16 model copy
    written by the same kernel; global-norm clipping and the overflow skip stay on the device.

    With ``zero`` (a parallel.zero.ZeroShard) only this rank's slice of master/m/v exists (ZeRO stage 1):
    gradients are reduce-scattered into the slice and updated parameters all-gathered.
    """

    def __init__(self, store, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=1.0, zero=None,
                 norm_groups=(), tp_size=1):
        self.store = store
        self.tp_size = tp_size
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        self.zero = zero
        self.norm_groups = tuple(g for g in norm_groups if g is not None)
        self.step_count = 0
        n = store.total
        self.lo, self.hi = (0, n) if zero is None else zero.range(n)
        dev = store.flat.device
        self.master = store.flat[self.lo:self.hi].float()
        self.m = torch.zeros(self.hi - self.lo, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.hi - self.lo, dtype=torch.float32, device=dev)
        self.lr_t = torch.full((1,), lr, dtype=torch.float32, device=dev)
        self._sq = torch.zeros(2, dtype=torch.float32, device=dev)

    def set_lr(self, lr):
        self.lr = lr
        self.lr_t.fill_(lr)

    def _split_replicated(self):
        """This rank's range [lo, hi) cut into (replicated pieces, unique pieces), as offsets into the shard.
        Pieces are 64-element aligned like the store, so they satisfy the kernels' alignment rule."""
        rep, uniq, cur = [], [], self.lo
        for a, b in getattr(self.store, "replicated_ranges", []):
            a, b = max(a, self.lo), min(b, self.hi)
            if a >= b:
                continue
            if a > cur:
                uniq.append((cur - self.lo, a - self.lo))
            rep.append((a - self.lo, b - self.lo))
            cur = b
        if cur < self.hi:
            uniq.append((cur - self.lo, self.hi - self.lo))
        return rep, uniq

    def _segments(self):
        """(lo, hi, weight_decay) pieces of this rank's range: the decayed prefix and the rest."""
        d = self.store.decay_end
        segs = []
        if self.lo < d:
            segs.append((self.lo, min(self.hi, d), self.wd))
        if self.hi > d:
            segs.append((max(self.lo, d), self.hi, 0.0))
        return [s for s in segs if s[1] > s[0]]

    def step(self, grad_scale=1.0):
        st = self.store
        self.step_count += 1
        grad = st.grad
        if self.zero is not None:
            grad_shard = self.zero.reduce_scatter_grads(grad, self.lo, self.hi)
        else:
            grad_shard = grad[self.lo:self.hi]
        rep, uniq = self._split_replicated()
        if rep and self.tp_size > 1:
            # tensors replicated over the tensor-parallel group enter the global norm once, not tp times
            sq = K.multi_tensor_sqsum([grad_shard[a:b] for a, b in uniq], out=self._sq) if uniq else self._sq.zero_()
            sq_rep = K.multi_tensor_sqsum([grad_shard[a:b] for a, b in rep])
            sq += sq_rep / self.tp_size
        else:
            sq = K.multi_tensor_sqsum([grad_shard], out=self._sq)
        groups = list(self.norm_groups) + ([self.zero.group] if self.zero is not None else [])
        for g in groups:
            dist.all_reduce(sq, group=g)
        factor, found_inf, self.last_norm = K.clip_factor(sq, self.clip if self.clip else 0.0)
        for lo, hi, wd in self._segments():
            a, b = lo - self.lo, hi - self.lo
            K.multi_tensor_adamw([grad_shard[a:b]], [self.master[a:b]], [st.flat[lo:hi]], [self.m[a:b]], [self.v[a:b]],
                                 lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=wd,
                                 scale=grad_scale, step=self.step_count, lr_tensor=self.lr_t, scale_tensor=factor,
                                 skip_if=found_inf)
        if self.zero is not None:
            self.zero.all_gather_params(st.flat, self.lo, self.hi)

    def state_dict(self):
        return {"step": self.step_count, "master": self.master, "m": self.m, "v": self.v, "lr": self.lr}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.set_lr(sd["lr"])


class FlatSGD:
    """SGD with momentum over a ParamStore: fp32 master weights and momentum in flat buffers, the bf16 model copy
    written by the same kernel; weight decay (L2 form, as torch.optim.SGD) only on the store's decayed prefix.
    Gradients must already be reduced over the data-parallel ranks."""

    def __init__(self, store, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=False):
        self.store, self.lr, self.momentum, self.wd, self.nesterov = store, lr, momentum, weight_decay, nesterov
        dev = store.flat.device
        self.master = store.flat.float()
        self.m = torch.zeros(store.total, dtype=torch.float32, device=dev) if momentum else None
        self.lr_t = torch.full((1,), lr, dtype=torch.float32, device=dev)
        self.step_count = 0

    def set_lr(self, lr):
        self.lr = lr
        self.lr_t.fill_(lr)

    def step(self, grad_scale=1.0):
        st = self.store
        self.step_count += 1
        d = st.decay_end
        for lo, hi, wd in ((0, d, self.wd), (d, st.total, 0.0)):
            if hi <= lo:
                continue
            K.multi_tensor_sgd([st.grad[lo:hi]], [self.master[lo:hi]], [st.flat[lo:hi]], [self.m[lo:hi]] if self.m is not None else None,
                               lr=self.lr, momentum=self.momentum, nesterov=self.nesterov, l2=wd, scale=grad_scale,
                               lr_tensor=self.lr_t)

    def state_dict(self):
        return {"step": self.step_count, "master": self.master, "m": self.m, "lr": self.lr}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        if self.m is not None and sd.get("m") is not None:
            self.m.copy_(sd["m"])
        self.set_lr(sd["lr"])


class PipelineP2P:
    """Activations / activation-gradients between neighbouring pipeline stages over NCCL (or gloo)
    send/recv. A send and the matching receive of the opposite direction are posted as one batch so the
    two neighbours never wait on each other in the 1F1B steady state."""

    def __init__(self, group, prev_rank, next_rank, shape, dtype, device):
        self.group, self.prev, self.next = group, prev_rank, next_rank
        self.shape, self.dtype, self.device = shape, dtype, device

    def _run(self, ops):
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()

    def _buf(self):
        return torch.empty(self.shape, dtype=self.dtype, device=self.device)

    def recv_forward(self):
        if self.prev is None:
            return None
        t = self._buf()
        self._run([dist.P2POp(dist.irecv, t, self.prev, self.group)])
        return t

    def recv_backward(self):
        if self.next is None:
            return None
        t = self._buf()
        self._run([dist.P2POp(dist.irecv, t, self.next, self.group)])
        return t

    def send_forward(self, x):
        if self.next is not None:
            self._run([dist.P2POp(dist.isend, x, self.next, self.group)])

    def send_backward(self, g):
        if self.prev is not None:
            self._run([dist.P2POp(dist.isend, g, self.prev, self.group)])

    def send_forward_recv_backward(self, x):
        if self.next is None:
            return None
        t = self._buf()
        self._run([dist.P2POp(dist.isend, x, self.next, self.group), dist.P2POp(dist.irecv, t, self.next, self.group)])
        return t

    def send_backward_recv_forward(self, g):
        if self.prev is None:
            return None
        t = self._buf()
        self._run([dist.P2POp(dist.isend, g, self.prev, self.group), dist.P2POp(dist.irecv, t, self.prev, self.group)])
        return t


class StagedTrainer:
    """Runs one optimizer step = ``n_micro`` micro-batches through a model stage with the 1F1B schedule
    (a single stage degenerates to forward+backward per micro-batch) and a fused optimizer update."""

    def __init__(self, stage, optimizer, n_micro, p2p: Optional[PipelineP2P] = None, pp_rank=0, pp_size=1,
                 embedding_group=None):
        self.stage, self.opt, self.n_micro = stage, optimizer, n_micro
        self.p2p, self.pp_rank, self.pp_size = p2p, pp_rank, pp_size
        self.embedding_group = embedding_group

    def _fwd(self, m, micro_inputs, micro_labels, recv):
        st = self.stage
        inp = micro_inputs[m] if st.first else recv
        lab = micro_labels[m] if st.last else None
        bs = tuple(micro_inputs[m].shape) if micro_inputs is not None else None
        return st.forward(m, inp, lab, loss_scale=1.0 / self.n_micro, bs=bs)

    def train_step(self, tokens):
        """tokens: int64 [n_micro * micro_batch, seq + 1] on the device (every pipeline rank receives the
        same batch; the first stage reads the inputs, the last stage the shifted labels).
        Returns the mean loss over the step as a 0-d device tensor (valid on the last stage)."""
        st, n = self.stage, self.n_micro
        mb = tokens.shape[0] // n
        if hasattr(st, "split_batch"):
            inputs, labels = st.split_batch(tokens, n)     # model-specific batch layout
        else:
            inputs = [tokens[i * mb:(i + 1) * mb, :-1].contiguous() for i in range(n)]
            labels = [tokens[i * mb:(i + 1) * mb, 1:].contiguous() for i in range(n)]
        st.store.start_accumulation()
        loss = torch.zeros((), dtype=torch.float32, device=tokens.device)
        if self.pp_size == 1:
            for m in range(n):
                out = self._fwd(m, inputs, labels, None)
                loss += out
                st.backward(m)
        else:
            p2p = self.p2p
            warm = min(self.pp_size - self.pp_rank - 1, n)
            steady = n - warm
            outs = {}
            recv = p2p.recv_forward() if not st.first else None
            fm = bm = 0
            for _ in range(warm):
                out = self._fwd(fm, inputs, labels, recv)
                fm += 1
                if st.last:
                    loss += out
                else:
                    p2p.send_forward(out)
                    outs[fm - 1] = out
                if fm < n:
                    recv = p2p.recv_forward() if not st.first else None
            grad = None
            for i in range(steady):
                out = self._fwd(fm, inputs, labels, recv)
                fm += 1
                if st.last:
                    loss += out
                    grad = None
                else:
                    grad = p2p.send_forward_recv_backward(out)
                dprev = st.backward(bm, grad)
                bm += 1
                if fm < n:
                    recv = p2p.send_backward_recv_forward(dprev)
                else:  # last steady iteration: nothing left to receive
                    p2p.send_backward(dprev)
                    recv = None
            for _ in range(warm):
                grad = p2p.recv_backward()
                dprev = st.backward(bm, grad)
                bm += 1
                if not st.first:
                    p2p.send_backward(dprev)
            # tied embedding: the first and last stage each hold a copy of wte; sum their gradients
            if self.embedding_group is not None and (st.first or st.last):
                dist.all_reduce(st.store.g["wte"], group=self.embedding_group)
        if hasattr(st, "sync_replicated_grads"):
            st.sync_replicated_grads()
        self.opt.step()
        return loss
