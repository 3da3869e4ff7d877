"""``flow.comm``: collectives on LOCAL tensors (reference: python/oneflow/comm/comm_ops.py:21-470).
CPU tensors use gloo, CUDA tensors NCCL; the SBP boxing layer and the parallel engines use the in-kernel
collectives of ``comm.symmetric`` instead."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _w():
    return dist.get_world_size() if dist.is_initialized() else 1


def all_reduce(tensor):
    """In-place sum over all ranks."""
    if _w() > 1:
        dist.all_reduce(tensor)
    return tensor


def all_gather(tensor_list, tensor):
    if _w() == 1:
        tensor_list[0].copy_(tensor)
        return
    dist.all_gather(tensor_list, tensor.contiguous())


def all_gather_into_tensor(output_tensor, input_tensor):
    if _w() == 1:
        output_tensor.copy_(input_tensor.reshape(output_tensor.shape))
        return
    if input_tensor.is_cuda:
        dist.all_gather_into_tensor(output_tensor, input_tensor.contiguous())
    else:
        parts = [torch.empty_like(input_tensor) for _ in range(_w())]
        dist.all_gather(parts, input_tensor.contiguous())
        output_tensor.copy_(torch.cat(parts, 0).reshape(output_tensor.shape))


def broadcast(tensor, src):
    if _w() > 1:
        dist.broadcast(tensor, src)
    return tensor


def scatter(tensor, scatter_list=None, src=0):
    if _w() == 1:
        tensor.copy_(scatter_list[0])
        return
    if tensor.is_cuda and dist.get_backend() != "gloo":
        # NCCL has no scatter: the source sends each piece
        me = dist.get_rank()
        if me == src:
            for r, piece in enumerate(scatter_list):
                if r == src:
                    tensor.copy_(piece)
                else:
                    dist.send(piece.contiguous(), r)
        else:
            dist.recv(tensor, src)
        return
    dist.scatter(tensor, scatter_list if dist.get_rank() == src else None, src=src)


def reduce(tensor, dst):
    if _w() > 1:
        dist.reduce(tensor, dst)
    return tensor


def gather(tensor, gather_list=None, dst=0):
    if _w() == 1:
        gather_list[0].copy_(tensor)
        return
    if tensor.is_cuda and dist.get_backend() != "gloo":
        parts = [torch.empty_like(tensor) for _ in range(_w())]
        dist.all_gather(parts, tensor.contiguous())
        if dist.get_rank() == dst:
            for g, p in zip(gather_list, parts):
                g.copy_(p)
        return
    dist.gather(tensor, gather_list if dist.get_rank() == dst else None, dst=dst)


def all_to_all(output_tensor_list, input_tensor_list):
    n = _w()
    if n == 1:
        output_tensor_list[0].copy_(input_tensor_list[0])
        return
    if input_tensor_list[0].is_cuda:
        dist.all_to_all(output_tensor_list, [t.contiguous() for t in input_tensor_list])
        return
    me = dist.get_rank()
    reqs = []
    for r in range(n):
        if r == me:
            output_tensor_list[r].copy_(input_tensor_list[r])
        else:
            reqs.append(dist.isend(input_tensor_list[r].contiguous(), r))
            reqs.append(dist.irecv(output_tensor_list[r], r))
    for q in reqs:
        q.wait()


def reduce_scatter(output, input_list):
    n = _w()
    if n == 1:
        output.copy_(input_list[0])
        return
    if output.is_cuda:
        dist.reduce_scatter(output, [t.contiguous() for t in input_list])
        return
    full = torch.stack([t.contiguous() for t in input_list])
    dist.all_reduce(full)
    output.copy_(full[dist.get_rank()])


def reduce_scatter_tensor(output_tensor, input_tensor):
    n = _w()
    chunks = list(input_tensor.reshape(n, -1).unbind(0))
    out_flat = output_tensor.reshape(-1)
    reduce_scatter(out_flat, chunks)
    return output_tensor


def barrier():
    if _w() > 1:
        dist.barrier()


def send(tensor, dst, send_meta=True):
    """With send_meta the shape and dtype travel first, so the receiver needs no prior knowledge
    (reference: oneflow/core/functional/impl/comm_functor.cpp:427-441)."""
    if send_meta:
        dist.send_object_list([(tuple(tensor.shape), str(tensor.dtype))], dst)
    dist.send(tensor.contiguous(), dst)


def recv(src, shape=None, dtype=None, device=None, *, out=None):
    if out is None:
        if shape is None:
            box = [None]
            dist.recv_object_list(box, src)
            shape, dtype_s = box[0]
            dtype = getattr(torch, dtype_s.split(".")[-1])
        if device is None:
            device = "cuda" if (dist.get_backend() == "nccl") else "cpu"
        out = torch.empty(shape, dtype=dtype, device=device)
    elif shape is None:
        box = [None]
        dist.recv_object_list(box, src)
    dist.recv(out, src)
    return out
