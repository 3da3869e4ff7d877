"""SBP / placement conversion ("boxing") of global tensors.

A conversion is planned as a sequence of named 1-D steps over one mesh axis each, mirroring the
reference's boxing function registry (oneflow/core/boxing/eager_boxing_interpreter_mgr.cpp:137-171):

    identity            same sbp
    ccl-p-to-b          all-reduce            (bool tensors reduce with max)
    ccl-p-to-s          reduce-scatter
    ccl-s-to-b          all-gather            (uneven BalancedSplitter shards supported)
    ccl-s-to-s          all-to-all
    symmetric-b-to-s    local slice, no traffic
    symmetric-b-to-p    first rank of the axis keeps the data, the others hold zeros
    symmetric-s-to-p    shard padded into a zero tensor of the full extent
    naive-1-to-1 / asymmetric-broadcast   placement changes (p2p send/recv)
    nd-sbp axis-wise / generic-nd         n-D conversions: axis by axis when the split dimensions do not
                                          collide, otherwise through the all-broadcast form

CUDA tensors with even dim-0 splits use the in-kernel collectives over symmetric memory
(comm.symmetric.DeviceCollectives); everything else goes through torch.distributed (NCCL / gloo).
Plans are cached per (shape, dtype, placement, in, out).
"""
from __future__ import annotations

import logging
from typing import List, Sequence, Tuple

import os

import torch
import torch.distributed as dist

from .balanced_splitter import BalancedSplitter
from .nd_sbp import local_shape, slice_view

log = logging.getLogger("oneflow_b200.boxing")
_PLAN_CACHE = {}
_DEVICE_COLL = {}
debug_routes = False


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def _device_coll(group, ranks, device):
    """In-kernel collectives for a CUDA sub-group (lazily created, needs the native library)."""
    key = tuple(ranks)
    c = _DEVICE_COLL.get(key)
    if c is None:
        from ..comm.symmetric import DeviceCollectives, SymmetricArena
        arena = SymmetricArena(group, ranks, device, 3 * (64 << 20) + (1 << 22))
        c = DeviceCollectives(arena, io_bytes=64 << 20)
        _DEVICE_COLL[key] = c
    return c


# Largest tensor the boxing steps hand to the in-kernel collectives (the exchange region holds 64 MB). As stand-alone calls
# NCCL's collectives measured faster at 8 MB and 64 MB on two B200s (the device collectives copy their input into the arena
# first); ONEFLOW_DEVICE_COLL_MAX_BYTES lowers the limit, 0 sends every boxing collective to NCCL.
_DEVICE_COLL_MAX_BYTES = int(os.environ.get("ONEFLOW_DEVICE_COLL_MAX_BYTES", str(64 << 20)))


def _use_device_coll(t, n, staged_fp32=True):
    """The in-kernel collectives take fp32 / bf16 tensors that fit their exchange region: the input region holds 64 MB;
    the two-shot all-reduce also stages an fp32 copy (``staged_fp32``), reduce-scatter / all-gather / all-to-all do not."""
    if not t.is_cuda or n < 2 or n > 8:
        return False
    if t.dtype not in (torch.float32, torch.bfloat16):
        return False
    from ..ops import _native
    need = t.numel() * (4 if staged_fp32 else t.element_size())
    return _native.kernels_available() and need <= min(64 << 20, _DEVICE_COLL_MAX_BYTES)


# ------------------------------------------------------------------------------------------------ 1-D steps
def _all_gather_uneven(local, dim, group, n, total):
    sp = BalancedSplitter(total, n)
    mx = sp.size(0)
    pad_shape = list(local.shape)
    pad_shape[dim] = mx
    if local.shape[dim] != mx:
        padded = local.new_zeros(pad_shape)
        padded.narrow(dim, 0, local.shape[dim]).copy_(local)
    else:
        padded = local.contiguous()
    parts = [torch.empty_like(padded) for _ in range(n)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p.narrow(dim, 0, sp.size(i)) for i, p in enumerate(parts)], dim)


def s_to_b(local, dim, group, ranks, idx, logical_extent):
    n = len(ranks)
    if n == 1:
        return local
    if dim == 0 and logical_extent % n == 0 and local.numel() % 8 == 0 and local.is_cuda and \
            local.numel() * n * local.element_size() <= (64 << 20) and _use_device_coll(local, n, staged_fp32=False):
        return _device_coll(group, ranks, local.device).all_gather(local.contiguous())
    return _all_gather_uneven(local, dim, group, n, logical_extent)


def p_to_b(local, group, ranks, idx):
    n = len(ranks)
    if n == 1:
        return local
    if local.dtype == torch.bool:
        t = local.to(torch.uint8)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return t.bool()
    if _use_device_coll(local, n):
        return _device_coll(group, ranks, local.device).all_reduce(local.contiguous())
    t = local.clone()
    dist.all_reduce(t, group=group)
    return t


def p_to_s(local, dim, group, ranks, idx):
    n = len(ranks)
    if n == 1:
        return local
    if dim == 0 and local.shape[0] % n == 0 and _use_device_coll(local, n, staged_fp32=False) and (local.numel() // n) % 8 == 0:
        return _device_coll(group, ranks, local.device).reduce_scatter(local.contiguous())
    full = p_to_b(local, group, ranks, idx)
    return b_to_s(full, dim, n, idx)


def b_to_s(local, dim, n, idx):
    b, e = BalancedSplitter(local.shape[dim], n).at(idx)
    return local.narrow(dim, b, e - b).contiguous()


def b_to_p(local, idx):
    return local.clone() if idx == 0 else torch.zeros_like(local)


def s_to_p(local, dim, n, idx, logical_extent):
    shape = list(local.shape)
    shape[dim] = logical_extent
    out = local.new_zeros(shape)
    b, e = BalancedSplitter(logical_extent, n).at(idx)
    out.narrow(dim, b, e - b).copy_(local)
    return out


def s_to_s(local, in_dim, out_dim, group, ranks, idx, logical_shape_axis):
    """S(in_dim) -> S(out_dim) along one mesh axis; logical_shape_axis is the shape seen by this axis."""
    n = len(ranks)
    if n == 1 or in_dim == out_dim:
        return local
    even = logical_shape_axis[in_dim] % n == 0 and logical_shape_axis[out_dim] % n == 0
    if even and _use_device_coll(local, n):
        inner = 1
        for s in logical_shape_axis[max(in_dim, out_dim) + 1:]:
            inner *= s
        if max(in_dim, out_dim) == len(logical_shape_axis) - 1:
            inner = 1
        vec = 16 // local.element_size()
        if inner % vec == 0 and inner > 0 and max(in_dim, out_dim) < len(logical_shape_axis) - 1:
            return _device_coll(group, ranks, local.device).all_to_all(local.contiguous(), in_dim, out_dim, logical_shape_axis)
    if even and local.is_cuda:
        # NCCL all-to-all: send the j-th slice along out_dim to rank j, concatenate what arrives along in_dim
        send = [c.contiguous() for c in local.chunk(n, out_dim)]
        recv = [torch.empty_like(send[0]) for _ in range(n)]
        dist.all_to_all(recv, send, group=group)
        return torch.cat(recv, in_dim)
    full = _all_gather_uneven(local, in_dim, group, n, logical_shape_axis[in_dim])
    return b_to_s(full, out_dim, n, idx)


# ------------------------------------------------------------------------------------------------ planning
def _axis_shape(logical_shape, hierarchy, nd_sbp, coords, axis):
    """Shape of the tensor as seen by mesh axis `axis`: splits by the OTHER axes already applied."""
    other = [s if a != axis else _B for a, s in enumerate(nd_sbp)]
    return local_shape(logical_shape, hierarchy, other, coords)


class _Bsbp:
    kind, axis = "B", -1


_B = _Bsbp()


def _collides(nd_sbp, axis):
    """True when changing mesh axis `axis` cannot be done as a 1-D step on the local shard: an INNER axis (higher
    index) splits the same tensor dimension, so the shard this axis sees is not contiguous in that dimension. Splits of
    the same dimension by OUTER axes are harmless: nested splits apply outermost first, so the inner step works inside
    the outer shard."""
    s = nd_sbp[axis]
    if s.kind != "S":
        return False
    return any(a > axis and o.kind == "S" and o.axis == s.axis for a, o in enumerate(nd_sbp))


def plan(in_nd, out_nd):
    """List of (axis, step_name, in_sbp, out_sbp) for a same-placement conversion, or the string "generic"
    when splits of several mesh axes collide on one tensor dimension."""
    key = (tuple(in_nd), tuple(out_nd))
    cached = _PLAN_CACHE.get(key)
    if cached is not None:
        return cached
    steps = []
    generic = False
    cur = list(in_nd)
    for axis, (a, b) in enumerate(zip(in_nd, out_nd)):
        if a == b:
            continue
        if _collides(cur, axis) or _collides(list(cur[:axis]) + [b] + list(cur[axis + 1:]), axis):
            generic = True
            break
        name = {("P", "B"): "ccl-p-to-b", ("P", "S"): "ccl-p-to-s", ("S", "B"): "ccl-s-to-b", ("S", "S"): "ccl-s-to-s",
                ("B", "S"): "symmetric-b-to-s", ("B", "P"): "symmetric-b-to-p", ("S", "P"): "symmetric-s-to-p"}[(a.kind, b.kind)]
        steps.append((axis, name, a, b))
        cur[axis] = b
    result = "generic" if generic else steps
    _PLAN_CACHE[key] = result
    return result


def _apply_step(local, step, logical_shape, placement, cur_nd, coords):
    axis, name, a, b = step
    me = _rank()
    ranks = placement.axis_ranks(axis, me)
    group = placement.axis_group(axis) if len(ranks) > 1 else None
    idx = coords[axis]
    n = len(ranks)
    shp = _axis_shape(logical_shape, placement.hierarchy, cur_nd, coords, axis)
    if debug_routes:
        log.warning("boxing %s on mesh axis %d: %s -> %s", name, axis, a, b)
    if n > 1 and name.startswith("ccl-"):
        # with ONEFLOW_TIMEOUT_SECONDS set, the ranks first agree (over the control store) that they all run this step
        from . import control_plane
        if control_plane.consistency_timeout() is not None:
            control_plane.check_consistency(ranks, f"{name} {tuple(logical_shape)} {a}->{b} axis {axis}")
    if name == "ccl-p-to-b":
        return p_to_b(local, group, ranks, idx)
    if name == "ccl-p-to-s":
        return p_to_s(local, b.axis, group, ranks, idx)
    if name == "ccl-s-to-b":
        return s_to_b(local, a.axis, group, ranks, idx, shp[a.axis])
    if name == "ccl-s-to-s":
        return s_to_s(local, a.axis, b.axis, group, ranks, idx, shp)
    if name == "symmetric-b-to-s":
        return b_to_s(local, b.axis, n, idx)
    if name == "symmetric-b-to-p":
        return b_to_p(local, idx)
    if name == "symmetric-s-to-p":
        return s_to_p(local, a.axis, n, idx, shp[a.axis])
    raise AssertionError(name)


def to_all_broadcast(local, logical_shape, placement, nd_sbp, coords):
    """generic-nd: bring every mesh axis to B, innermost axis first."""
    cur = list(nd_sbp)
    from .. import sbp as S
    for axis in reversed(range(len(cur))):
        a = cur[axis]
        if a.kind == "B":
            continue
        step = (axis, "ccl-s-to-b" if a.kind == "S" else "ccl-p-to-b", a, S.broadcast)
        local = _apply_step(local, step, logical_shape, placement, cur, coords)
        cur[axis] = S.broadcast
    return local


def from_all_broadcast(full, placement, out_nd, coords):
    """Slice / zero a fully replicated tensor down to out_nd (no traffic)."""
    local = full
    for axis, b in enumerate(out_nd):
        if b.kind == "S":
            local = b_to_s(local, b.axis, placement.hierarchy[axis], coords[axis])
        elif b.kind == "P":
            local = b_to_p(local, coords[axis])
    return local


def convert_same_placement(local, logical_shape, placement, in_nd, out_nd):
    me = _rank()
    coords = placement.coords(me)
    if coords is None:
        return local  # rank outside the placement: placeholder stays a placeholder
    in_nd, out_nd = tuple(in_nd), tuple(out_nd)
    if in_nd == out_nd:
        return local
    p = plan(in_nd, out_nd)
    if p == "generic":
        full = to_all_broadcast(local, logical_shape, placement, in_nd, coords)
        return from_all_broadcast(full, placement, out_nd, coords)
    cur = list(in_nd)
    for step in p:
        local = _apply_step(local, step, logical_shape, placement, cur, coords)
        cur[step[0]] = step[3]
    return local


def convert(local, logical_shape, dtype, in_placement, in_nd, out_placement, out_nd):
    """Full conversion, placements may differ (different ranks, hierarchy or device type).
    Every rank of both placements must call this (SPMD)."""
    me = _rank()
    same_ranks = in_placement.ranks_flat == out_placement.ranks_flat and in_placement.hierarchy == out_placement.hierarchy
    if same_ranks:
        out = convert_same_placement(local, logical_shape, in_placement, in_nd, out_nd)
        if in_placement.type != out_placement.type and out_placement.contains(me):
            out = out.to(out_placement.device())  # cuda-copy-h2d / d2h step
        return out
    in_coords = in_placement.coords(me)
    out_coords = out_placement.coords(me)
    if in_placement.hierarchy == out_placement.hierarchy and tuple(in_nd) == tuple(out_nd):
        # same mesh shape, same layout, other ranks (a pipeline stage boundary): every rank hands its shard to the
        # rank at the same mesh coordinates, nothing is gathered
        return _one_to_one(local, logical_shape, dtype, in_placement, out_placement, in_nd, in_coords, out_coords)
    full = None
    if in_coords is not None:
        full = to_all_broadcast(local, logical_shape, in_placement, in_nd, in_coords)
    # naive-1-to-1 / asymmetric-broadcast: every destination rank that lacks the data receives the full
    # tensor from one source rank (round-robin over the sources)
    src_ranks = list(in_placement.ranks_flat)
    need = [r for r in out_placement.ranks_flat if r not in src_ranks]
    dev_out = out_placement.device() if out_coords is not None else None
    for k, dst in enumerate(need):
        src = src_ranks[k % len(src_ranks)]
        if me == src:
            t = full
            if out_placement.type == "cpu" and t.is_cuda:
                t = t.cpu()
            if out_placement.type == "cuda" and not t.is_cuda and dist.get_backend() == "nccl":
                t = t.to(in_placement.device() if in_placement.type == "cuda" else torch.device("cuda", torch.cuda.current_device()))
            dist.send(t.contiguous(), dst)
        elif me == dst:
            recv_dev = dev_out
            if dist.get_backend() == "gloo":
                recv_dev = torch.device("cpu")
            buf = torch.empty(tuple(logical_shape), dtype=dtype, device=recv_dev)
            dist.recv(buf, src)
            full = buf.to(dev_out)
    if out_coords is None:
        return torch.empty((0,), dtype=dtype, device=local.device if local is not None else "cpu")
    if full.device != dev_out:
        full = full.to(dev_out)
    return from_all_broadcast(full, out_placement, out_nd, out_coords)


_P2P_GROUPS = {}
_P2P_PENDING = []      # (work, tensor) of asynchronous sends still in flight: keeps the buffers alive


def _p2p_group(src, dst):
    """One communicator per ordered rank pair: traffic in the two directions of a pipeline boundary never queues
    behind each other (a send only completes once the peer posted its receive), and it runs on that communicator's
    own stream beside the compute stream. gloo shares the default group."""
    if dist.get_backend() != "nccl":
        return None
    key = (src, dst)
    g = _P2P_GROUPS.get(key)
    if g is None:
        g = dist.new_group(ranks=sorted([src, dst]), use_local_synchronization=True)
        _P2P_GROUPS[key] = g
    return g


def _reap_sends(limit=64):
    if len(_P2P_PENDING) > limit:
        keep = []
        for w, t in _P2P_PENDING:
            if not w.is_completed():
                keep.append((w, t))
        _P2P_PENDING[:] = keep[-4 * limit:]


def _one_to_one(local, logical_shape, dtype, in_pl, out_pl, nd, in_coords, out_coords):
    me = _rank()
    out = None
    if in_coords is not None:
        dst = out_pl.rank_at(in_coords)
        if dst == me:
            out = local
        else:
            t = local.contiguous()
            if out_pl.type == "cuda" and not t.is_cuda and dist.get_backend() == "nccl":
                t = t.to(torch.device("cuda", torch.cuda.current_device()))
            if t.is_cuda and dist.get_backend() == "gloo":
                t = t.cpu()
            if debug_routes:
                log.warning("boxing naive-1-to-1: rank %d -> %d, %s", me, dst, tuple(t.shape))
            w = dist.isend(t, dst, group=_p2p_group(me, dst))
            _P2P_PENDING.append((w, t))
            _reap_sends()
    if out_coords is None:
        return torch.empty((0,), dtype=dtype, device=local.device if local is not None else "cpu")
    if out is None:
        src = in_pl.rank_at(out_coords)
        shape = local_shape(logical_shape, out_pl.hierarchy, nd, out_coords)
        dev = out_pl.device()
        recv_dev = torch.device("cpu") if dist.get_backend() == "gloo" else dev
        buf = torch.empty(tuple(shape), dtype=dtype, device=recv_dev)
        dist.irecv(buf, src, group=_p2p_group(src, me)).wait()
        out = buf.to(dev) if buf.device != dev else buf
    elif out.device != out_pl.device():
        out = out.to(out_pl.device())
    return out


def flush_sends():
    """Waits for the asynchronous stage-boundary sends issued so far (end of a step)."""
    for w, _t in _P2P_PENDING:
        w.wait()
    _P2P_PENDING.clear()


# ``flow.boxing.enable_fusion`` / ``flow.boxing.nccl.*`` (reference: python/oneflow/boxing/__init__.py:16-17)
from . import boxing_nccl as nccl  # noqa: E402,F401
from .config_util import api_enable_fusion as enable_fusion  # noqa: E402,F401
