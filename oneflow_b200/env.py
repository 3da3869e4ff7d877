"""``flow.env``: rank / world queries and process-group bootstrap from MASTER_ADDR / MASTER_PORT /
WORLD_SIZE / RANK / LOCAL_RANK (reference: python/oneflow/env.py:19-93,
python/oneflow/framework/env_util.py:167-192). The control plane is the in-tree control store
(framework/control_plane.py over csrc/core/control_store.cpp): rank 0 hosts it on MASTER_PORT, the process groups
rendezvous through it, every rank heartbeats into it and the rank-consistency check of global-tensor operations
runs over it (``ONEFLOW_CONTROL_STORE=torch`` falls back to torch.distributed's TCPStore). The data plane is gloo for
CPU tensors and NCCL plus the in-tree peer-memory kernels for CUDA tensors."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

_initialized_here = False


def init(backend=None, timeout_seconds=None):
    """Joins the job described by the launcher's environment variables (no-op for a single process)."""
    global _initialized_here
    if dist.is_initialized():
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1 and "RANK" not in os.environ:
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
    timeout = datetime.timedelta(seconds=timeout_seconds or int(os.environ.get("ONEFLOW_TIMEOUT_SECONDS", "7200")))
    kwargs = {}
    if torch.cuda.is_available():
        torch.cuda.set_device(get_local_rank())
    rank = int(os.environ.get("RANK", "0"))
    from .ops import _native
    native = os.environ.get("ONEFLOW_CONTROL_STORE", "native") != "torch" and _native.core_available()
    elastic = "TORCHELASTIC_RUN_ID" in os.environ
    if native and not torch.cuda.is_available() and not elastic:
        # CPU job started by this package's launcher: the control store IS the rendezvous of every process group
        from .framework import control_plane
        store = control_plane.start(rank, world, os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]),
                                    timeout_s=min(timeout.total_seconds(), 1800.0))
        dist.init_process_group(backend, timeout=timeout, store=store, rank=rank, world_size=world, **kwargs)
    else:
        # NCCL's communicator bootstrap calls store methods that a store implemented outside torch cannot provide,
        # and torch.distributed.run already serves a store on MASTER_PORT: the process groups use torch's store, the
        # control store (heartbeats, consistency check, barriers) takes a free port that rank 0 announces
        dist.init_process_group(backend, timeout=timeout, **kwargs)
        if native:
            from .framework import control_plane
            port = [0]
            if rank == 0:
                from .runtime.core import ControlServer
                control_plane._server = ControlServer(world, 0)
                port[0] = control_plane._server.port
            dist.broadcast_object_list(port, src=0)
            control_plane.start(rank, world, os.environ["MASTER_ADDR"], int(port[0]), timeout_s=min(timeout.total_seconds(), 1800.0))
    _initialized_here = True


def get_rank():
    return dist.get_rank() if dist.is_initialized() else int(os.environ.get("RANK", "0"))


def get_world_size():
    return dist.get_world_size() if dist.is_initialized() else int(os.environ.get("WORLD_SIZE", "1"))


def get_local_rank():
    return int(os.environ.get("LOCAL_RANK", "0"))


def get_node_size():
    local = int(os.environ.get("LOCAL_WORLD_SIZE", str(get_world_size())))
    return max(1, get_world_size() // max(local, 1))


def is_multi_client():
    return True


def init_rdma():
    """Kept for API compatibility: intra-node traffic uses NVLink peer memory, there is no RDMA path."""
    return None


def destory_rdma():
    """Counterpart of :func:`init_rdma` under the reference's (misspelt) name; nothing to tear down."""
    return None


destroy_rdma = destory_rdma


def rdma_is_initialized():
    return False


def all_device_placement(device_type):
    from .framework.placement import placement
    return placement.all(device_type)


def lost_ranks(max_age_seconds=5.0):
    """Ranks whose heartbeat into the control store is overdue (host-side failure detection)."""
    from .framework import control_plane
    return control_plane.lost_ranks(max_age_seconds)


def shutdown():
    global _initialized_here
    if dist.is_initialized() and _initialized_here:
        dist.destroy_process_group()
        _initialized_here = False
    from .framework import control_plane
    control_plane.shutdown()
