"""``flow.distributed``: the launcher (``python -m oneflow_b200.distributed.launch``), rank helpers, and the
torch.distributed-shaped collective entry points, which forward to :mod:`oneflow_b200.comm`
(reference: python/oneflow/distributed/__init__.py:24-200 — SUM only, default group only, synchronous only)."""
import datetime

from .. import comm as _comm
from ..env import get_local_rank  # noqa: F401
from .. import env as _env

default_pg_timeout = datetime.timedelta(minutes=30)


class ReduceOp:
    SUM = "sum"


def _only_default(group, async_op=False):
    if group is not None:
        raise NotImplementedError("only the default group is supported")
    if async_op:
        raise NotImplementedError("async_op is not supported")


def is_available():
    return True


def is_initialized():
    return True


def get_rank(group=None):
    _only_default(group)
    return _env.get_rank()


def get_world_size(group=None):
    _only_default(group)
    return _env.get_world_size()


def send(tensor, dst, group=None, tag=0):
    _only_default(group)
    assert tag == 0, "tag is not supported"
    return _comm.send(tensor, dst)


def recv(tensor, src, group=None, tag=0):
    _only_default(group)
    assert tag == 0, "tag is not supported"
    return _comm.recv(src, out=tensor)


def broadcast(tensor, src, group=None, async_op=False):
    _only_default(group, async_op)
    return _comm.broadcast(tensor, src)


def barrier(group=None, async_op=False, device_ids=None):
    _only_default(group, async_op)
    return _comm.barrier()


def _sum_only(op):
    if op not in (ReduceOp.SUM, None) and str(op).lower() not in ("sum", "reduceop.sum", "redoptype.sum"):
        raise NotImplementedError("only ReduceOp.SUM is supported")


def all_reduce(tensor, op=ReduceOp.SUM, group=None, async_op=False):
    _sum_only(op)
    _only_default(group, async_op)
    return _comm.all_reduce(tensor)


def all_gather(tensor_list, tensor, group=None, async_op=False):
    _only_default(group, async_op)
    return _comm.all_gather(tensor_list, tensor)


def reduce(tensor, dst, op=ReduceOp.SUM, group=None, async_op=False):
    _sum_only(op)
    _only_default(group, async_op)
    return _comm.reduce(tensor, dst)


def all_to_all(output_tensor_list, input_tensor_list, group=None, async_op=False):
    _only_default(group, async_op)
    return _comm.all_to_all(output_tensor_list, input_tensor_list)


def reduce_scatter(output, input_list, op=ReduceOp.SUM, group=None, async_op=False):
    _sum_only(op)
    _only_default(group, async_op)
    return _comm.reduce_scatter(output, input_list)


def gather(tensor, gather_list=None, dst=0, group=None, async_op=False):
    _only_default(group, async_op)
    return _comm.gather(tensor, gather_list, dst)
