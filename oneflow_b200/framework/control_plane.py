"""The job's control plane on the in-tree control store (csrc/core/control_store.cpp): rendezvous, barriers,
heartbeats and the rank-consistency check.

The reference bootstraps every rank against a key-value service (CtrlServer / CtrlClient over gRPC,
oneflow/core/control/ctrl_client.cpp:37-58): collective communicators exchange their ids through it
(oneflow/core/job/eager_nccl_comm_manager.cpp:54-80), barriers and the liveness of ranks run over it. Here rank 0
hosts the store on MASTER_PORT, every rank connects a client, and

* ``ControlStore`` presents that client as a ``torch.distributed.Store``, so process-group creation (the NCCL /
  gloo rendezvous of this job and of every sub-group) reads and writes this store, not torch's TCPStore;
* every client sends heartbeats; ``lost_ranks()`` names ranks whose heartbeat is overdue (failure detection on the
  host, no GPU involved);
* ``check_consistency(group ranks, signature)`` is called by the boxing layer before a step that communicates, when
  ``ONEFLOW_TIMEOUT_SECONDS`` is set: every rank of the group publishes what it is about to run under a per-group
  sequence number and reads its peers' entries. A peer that publishes something else, or nothing within the time
  limit (it took another branch and never reached this global-tensor operation), raises an error on the ranks that
  wait -- instead of a collective that blocks until the process-group time-out. Reference: the meta consistency
  check on transport tokens (oneflow/core/framework/consistency_check.cpp, tensor_rpc_util.cpp).
"""
from __future__ import annotations

import datetime
import os
import time

import torch.distributed as dist

_server = None
_client = None
_seq = {}
_epoch = [0]

DIVERGED = ("Maybe executing different code in different ranks, please check if the code is branched and operates on the "
            "global tensor")


class ControlStore(dist.Store):
    """``torch.distributed.Store`` over a ``runtime.ControlClient``."""

    # torch keeps only the C++ half of a store it is handed; were the Python half collected, every call back into these
    # methods would fail as "not implemented". Every instance therefore stays referenced for the life of the process.
    _alive = []

    def __init__(self, client, timeout_s=300.0):
        super().__init__()
        self.c = client
        self._timeout_s = float(timeout_s)
        ControlStore._alive.append(self)

    def set(self, key, value):
        if isinstance(value, str):
            value = value.encode()
        self.c.set(key, bytes(value))

    def get(self, key):
        from ..runtime.core import CoreError
        try:
            return self.c.get(key, timeout_s=self._timeout_s)
        except (CoreError, TimeoutError) as e:
            raise RuntimeError(f"control store: no value for key {key!r} within {self._timeout_s} s ({e})") from None

    def add(self, key, amount):
        return int(self.c.add(key, int(amount)))

    def compare_set(self, key, expected, desired):
        to_b = lambda v: v.encode() if isinstance(v, str) else bytes(v)  # noqa: E731
        return self.c.compare_set(key, to_b(expected), to_b(desired))

    def delete_key(self, key):
        return self.c.delete(key)

    def num_keys(self):
        return int(self.c.num_keys())

    def check(self, keys):
        return all(self.c.has(k) for k in keys)

    def wait(self, keys, timeout=None):
        limit = timeout.total_seconds() if isinstance(timeout, datetime.timedelta) else self._timeout_s
        deadline = time.monotonic() + limit
        for k in keys:
            while not self.c.has(k):
                if time.monotonic() > deadline:
                    raise RuntimeError(f"control store: timed out after {limit} s waiting for key {k!r}")
                time.sleep(0.002)

    def set_timeout(self, timeout):
        self._timeout_s = timeout.total_seconds() if isinstance(timeout, datetime.timedelta) else float(timeout)

    # the extended interface newer process-group constructors ask for
    def clone(self):
        return ControlStore(self.c, self._timeout_s)

    def has_extended_api(self):
        return True

    def append(self, key, value):
        if isinstance(value, str):
            value = value.encode()
        while True:       # read-modify-write through compare-and-set: concurrent appends never lose a piece
            old = self.c.get(key, timeout_s=self._timeout_s) if self.c.has(key) else b""
            if self.c.compare_set(key, old, old + bytes(value)) == old + bytes(value):
                return

    def multi_get(self, keys):
        return [self.get(k) for k in keys]

    def multi_set(self, keys, values):
        for k, v in zip(keys, values):
            self.set(k, v)

    @property
    def timeout(self):
        return datetime.timedelta(seconds=self._timeout_s)


def start(rank, world, host, port, timeout_s=300.0, heartbeat_s=1.0):
    """Rank 0 hosts the store on ``port``; every rank connects. Returns a ``ControlStore`` for ``init_process_group``."""
    global _server, _client
    from ..runtime.core import ControlClient, ControlServer
    if _client is not None:
        return ControlStore(_client, timeout_s)
    if host in ("localhost", ""):
        host = "127.0.0.1"
    if rank == 0 and _server is None:
        _server = ControlServer(world, port)
    _client = ControlClient(host, port, rank, timeout_s=timeout_s)
    if heartbeat_s:
        _client.start_heartbeat(heartbeat_s)
    return ControlStore(_client, timeout_s)


def client():
    return _client


def lost_ranks(max_age_s=5.0):
    """Ranks whose heartbeat is older than ``max_age_s`` (empty without a control plane)."""
    return _client.lost_ranks(max_age_s) if _client is not None else []


def barrier(name, world, timeout_s=None):
    if _client is None:
        return dist.barrier()
    from ..runtime.core import CoreError
    try:
        _client.barrier(name, world, timeout_s if timeout_s is not None else consistency_timeout() or 300.0)
    except (CoreError, TimeoutError) as e:
        raise RuntimeError(f"{e}. {DIVERGED}") from None


def consistency_timeout():
    """Seconds of ``ONEFLOW_TIMEOUT_SECONDS`` when the consistency check is on, else None."""
    v = os.environ.get("ONEFLOW_TIMEOUT_SECONDS")
    if not v or _client is None:
        return None
    try:
        t = float(v)
    except ValueError:
        return None
    return t if 0 < t < 3600 else None


def check_consistency(ranks, signature: str):
    """Every rank of ``ranks`` must call this with the same ``signature`` in the same order."""
    limit = consistency_timeout()
    if limit is None or len(ranks) < 2:
        return
    from ..runtime.core import CoreError
    me = dist.get_rank()
    key = ",".join(str(r) for r in ranks)
    n = _seq.get(key, 0) + 1
    _seq[key] = n
    base = f"cc/{_epoch[0]}/{key}/{n}"
    _client.set(f"{base}/{me}", signature.encode())
    for r in ranks:
        if r == me:
            continue
        try:
            other = _client.get(f"{base}/{r}", timeout_s=limit).decode()
        except (CoreError, TimeoutError):
            lost = lost_ranks(max(2.0, limit))
            raise RuntimeError(f"rank {r} did not reach global-tensor operation #{n} of group [{key}] ({signature}) within "
                               f"{limit} s{' (its heartbeat is overdue: the rank may be gone)' if r in lost else ''}. {DIVERGED}") from None
        if other != signature:
            raise RuntimeError(f"global-tensor operation #{n} of group [{key}] differs between ranks: rank {me} runs {signature}, "
                               f"rank {r} runs {other}. {DIVERGED}")
    if n > 2:
        _client.delete(f"cc/{_epoch[0]}/{key}/{n - 2}/{me}")


def resync():
    """After a reported divergence the ranks' operation counters no longer agree. A job that catches the error and goes
    on calls this on every rank at a common point (after a barrier): counting restarts under a new epoch."""
    _epoch[0] += 1
    _seq.clear()


def shutdown():
    global _server, _client
    if _client is not None:
        _client.close()
        _client = None
    if _server is not None:
        _server.stop()
        _server = None
