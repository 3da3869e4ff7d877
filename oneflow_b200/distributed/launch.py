"""``python -m oneflow.distributed.launch --nproc_per_node N [--nnodes M --node_rank R --master_addr A
--master_port P] script.py args...``

Starts one process per local rank with MASTER_ADDR / MASTER_PORT / WORLD_SIZE / RANK / LOCAL_RANK set,
``OMP_NUM_THREADS=1`` by default when several ranks share a node, and per-rank log directories when
``--logdir`` is given. The first rank that exits non-zero takes the whole process group down, so a failed
rank never leaves its peers waiting on a collective.
Reference: python/oneflow/distributed/launch.py:28-222.
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="oneflow_b200 distributed launcher")
    p.add_argument("--nnodes", type=int, default=1)
    p.add_argument("--node_rank", type=int, default=0)
    p.add_argument("--nproc_per_node", type=int, default=1)
    p.add_argument("--master_addr", default="127.0.0.1")
    p.add_argument("--master_port", type=int, default=29500)
    p.add_argument("-m", "--module", action="store_true", help="run the script as a python module")
    p.add_argument("--no_python", action="store_true")
    p.add_argument("--redirect_stdout_and_stderr", action="store_true")
    p.add_argument("--logdir", default="log")
    p.add_argument("training_script")
    p.add_argument("training_script_args", nargs=argparse.REMAINDER)
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    world = args.nnodes * args.nproc_per_node
    base_env = os.environ.copy()
    base_env["MASTER_ADDR"] = args.master_addr
    base_env["MASTER_PORT"] = str(args.master_port)
    base_env["WORLD_SIZE"] = str(world)
    base_env["LOCAL_WORLD_SIZE"] = str(args.nproc_per_node)
    if "OMP_NUM_THREADS" not in os.environ and args.nproc_per_node > 1:
        base_env["OMP_NUM_THREADS"] = "1"
    procs = []
    for local_rank in range(args.nproc_per_node):
        env = dict(base_env)
        env["RANK"] = str(args.nproc_per_node * args.node_rank + local_rank)
        env["LOCAL_RANK"] = str(local_rank)
        cmd = [] if args.no_python else [sys.executable, "-u"]
        if args.module and not args.no_python:
            cmd.append("-m")
        cmd += [args.training_script] + args.training_script_args
        out = err = None
        if args.redirect_stdout_and_stderr:
            d = os.path.join(args.logdir, f"local_rank_{local_rank}")
            os.makedirs(d, exist_ok=True)
            env["GLOG_log_dir"] = d
            out, err = open(os.path.join(d, "stdout"), "w"), open(os.path.join(d, "stderr"), "w")
        procs.append(subprocess.Popen(cmd, env=env, stdout=out, stderr=err, start_new_session=True))

    def kill_all(sig=signal.SIGTERM):
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, sig)
                except ProcessLookupError:
                    pass

    def on_signal(signum, frame):
        kill_all(signal.SIGTERM)
        sys.exit(128 + signum)
    signal.signal(signal.SIGINT, on_signal)
    signal.signal(signal.SIGTERM, on_signal)

    rc = 0
    alive = set(range(len(procs)))
    while alive:
        for i in list(alive):
            r = procs[i].poll()
            if r is None:
                continue
            alive.discard(i)
            if r != 0 and rc == 0:
                rc = r
                kill_all(signal.SIGTERM)
                time.sleep(1.0)
                kill_all(signal.SIGKILL)
        time.sleep(0.05)
    if rc != 0:
        raise subprocess.CalledProcessError(returncode=rc, cmd=" ".join([args.training_script] + args.training_script_args))
    return 0


if __name__ == "__main__":
    sys.exit(main())
