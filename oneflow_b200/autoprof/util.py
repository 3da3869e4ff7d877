"""Profiling of whole scripts into a CSV table (reference: python/oneflow/autoprof/util.py)."""
from __future__ import annotations

import csv
import runpy

FIELDS = ["script", "op", "kind", "count", "cpu_time_us", "cuda_time_us", "bytes", "bandwidth_gbs", "flops", "input_shapes"]


def profile_script(path, activities=None):
    """Runs ``path`` as ``__main__`` under the profiler; returns the averaged events."""
    import torch
    from .. import profiler as P
    acts = activities or ([P.ProfilerActivity.CPU, P.ProfilerActivity.CUDA] if torch.cuda.is_available() else [P.ProfilerActivity.CPU])
    with P.profile(activities=acts, record_shapes=True, record_bandwidth_for_cuda=P.ProfilerActivity.CUDA in acts) as prof:
        runpy.run_path(path, run_name="__main__")
    return prof.key_averages(group_by_input_shape=True)


def write_csv(rows, filename):
    """``rows``: (script, averaged event) pairs."""
    with open(filename, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(FIELDS)
        for script, ev in rows:
            cuda = ev.cuda_time_total
            bw = (ev.nbytes / (cuda * 1e-6) / 1e9) if cuda and ev.nbytes else ""
            w.writerow([script, ev.name, ev.kind, ev.count, f"{ev.cpu_time_total:.1f}", "" if cuda is None else f"{cuda:.1f}", ev.nbytes or "",
                        f"{bw:.1f}" if bw != "" else "", ev.flops or "", ev.input_shapes or ""])
    return filename


def print_summary_from_csv(filename, top=20):
    with open(filename, newline="") as f:
        rows = list(csv.DictReader(f))
    key = lambda r: float(r["cuda_time_us"] or r["cpu_time_us"] or 0.0)
    rows.sort(key=key, reverse=True)
    total = sum(key(r) for r in rows) or 1.0
    print(f"{'op':40s} {'count':>7s} {'time us':>12s} {'share':>7s} {'GB/s':>8s}")
    for r in rows[:top]:
        print(f"{r['op'][:40]:40s} {r['count']:>7s} {key(r):12.1f} {100 * key(r) / total:6.1f}% {r['bandwidth_gbs']:>8s}")
    print(f"{len(rows)} operators, {total:.1f} us in total ({filename})")
