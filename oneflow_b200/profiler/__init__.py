"""``flow.profiler``: ``profile(activities, record_shapes, record_attrs, record_bandwidth_for_cuda)``, ``record_function`` and
``key_averages().table()`` in the reference's layout, NVTX ranges for device timelines and a CUDA-event kernel timer.

Two sources feed one event list while a ``profile`` is active:
  * every call into the native kernel library (``ops/_native.py`` hands out a wrapper of the library) is bracketed with CUDA
    events on the launching stream and a host timer; the tensors whose pointers the call received give the input shapes and
    the bytes for the bandwidth column (bytes of all operands / device time: what the reference reports with
    ``record_bandwidth_for_cuda``), GEMM calls add their FLOPs;
  * every ATen operator that runs (``TorchDispatchMode``) is recorded the same way, so the ops that stay in PyTorch appear in
    the same table.
``record_function`` ranges are custom events that own the kernel events launched inside them.

Reference: python/oneflow/profiler/profiler.py:42-117 (profile), python/oneflow/profiler/events.py:285-375 (key_averages and
the table), oneflow/core/profiler/{profiler.cpp,event.cpp,kineto_shim.cpp} (CPU / CUDA events, bandwidth from memory size)."""
import contextlib
import time
from collections import OrderedDict
from enum import Enum

import torch
from torch.profiler import ProfilerAction, tensorboard_trace_handler  # noqa: F401
from torch.utils._python_dispatch import TorchDispatchMode


class ProfilerActivity(Enum):
    CPU = 1
    CUDA = 2


def supported_activities():
    acts = {ProfilerActivity.CPU}
    if torch.cuda.is_available():
        acts.add(ProfilerActivity.CUDA)
    return acts


def _fmt_time(us):
    if us is None:
        return "-"
    if us >= 1e6:
        return f"{us / 1e6:.3f}s"
    if us >= 1e3:
        return f"{us / 1e3:.3f}ms"
    return f"{us:.3f}us"


class Event:
    """One row: a kernel (native or ATen) or a ``record_function`` range. Times in microseconds."""

    def __init__(self, name, kind, cpu_us, cuda_pair=None, shapes="", attrs="", nbytes=0, flops=0.0):
        self.name, self.kind = name, kind              # kind: "kernel" | "custom"
        self.cpu_time_total = float(cpu_us)
        self._cuda_pair = cuda_pair                    # (start event, end event) until resolved
        self.cuda_time_total = None
        self.count = 1
        self.input_shapes, self.attributes = shapes, attrs
        self.nbytes, self.flops = int(nbytes), float(flops)
        self.children = []

    def _resolve(self):
        if self._cuda_pair is not None:
            a, b = self._cuda_pair
            self.cuda_time_total = a.elapsed_time(b) * 1e3
            self._cuda_pair = None
        for c in self.children:
            c._resolve()

    @property
    def cpu_time(self):
        return self.cpu_time_total / self.count

    @property
    def cuda_time(self):
        return None if self.cuda_time_total is None else self.cuda_time_total / self.count

    @property
    def bandwidth(self):
        """GB/s over the device time of all calls, or None without a device time or bytes."""
        if not self.cuda_time_total or not self.nbytes:
            return None
        return self.nbytes / (self.cuda_time_total * 1e-6) / 1e9

    def key(self, by_shape, by_attr):
        return (self.name, self.kind, self.input_shapes if by_shape else "", self.attributes if by_attr else "")

    def update(self, other):
        self.cpu_time_total += other.cpu_time_total
        if other.cuda_time_total is not None:
            self.cuda_time_total = (self.cuda_time_total or 0.0) + other.cuda_time_total
        self.count += other.count
        self.nbytes += other.nbytes
        self.flops += other.flops

    def to_dict(self):
        bw = self.bandwidth
        return {"name": self.name, "cpu_time_total": _fmt_time(self.cpu_time_total), "cpu_time": _fmt_time(self.cpu_time),
                "cuda_time_total": _fmt_time(self.cuda_time_total), "cuda_time": _fmt_time(self.cuda_time), "count": self.count,
                "input_shapes": self.input_shapes or "-", "attributes": self.attributes or "-",
                "bandwidth": f"{bw:.3f}GB/s" if bw is not None else "-"}


class Events(list):
    def key_averages(self, group_by_input_shape=False, group_by_attributes=False):
        stats = OrderedDict()

        def deal(e):
            k = e.key(group_by_input_shape, group_by_attributes)
            if k in stats:
                stats[k].update(e)
            else:
                c = Event(e.name, e.kind, e.cpu_time_total, None, e.input_shapes if group_by_input_shape else "",
                          e.attributes if group_by_attributes else "", e.nbytes, e.flops)
                c.cuda_time_total, c.count = e.cuda_time_total, e.count
                stats[k] = c

        for e in self:
            for c in e.children:
                deal(c)
            deal(e)
        out = Events(stats.values())
        out._show = (group_by_input_shape, group_by_attributes)
        return out

    def table(self):
        show_shapes, show_attrs = getattr(self, "_show", (False, False))
        show_shapes = show_shapes and any(e.input_shapes for e in self)
        show_attrs = show_attrs and any(e.attributes for e in self)
        show_bw = any(e.bandwidth is not None for e in self)
        cols = [("Name", "name"), ("CPU time total", "cpu_time_total"), ("CPU time", "cpu_time"), ("GPU time total", "cuda_time_total"),
                ("GPU time", "cuda_time"), ("Number of calls", "count")]
        if show_shapes:
            cols.append(("Input shapes", "input_shapes"))
        if show_attrs:
            cols.append(("Attributes", "attributes"))
        if show_bw:
            cols.append(("Bandwidth", "bandwidth"))
        rows = [[str(e.to_dict()[k]) for _, k in cols] for e in self]
        widths = [max(len(h), *(len(r[i]) for r in rows)) if rows else len(h) for i, (h, _) in enumerate(cols)]
        line = lambda cells: "  ".join(c.ljust(w) for c, w in zip(cells, widths)).rstrip()  # noqa: E731
        out = [line([h for h, _ in cols]), line(["-" * w for w in widths])]
        out += [line(r) for r in rows]
        return "\n".join(out) + "\n"

    def __str__(self):
        return self.table()


def _shapes_of(tensors):
    return "[" + ", ".join("(" + ",".join(str(int(d)) for d in t.shape) + ")" for t in tensors) + "]"


class _Recorder(TorchDispatchMode):
    def __init__(self, use_cuda, record_shapes, record_attrs, record_bandwidth):
        super().__init__()
        self.use_cuda, self.record_shapes, self.record_attrs, self.record_bandwidth = use_cuda, record_shapes, record_attrs, record_bandwidth
        self.events = Events()
        self.stack = []                 # open record_function ranges
        self._pending, self._note = [], {}

    # ---- called from ops/_native.py
    def saw_tensor(self, t):
        self._pending.append(t)

    def note(self, flops=0.0, attrs=""):
        self._note = {"flops": flops, "attrs": attrs}

    def _pair(self):
        if not self.use_cuda:
            return None
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def _add(self, ev):
        (self.stack[-1].children if self.stack else self.events).append(ev)

    def native_call(self, name, fn, args):
        tensors, self._pending = self._pending, []
        note, self._note = self._note, {}
        pair = self._pair()
        if pair:
            pair[0].record()
        t0 = time.perf_counter()
        rc = fn(*args)
        cpu_us = (time.perf_counter() - t0) * 1e6
        if pair:
            pair[1].record()
        nbytes = sum(t.numel() * t.element_size() for t in tensors) if self.record_bandwidth else 0
        self._add(Event(name[4:] if name.startswith("ofb_") else name, "kernel", cpu_us, pair,
                        _shapes_of(tensors) if self.record_shapes else "", note.get("attrs", "") if self.record_attrs else "", nbytes,
                        note.get("flops", 0.0)))
        return rc

    # ---- ATen operators
    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        name = getattr(func, "__name__", None) or str(func)
        pkt = getattr(func, "overloadpacket", None)
        name = f"aten::{pkt.__name__}" if pkt is not None else name
        flat = [a for a in args if torch.is_tensor(a)]
        for a in args:
            if isinstance(a, (list, tuple)):
                flat += [x for x in a if torch.is_tensor(x)]
        on_cuda = self.use_cuda and any(t.is_cuda for t in flat)
        pair = self._pair() if on_cuda else None
        if pair:
            pair[0].record()
        t0 = time.perf_counter()
        out = func(*args, **kwargs)
        cpu_us = (time.perf_counter() - t0) * 1e6
        if pair:
            pair[1].record()
        nbytes = 0
        if self.record_bandwidth and pair:
            outs = [o for o in (out if isinstance(out, (list, tuple)) else (out,)) if torch.is_tensor(o)]
            nbytes = sum(t.numel() * t.element_size() for t in flat + outs)
        attrs = ""
        if self.record_attrs:
            attrs = ", ".join(repr(a) for a in args if isinstance(a, (int, float, bool, str)))
        self._add(Event(name, "kernel", cpu_us, pair, _shapes_of(flat) if self.record_shapes else "", attrs, nbytes))
        return out

    # ---- record_function
    def open_range(self, name):
        ev = Event(name, "custom", 0.0, self._pair())
        ev._t0 = time.perf_counter()
        if ev._cuda_pair:
            ev._cuda_pair[0].record()
        self.stack.append(ev)
        return ev

    def close_range(self, ev):
        if not self.stack or self.stack[-1] is not ev:
            raise RuntimeError("record_function ranges must be closed in the order they were opened")
        self.stack.pop()
        ev.cpu_time_total = (time.perf_counter() - ev._t0) * 1e6
        if ev._cuda_pair:
            ev._cuda_pair[1].record()
        self._add(ev)


_active = None


class profile:
    """``with flow.profiler.profile(record_shapes=True, record_bandwidth_for_cuda=True) as prof: ...`` then
    ``print(prof.key_averages(group_by_input_shape=True).table())``."""

    def __init__(self, activities=None, record_shapes=False, record_attrs=False, record_bandwidth_for_cuda=False):
        acts = set(activities) if activities else supported_activities()
        acts = {ProfilerActivity[a.name] if not isinstance(a, ProfilerActivity) else a for a in acts}     # torch's enum is accepted too
        if not acts:
            raise AssertionError("At least one ProfilerActivity must be specified.")
        for a in acts:
            if a not in supported_activities():
                raise AssertionError(f"Unsupported ProfilerActivity {a}")
        if record_bandwidth_for_cuda and ProfilerActivity.CUDA not in acts:
            raise AssertionError("record_bandwidth_for_cuda = True can only work with cuda.")
        self.activities = acts
        self.record_shapes, self.record_attrs, self.record_bandwidth_for_cuda = record_shapes, record_attrs, record_bandwidth_for_cuda
        self.profile_events = None
        self._rec = None

    def __enter__(self):
        global _active
        if _active is not None:
            raise RuntimeError("a profiler is already running")
        from ..ops import _native
        self._rec = _Recorder(ProfilerActivity.CUDA in self.activities, self.record_shapes, self.record_attrs, self.record_bandwidth_for_cuda)
        _active = self._rec
        _native.set_recorder(self._rec)
        self._rec.__enter__()
        return self

    def __exit__(self, *exc):
        global _active
        from ..ops import _native
        self._rec.__exit__(*exc)
        _native.set_recorder(None)
        _active = None
        if self._rec.use_cuda:
            torch.cuda.synchronize()
        for e in self._rec.events:
            e._resolve()
        self.profile_events = self._rec.events
        return False

    def _check(self):
        if self.profile_events is None:
            raise RuntimeError("Profiler didn't finish running")

    def key_averages(self, group_by_input_shape=False, group_by_attributes=False):
        self._check()
        return self.profile_events.key_averages(group_by_input_shape, group_by_attributes)

    def events(self):
        self._check()
        return self.profile_events


class record_function:
    """A named range: the kernels launched inside it are listed under it; outside a profiler it is only an NVTX range."""

    def __init__(self, name):
        self.name, self._ev = name, None

    def __enter__(self):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        if _active is not None:
            self._ev = _active.open_range(self.name)
        return self

    def __exit__(self, *exc):
        if self._ev is not None and _active is not None:
            _active.close_range(self._ev)
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


@contextlib.contextmanager
def nvtx_range(name):
    """Device-timeline range (the reference's nvtx_start / nvtx_end ops, user/kernels/nvtx_range_kernel.cu)."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class CudaTimer:
    """CUDA-event timing on the current stream: ``with CudaTimer() as t: ...; t.ms``."""

    def __enter__(self):
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self.e0.record()
        return self

    def __exit__(self, *exc):
        self.e1.record()
        torch.cuda.synchronize()
        self.ms = self.e0.elapsed_time(self.e1)
        return False


def range_push(range_name):
    """Open an NVTX range on the calling thread (reference: python/oneflow/profiler/__init__.py:40-45)."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(range_name)


def range_pop():
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def profiler_start():
    """Start the CUDA profiler's capture window (``cudaProfilerStart``), for tools run with a capture range."""
    if torch.cuda.is_available():
        torch.cuda.profiler.start()


def profiler_stop():
    if torch.cuda.is_available():
        torch.cuda.profiler.stop()


def kineto_available():
    return torch.autograd.kineto_available()
