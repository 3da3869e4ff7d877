"""Symmetric (peer-mapped) device memory and the in-kernel collectives built on it.

One ``SymmetricArena`` per process group: every rank cudaMalloc's an arena, the CUDA IPC handles
travel through the group's store (``all_gather_object``), and every rank maps all peers. Kernels
in ``csrc/comm`` then read / write peer memory over NVLink directly. This module also exposes the
stand-alone collectives (all-reduce, reduce-scatter, all-gather, all-to-all, each fused with a cast
and scale) that the SBP boxing layer uses on CUDA tensors; NCCL is not involved.

The role of the reference's EagerCclCommMgr + ccl::AllReduce/AllGather/... primitives
(oneflow/core/job/eager_nccl_comm_manager.cpp:54-80,
oneflow/user/kernels/collective_communication/include/collective_communication.h:55-84).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_ubyte, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..ops import _native
from ..ops import kernels as _k

_SIGNAL_BYTES = 4096
_DT = {torch.float32: 0, torch.bfloat16: 1}


class CommCtxStruct(Structure):
    _fields_ = [("rank", c_int), ("n", c_int), ("arena", c_void_p * 8), ("signals", c_void_p * 8)]


class _DevMem:
    """Exposes a raw device range to torch through __cuda_array_interface__ (zero copy)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _align(n, a=4096):
    return (n + a - 1) // a * a


class SymmetricArena:
    def __init__(self, group, ranks, device, nbytes):
        lib = _native.kernels()
        self.group, self.ranks, self.device = group, list(ranks), torch.device(device)
        self.n = len(self.ranks)
        self.rank = self.ranks.index(dist.get_rank()) if dist.is_initialized() and self.n > 1 else 0
        self.nbytes = _align(int(nbytes) + _SIGNAL_BYTES, 1 << 21)
        ptr = c_void_p()
        handle = (c_ubyte * 64)()
        with torch.cuda.device(self.device):
            _native.check(lib.ofb_symm_alloc(c_longlong(self.nbytes), ctypes.byref(ptr), handle), "symm_alloc")
        self.local_ptr = ptr.value
        handles = [None] * self.n
        if self.n > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        else:
            handles = [bytes(handle)]
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            p = c_void_p()
            buf = (c_ubyte * 64).from_buffer_copy(h)
            with torch.cuda.device(self.device):
                _native.check(lib.ofb_symm_open(buf, ctypes.byref(p)), "symm_open")
            self.ptrs.append(p.value)
        self._cursor = _SIGNAL_BYTES  # the first page of every arena is the SignalBlock
        self.ctx = CommCtxStruct()
        self.ctx.rank, self.ctx.n = self.rank, self.n
        for i in range(8):
            self.ctx.arena[i] = self.ptrs[i] if i < self.n else None
            self.ctx.signals[i] = self.ptrs[i] if i < self.n else None
        self._torch_view = torch.as_tensor(_DevMem(self.local_ptr, self.nbytes), device=self.device)
        if self.n > 1:
            dist.barrier(group=group)

    def region(self, nbytes, align=4096):
        """Reserves the same byte range in every rank's arena; returns its offset."""
        off = _align(self._cursor, align)
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted ({off + nbytes} > {self.nbytes} bytes)")
        self._cursor = off + nbytes
        return off

    def view(self, off, shape, dtype):
        """A torch tensor over this rank's copy of a region."""
        n = int(torch.tensor(shape).prod().item()) if len(shape) else 1
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self._torch_view[off:off + nbytes].view(dtype).view(shape)

    def close(self):
        lib = _native.kernels()
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                lib.ofb_symm_close(c_void_p(p))
        lib.ofb_symm_free(c_void_p(self.local_ptr))
        self.ptrs = []


class DeviceCollectives:
    """all_reduce / reduce_scatter / all_gather / all_to_all over a SymmetricArena, each one kernel with the
    cast and scale fused. Inputs are staged into the arena by a device copy (``stage`` may also be written
    in place by the producer through ``input_view``)."""

    def __init__(self, arena: SymmetricArena, io_bytes=64 << 20, ctas=64):
        self.arena = arena
        self.io_bytes = io_bytes
        self.in_off = arena.region(io_bytes)
        self.stage_off = arena.region(2 * io_bytes)  # fp32 staging of the two-shot all-reduce
        self.epoch = 0
        self.ctas = ctas

    def input_view(self, shape, dtype):
        return self.arena.view(self.in_off, shape, dtype)

    def _run(self, mode, x, out, count, scale, staged):
        a = self.arena
        esz = x.element_size() if x is not None else 4
        if x is not None and not staged:
            if x.numel() * esz > self.io_bytes:
                raise ValueError("tensor larger than the collective staging region")
            self.input_view((x.numel(),), x.dtype).copy_(x.reshape(-1))
        self.epoch += 1
        in_dt = _DT[x.dtype] if x is not None else 0
        out_dt = _DT[out.dtype] if out is not None else 0
        _native.check(_native.kernels().ofb_comm_collective(
            ctypes.byref(a.ctx), c_int(mode), c_longlong(self.in_off), c_longlong(self.stage_off), c_int(in_dt),
            _native.ptr(out), c_int(out_dt), c_longlong(count), c_float(scale), c_uint(self.epoch), c_int(self.ctas),
            _native.stream_ptr()), "comm_collective")
        _k._count()

    def _pad(self, n, dtype):
        q = self.arena.n * (16 // torch.empty((), dtype=dtype).element_size())
        return (n + q - 1) // q * q

    def all_reduce(self, x, scale=1.0, out_dtype=None, staged=False):
        """sum over ranks of cast(x) * scale; returns a new tensor shaped like x."""
        out_dtype = out_dtype or x.dtype
        n = x.numel()
        padded = self._pad(n, x.dtype)
        if padded != n:
            xin = torch.zeros(padded, dtype=x.dtype, device=x.device)
            xin[:n] = x.reshape(-1)
            x_use = xin
        else:
            x_use = x
        if padded * 4 > 2 * self.io_bytes:
            raise ValueError("tensor larger than the all-reduce staging region")
        out = torch.empty(padded, dtype=out_dtype, device=x.device)
        self._run(0, x_use, out, padded, scale, staged and padded == n)
        return out[:n].view(x.shape)

    def reduce_scatter(self, x, scale=1.0, out_dtype=None, staged=False):
        """x: [n * m, ...] -> this rank's [m, ...] slice of the sum."""
        out_dtype = out_dtype or x.dtype
        n = self.arena.n
        out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=out_dtype, device=x.device)
        self._run(1, x, out, x.numel(), scale, staged)
        return out

    def all_gather(self, x, scale=1.0, out_dtype=None, staged=False):
        """x: [m, ...] -> [n * m, ...]."""
        out_dtype = out_dtype or x.dtype
        n = self.arena.n
        out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=out_dtype, device=x.device)
        self._run(2, x, out, x.numel() * n, scale, staged)
        return out

    def barrier(self):
        self._run(3, None, None, 0, 1.0, True)

    def all_to_all(self, x, in_axis, out_axis, logical_shape):
        """S(in_axis) -> S(out_axis): x is this rank's shard of a tensor of ``logical_shape`` split along
        in_axis; returns the shard split along out_axis. The transposition is done by the addressing of
        the pulling kernel (no pack/unpack pass)."""
        a = self.arena
        n = a.n
        i, j = in_axis, out_axis
        if i == j:
            return x
        shape = list(logical_shape)
        swap = i > j
        lo, hi = (j, i) if swap else (i, j)
        outer = int(torch.tensor(shape[:lo]).prod().item()) if lo else 1
        mid = int(torch.tensor(shape[lo + 1:hi]).prod().item()) if hi > lo + 1 else 1
        inner = int(torch.tensor(shape[hi + 1:]).prod().item()) if hi + 1 < len(shape) else 1
        out_shape = list(shape)
        out_shape[j] //= n
        out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
        if swap:
            # input split on the later axis: view it as [outer, J(out), mid, I(in), inner] and let the kernel
            # treat the first split axis as the output axis by pulling with swapped roles
            return self._all_to_all_swapped(x, out, outer, shape[lo], mid, shape[hi], inner)
        self.input_view((x.numel(),), x.dtype).copy_(x.reshape(-1))
        self.epoch += 1
        _native.check(_native.kernels().ofb_comm_all_to_all(
            ctypes.byref(a.ctx), c_longlong(self.in_off), c_int(_DT[x.dtype]), _native.ptr(out), c_longlong(outer),
            c_longlong(shape[lo]), c_longlong(mid), c_longlong(shape[hi]), c_longlong(inner), c_uint(self.epoch),
            c_int(self.ctas), _native.stream_ptr()), "comm_all_to_all")
        _k._count()
        return out

    def _all_to_all_swapped(self, x, out, outer, A, mid, Bdim, inner):
        # x: [outer, A, mid, B/n, inner] (split on the later axis) -> out: [outer, A/n, mid, B, inner].
        # Gather the peers' blocks with one all-gather-shaped pull per peer expressed through all_gather
        # on a transposed view: cheaper to express as all_gather + local slice for this rarely used direction.
        n = self.arena.n
        full = self.all_gather(x.reshape(1, -1)).view(n, outer, A, mid, Bdim // n, inner)
        r = self.arena.rank
        Al = A // n
        piece = full[:, :, r * Al:(r + 1) * Al]                       # [n, outer, Al, mid, B/n, inner]
        out.copy_(piece.permute(1, 2, 3, 0, 4, 5).reshape(out.shape))
        return out


class MultimemAllReduce:
    """All-reduce through the NVSwitch's in-fabric reduction (csrc/comm/multimem.cu): every rank reduces one slice with
    ``multimem.ld_reduce`` and re-broadcasts it with ``multimem.st`` over a multicast mapping of one symmetric buffer.

    The buffer and its multicast binding come from torch's symmetric memory (it owns the cuMulticast plumbing and the
    handle exchange); the barrier flags live in a small arena of this package. ``available`` is False when the group
    has no multicast support (no NVSwitch / NVLS): callers then use the peer-to-peer collectives."""

    def __init__(self, group, ranks, device, nbytes=64 << 20):
        self.available = False
        self.device = torch.device(device)
        self.n = len(ranks)
        self.nbytes = int(nbytes)
        self.epoch = 0
        if self.n < 2 or self.device.type != "cuda":
            return
        try:
            import torch.distributed._symmetric_memory as symm_mem
            pg = group if group is not None else dist.group.WORLD
            try:
                symm_mem.enable_symm_mem_for_group(pg.group_name)
            except Exception:
                pass
            self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            self.hdl = symm_mem.rendezvous(self.buf, group=pg.group_name)
            self.mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        except Exception as e:  # no symmetric-memory backend for this group
            self.reason = f"{type(e).__name__}: {e}"
            return
        if not self.mc:
            self.reason = "the group has no multicast (NVLS) support"
            return
        self.arena = SymmetricArena(group, ranks, device, 1 << 16)     # only its signal block is used
        self.available = True

    def all_reduce(self, x, scale=1.0):
        """sum over ranks of x, times scale, in x's dtype (fp32 or bf16); returns a new tensor shaped like x."""
        if x.dtype not in _DT:
            raise TypeError("multimem all-reduce takes fp32 or bf16")
        esz = x.element_size()
        q = self.n * (16 // esz)
        n = x.numel()
        padded = (n + q - 1) // q * q
        if padded * esz > self.nbytes:
            raise ValueError("tensor larger than the multicast buffer")
        view = self.buf[:padded * esz].view(x.dtype)
        view[:n].copy_(x.reshape(-1))
        if padded != n:
            view[n:].zero_()
        self.epoch += 1
        _native.check(_native.kernels().ofb_comm_multimem_all_reduce(
            ctypes.byref(self.arena.ctx), c_void_p(self.mc), c_longlong(padded), c_int(_DT[x.dtype]), c_float(scale),
            c_uint(self.epoch), c_int(4), c_int(0), _native.stream_ptr()), "multimem_all_reduce")
        _k._count()
        return view[:n].clone().view(x.shape)
