"""Dense token/position embedding lookup and gradient on the native kernels
(csrc/kernels/embedding_ops.cu); CPU tensors take the PyTorch statement of the same op."""
from __future__ import annotations

from ctypes import c_int, c_longlong

import torch

from . import _native
from . import kernels as _k
from ._native import check, ptr, stream_ptr


def embedding_fwd(ids, wte, wpe=None, seq=1, vocab_start=0, pos_offset=0):
    """out[t] = wte[ids[t] - vocab_start] (+ wpe[t % seq + pos_offset]); ids outside the shard give zero rows."""
    ids = ids.reshape(-1)
    tokens, hidden = ids.numel(), wte.shape[1]
    if not wte.is_cuda:
        local = ids - vocab_start
        mine = (local >= 0) & (local < wte.shape[0])
        out = torch.where(mine[:, None], wte.float()[local.clamp(0, wte.shape[0] - 1)], torch.zeros(()))
        if wpe is not None:
            pos = torch.arange(tokens) % seq + pos_offset
            out = out + wpe.float()[pos]
        return out.to(wte.dtype)
    out = torch.empty((tokens, hidden), dtype=wte.dtype, device=wte.device)
    check(_native.kernels().ofb_embedding_fwd(ptr(ids), ptr(wte), ptr(wpe), ptr(out), c_longlong(tokens), c_int(seq),
                                              c_int(hidden), c_longlong(vocab_start), c_longlong(wte.shape[0]),
                                              c_int(pos_offset), stream_ptr()), "embedding_fwd")
    _k._count()
    return out


def embedding_bwd(ids, dout, dwte, dwpe=None, seq=1, vocab_start=0, pos_offset=0):
    """Accumulates dout rows into the fp32 gradient buffers dwte [vocab_rows, hidden] / dwpe."""
    ids = ids.reshape(-1)
    tokens, hidden = dout.shape
    if not dout.is_cuda:
        local = ids - vocab_start
        if dwte is not None:
            mine = (local >= 0) & (local < dwte.shape[0])
            dwte.index_add_(0, local[mine], dout.float()[mine])
        if dwpe is not None:
            pos = torch.arange(tokens) % seq + pos_offset
            dwpe.index_add_(0, pos, dout.float())
        return
    rows = dwte.shape[0] if dwte is not None else 0
    check(_native.kernels().ofb_embedding_bwd(ptr(ids), ptr(dout), ptr(dwte), ptr(dwpe), c_longlong(tokens), c_int(seq),
                                              c_int(hidden), c_longlong(vocab_start), c_longlong(rows), c_int(pos_offset),
                                              stream_ptr()), "embedding_bwd")
    _k._count()
