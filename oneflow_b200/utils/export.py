"""Export of feed-forward networks for the C++ inference API (csrc/api/oneflow_api.h).

``export_inference_graph(module, directory)`` walks an ``nn.Sequential`` (nested ones are flattened) of Linear, ReLU,
GELU and LayerNorm layers and writes ``graph.txt`` plus one raw bf16 file per parameter; an activation that follows a
Linear is folded into that layer's GEMM epilogue. ``InferenceGraph`` loads such a directory through the C ABI of
``libofb_api.so`` (what a C++ program does with ``oneflow_api::Graph::Load``).

Reference: oneflow/api/cpp (Graph::Load of a saved nn.Graph), python/oneflow/framework/check_point_v2.py save(..., save_as_external_data)."""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch


def _flatten(module):
    if isinstance(module, torch.nn.Sequential):
        for m in module:
            yield from _flatten(m)
    else:
        yield module


def _act_name(m):
    if isinstance(m, torch.nn.ReLU):
        return "relu"
    if isinstance(m, torch.nn.GELU):
        return "gelu_tanh" if getattr(m, "approximate", "none") == "tanh" else "gelu"
    return None


def _write_bf16(path, t):
    t.detach().to(torch.bfloat16).contiguous().cpu().view(torch.int16).numpy().tofile(path)


def export_inference_graph(module, directory):
    os.makedirs(directory, exist_ok=True)
    layers = list(_flatten(module))
    lines = ["oneflow_b200 inference graph v1"]
    i, width = 0, None
    while i < len(layers):
        m = layers[i]
        if isinstance(m, torch.nn.Linear):
            act = _act_name(layers[i + 1]) if i + 1 < len(layers) else None
            wf = f"p{i}.weight.bin"
            _write_bf16(os.path.join(directory, wf), m.weight)
            bf = "-"
            if m.bias is not None:
                bf = f"p{i}.bias.bin"
                _write_bf16(os.path.join(directory, bf), m.bias)
            lines.append(f"linear {m.in_features} {m.out_features} {wf} {bf} {act or 'none'}")
            width = m.out_features
            i += 2 if act else 1
        elif isinstance(m, torch.nn.LayerNorm):
            if len(m.normalized_shape) != 1:
                raise ValueError("only LayerNorm over the last dimension can be exported")
            n = m.normalized_shape[0]
            gf, bf = f"p{i}.gamma.bin", f"p{i}.beta.bin"
            _write_bf16(os.path.join(directory, gf), m.weight if m.weight is not None else torch.ones(n))
            _write_bf16(os.path.join(directory, bf), m.bias if m.bias is not None else torch.zeros(n))
            lines.append(f"layer_norm {n} {gf} {bf} {m.eps}")
            width = n
            i += 1
        elif _act_name(m) is not None:
            if width is None:
                raise ValueError("an activation cannot be the first layer (its width is unknown)")
            lines.append(f"activation {width} {_act_name(m)}")
            i += 1
        elif isinstance(m, (torch.nn.Dropout, torch.nn.Identity)):
            i += 1
        else:
            raise ValueError(f"cannot export layer of type {type(m).__name__}")
    with open(os.path.join(directory, "graph.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return directory


class InferenceGraph:
    """ctypes face of the C ABI of the C++ inference API."""

    def __init__(self, directory, device=0):
        lib_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libofb_api.so")
        self.lib = ctypes.CDLL(lib_path)
        self.lib.ofb_api_graph_load.restype = ctypes.c_void_p
        self.lib.ofb_api_last_error.restype = ctypes.c_char_p
        self.lib.ofb_api_graph_in_features.restype = ctypes.c_longlong
        self.lib.ofb_api_graph_out_features.restype = ctypes.c_longlong
        self.h = self.lib.ofb_api_graph_load(directory.encode(), ctypes.c_int(device))
        if not self.h:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())
        self.in_features = self.lib.ofb_api_graph_in_features(ctypes.c_void_p(self.h))
        self.out_features = self.lib.ofb_api_graph_out_features(ctypes.c_void_p(self.h))

    def forward(self, x):
        x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
        rows = x.shape[0]
        y = np.empty((rows, self.out_features), dtype=np.float32)
        rc = self.lib.ofb_api_graph_forward(ctypes.c_void_p(self.h), x.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(rows),
                                            y.ctypes.data_as(ctypes.c_void_p))
        if rc != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())
        return y

    def close(self):
        if self.h:
            self.lib.ofb_api_graph_free(ctypes.c_void_p(self.h))
            self.h = None
