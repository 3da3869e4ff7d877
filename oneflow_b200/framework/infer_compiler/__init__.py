"""PyTorch modules run through the native graph runtime: ``compile_from_torch(module)`` wraps a module so that every call goes
through a compiled plan (exported on first use per input signature, cached afterwards), and ``oneflow_backend`` is the same as
a ``torch.compile`` backend (``torch.compile(module, backend=oneflow_backend)``).

The wrapped module is exported with ``utils.export.export_graph`` (torch.fx over example inputs; weights stored as bf16) and run
by ``InferenceGraph`` on the device of its inputs (CUDA inputs: the sm_100a kernels of that GPU, replayed as one CUDA graph from
the second call on; CPU inputs: the host implementation of the same operators). ``save_graph`` / ``load_graph`` keep the
exported directory, so a process can start from a graph another one compiled.

Reference: python/oneflow/framework/infer_compiler/with_oneflow_compile.py (compile_from_torch, DeployableModule: a torch module
whose forward runs a cached nn.Graph of its OneFlow twin, graph files saved and loaded), with_oneflow_backend.py (the
torch.compile backend)."""
from __future__ import annotations

import os
import shutil
import tempfile

import numpy as np
import torch

from ...utils import export as _export

__all__ = ["compile_from_torch", "oneflow_compile", "DeployableModule", "oneflow_backend"]


def _signature(tensors):
    return tuple((tuple(t.shape), str(t.dtype), t.device.type, t.device.index) for t in tensors)


class _CompiledCall:
    """One exported directory + loaded graph for one input signature."""

    def __init__(self, module, tensors, directory, n_streams):
        self.directory = directory
        cpu_inputs = tuple(t.detach().cpu() for t in tensors)
        with torch.no_grad():
            ref = module(*cpu_inputs) if not isinstance(module, torch.fx.GraphModule) else module(*cpu_inputs)
        self.single = torch.is_tensor(ref)
        outs = (ref,) if self.single else tuple(ref)
        self.out_shapes = [tuple(o.shape) for o in outs]
        self.out_dtypes = [o.dtype for o in outs]
        _export.export_graph(module, cpu_inputs, directory)
        dev = tensors[0].device
        self.graph = _export.InferenceGraph(directory, device=(dev.index or 0) if dev.type == "cuda" else -1, n_streams=n_streams)

    def __call__(self, tensors):
        outs = self.graph.run(*[t.detach().cpu().numpy() for t in tensors])
        dev = tensors[0].device
        res = [torch.from_numpy(o).reshape(s).to(dt if dt.is_floating_point else torch.float32).to(dev)
               for o, s, dt in zip(outs, self.out_shapes, self.out_dtypes)]
        return res[0] if self.single else tuple(res)


class DeployableModule(torch.nn.Module):
    """A torch module whose ``forward`` runs compiled plans of itself. Attribute access falls through to the wrapped module
    (``.weight``, ``.config`` ... keep working); ``use_graph=False`` calls the module eagerly."""

    def __init__(self, torch_module, use_graph=True, options=None):
        super().__init__()
        object.__setattr__(self, "_deployed", torch_module)
        self._use_graph = use_graph
        self._options = dict(options or {})
        self._calls = {}
        self._root = None

    # the wrapped module is not registered as a sub-module: state_dict() of the wrapper is that of the module itself
    def state_dict(self, *args, **kwargs):
        return self._deployed.state_dict(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(object.__getattribute__(self, "_deployed"), name)

    def _directory(self, index):
        if self._root is None:
            self._root = tempfile.mkdtemp(prefix="oneflow_deploy_")
        return os.path.join(self._root, f"graph{index}")

    def forward(self, *args):
        if not self._use_graph:
            return self._deployed(*args)
        if not all(torch.is_tensor(a) for a in args):
            raise TypeError("a compiled module takes tensors; close over everything else before compiling")
        key = _signature(args)
        call = self._calls.get(key)
        if call is None:
            limit = int(self._options.get("size", 9))        # cached graphs, as the reference's graph cache size
            if len(self._calls) >= limit:
                old = next(iter(self._calls))
                self._calls.pop(old).graph.close()
            call = self._calls[key] = _CompiledCall(self._deployed, args, self._directory(len(self._calls)), int(self._options.get("n_streams", 2)))
        return call(args)

    def get_graph(self):
        """The most recently compiled graph (``InferenceGraph``), e.g. for ``stats()``."""
        return next(reversed(self._calls.values())).graph if self._calls else None

    def save_graph(self, file_path):
        """Copies the exported directories (graph.txt + weights) of every compiled signature under ``file_path``."""
        os.makedirs(file_path, exist_ok=True)
        for i, call in enumerate(self._calls.values()):
            shutil.copytree(call.directory, os.path.join(file_path, f"graph{i}"), dirs_exist_ok=True)
        return file_path

    def load_graph(self, file_path, example_inputs, device=None, run_warmup=True):
        """Registers a saved directory for the signature of ``example_inputs`` without exporting again."""
        args = tuple(example_inputs)
        call = object.__new__(_CompiledCall)
        call.directory = file_path if os.path.exists(os.path.join(file_path, "graph.txt")) else os.path.join(file_path, "graph0")
        with torch.no_grad():
            ref = self._deployed(*[t.detach().cpu() for t in args])
        call.single = torch.is_tensor(ref)
        outs = (ref,) if call.single else tuple(ref)
        call.out_shapes, call.out_dtypes = [tuple(o.shape) for o in outs], [o.dtype for o in outs]
        dev = args[0].device if device is None else torch.device(device)
        call.graph = _export.InferenceGraph(call.directory, device=(dev.index or 0) if dev.type == "cuda" else -1,
                                            n_streams=int(self._options.get("n_streams", 2)))
        self._calls[_signature(args)] = call
        if run_warmup:
            call(args)
        return self


def compile_from_torch(torch_module, *, use_graph=True, options=None):
    """Wraps ``torch_module`` into a ``DeployableModule`` (the module itself is left untouched and keeps its weights)."""
    if isinstance(torch_module, DeployableModule):
        return torch_module
    return DeployableModule(torch_module, use_graph=use_graph, options=options)


oneflow_compile = compile_from_torch


def oneflow_backend(gm, example_inputs, *args, **kwargs):
    """``torch.compile`` backend: the FX graph dynamo hands over is exported once and run by the native graph runtime."""
    tensors = [t for t in example_inputs if torch.is_tensor(t)]
    if len(tensors) != len(example_inputs):
        return gm.forward                                     # symbolic sizes and the like: leave the graph to eager
    state = {}

    def run(*inputs):
        key = _signature(inputs)
        if key not in state:
            try:
                state[key] = _CompiledCall(gm, inputs, tempfile.mkdtemp(prefix="oneflow_backend_"), 2)
            except ValueError:                                # an operator the exporter does not know: eager for this graph
                state[key] = None
        call = state[key]
        if call is None:
            return gm.forward(*inputs)
        out = call(inputs)
        return out if isinstance(out, tuple) else (out,)

    return run
