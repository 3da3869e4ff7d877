"""``flow.fx``: symbolic tracing of modules into an editable graph (reference: python/oneflow/fx/, a port of
torch.fx). The tracer is torch.fx's; this framework's own layers (whose ``forward`` branches on the input's layout,
dtype or placement) are leaves of the trace like the library's layers."""
from torch.fx import *  # noqa: F401,F403
import torch.fx as _fx
from torch.fx import Graph, GraphModule, Interpreter, Node, Proxy, Transformer, wrap  # noqa: F401


class Tracer(_fx.Tracer):
    def is_leaf_module(self, m, module_qualified_name):
        mod = type(m).__module__
        if mod.startswith(("oneflow_b200.nn", "oneflow.nn")) and not isinstance(m, (_fx.GraphModule,)):
            import torch
            return not isinstance(m, (torch.nn.Sequential, torch.nn.ModuleList, torch.nn.ModuleDict))
        return super().is_leaf_module(m, module_qualified_name)


def symbolic_trace(root, concrete_args=None):
    """Trace ``root`` (a module or function) into a :class:`GraphModule`."""
    tracer = Tracer()
    graph = tracer.trace(root, concrete_args)
    name = root.__class__.__name__ if hasattr(root, "forward") else root.__name__
    return _fx.GraphModule(tracer.root, graph, name)


def __getattr__(name):
    return getattr(_fx, name)
