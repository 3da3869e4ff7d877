from .graph import Graph, GraphModule, ModuleProxy, Proxy  # noqa: F401
from .graph_config import GraphConfig  # noqa: F401

GraphTensor = object  # graph-only tensor kind of the reference; tensors here are always eager
