"""``oneflow.nn.parameter``: import path of ``Parameter`` (reference: python/oneflow/nn/parameter.py:18)."""
from . import Parameter  # noqa: F401
