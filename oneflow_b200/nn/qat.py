"""``flow.nn.qat``: quantisation-aware-training layers (reference: python/oneflow/nn/qat/conv.py)."""
from .modules.compat import QatConv1d, QatConv2d, QatConv3d  # noqa: F401
