"""``oneflow.nn.modules.quantization`` import path."""
from ..extra_modules import Quantization  # noqa: F401
