"""``oneflow.nn.modules.fake_quantization`` import path."""
from ..extra_modules import FakeQuantization  # noqa: F401
