"""``oneflow.nn.modules.min_max_observer`` import path (reference: python/oneflow/nn/modules/min_max_observer.py)."""
from ..extra_modules import MinMaxObserver  # noqa: F401
