"""``oneflow.nn.modules.moving_average_min_max_observer`` import path."""
from ..extra_modules import MovingAverageMinMaxObserver  # noqa: F401
