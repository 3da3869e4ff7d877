"""``flow.data`` (reference: python/oneflow/data.py)."""
from .experimental.load_mnist import load_mnist  # noqa: F401
