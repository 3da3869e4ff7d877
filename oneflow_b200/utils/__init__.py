"""``flow.utils``: data loading, activation checkpointing, global-view pytree helpers, tensor interop."""
from . import checkpoint, data, global_view, tensor  # noqa: F401
