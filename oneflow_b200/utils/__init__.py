"""``flow.utils``: data loading, activation checkpointing, global-view pytree helpers, tensor interop."""
from . import checkpoint, data, dlpack, global_view, tensor  # noqa: F401
from torch.utils import hooks, model_zoo  # noqa: F401,E402
from ..framework.config_util import api_load_library as load_library  # noqa: F401,E402
