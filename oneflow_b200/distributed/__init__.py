"""``flow.distributed``: the launcher (``python -m oneflow_b200.distributed.launch``) and rank helpers."""
from ..env import get_local_rank, get_rank, get_world_size  # noqa: F401
