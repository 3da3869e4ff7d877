"""``oneflow.nn.utils.skip_init`` import path (reference: python/oneflow/nn/utils/skip_init.py)."""
from torch.nn.utils import skip_init  # noqa: F401
