"""``flow.nn.image``: the image modules under their short names (reference: python/oneflow/nn/image.py:16-20)."""
from .modules.dataset import ImageBatchAlign as batch_align  # noqa: F401
from .modules.dataset import ImageDecode as decode  # noqa: F401
from .modules.dataset import ImageFlip as flip  # noqa: F401
from .modules.dataset import ImageNormalize as normalize  # noqa: F401
from .modules.dataset import ImageResize as Resize  # noqa: F401
