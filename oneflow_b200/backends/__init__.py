"""``flow.backends``: cuda / cudnn / mps switches."""
from torch.backends import mps  # noqa: F401

from . import cuda, cudnn  # noqa: F401
