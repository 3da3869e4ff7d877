"""``flow.backends``: cuda / cudnn / mps switches (torch.backends)."""
from torch.backends import cuda, cudnn, mps  # noqa: F401
