"""``flow.nn.init``: torch.nn.init (the in-place initialisers work on global tensors through the dispatch)."""
from torch.nn.init import *  # noqa: F401,F403
import torch.nn.init as _I


def __getattr__(name):
    return getattr(_I, name)
