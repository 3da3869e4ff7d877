"""``flow.optim``: optimizers, LR schedulers and SWA utilities."""
import torch.optim as _torch_optim
from torch.optim import swa_utils  # noqa: F401

from . import lr_scheduler  # noqa: F401
from .optimizer import LAMB, LBFGS, SGD, Adadelta, Adagrad, Adam, AdamW, RMSprop  # noqa: F401

Optimizer = _torch_optim.Optimizer


def __getattr__(name):
    return getattr(_torch_optim, name)
