"""``flow.optim``: optimizers, LR schedulers and SWA utilities."""
import torch.optim as _torch_optim
from torch.optim import swa_utils  # noqa: F401

from . import lr_scheduler, optimizer  # noqa: F401
from .optimizer import LAMB, LBFGS, SGD, Adadelta, Adagrad, Adam, AdamW, Ftrl, ParamGroup, RMSprop  # noqa: F401

from .optimizer import _ClipMixin  # noqa: E402

Optimizer = _torch_optim.Optimizer
# every optimizer (also user subclasses of the base class) answers the reference's extra methods
if not hasattr(Optimizer, "clip_grad"):
    Optimizer.clip_grad = _ClipMixin.clip_grad
if not hasattr(Optimizer, "support_sparse"):
    Optimizer.support_sparse = lambda self: False


def __getattr__(name):
    return getattr(_torch_optim, name)
