"""``flow.autograd``: torch.autograd under the flow names (backward, grad, Function, functional.*, graph
saved-tensor hooks, grad modes). Reference: python/oneflow/autograd/*.py."""
from torch.autograd import *  # noqa: F401,F403
from torch.autograd import Function, backward, functional, grad, graph  # noqa: F401
from torch import enable_grad, inference_mode, no_grad, set_grad_enabled  # noqa: F401
from torch import is_grad_enabled  # noqa: F401,E402
from torch.autograd.functional import hessian, hvp, jacobian, jvp, vhp, vjp  # noqa: F401,E402


def _is_data_valid(ctx):
    """True while the context of an ``autograd.Function`` still holds what ``forward`` saved (backward without
    ``retain_graph`` releases it; reference: oneflow/api/python/autograd/function_node.cpp)."""
    try:
        ctx.saved_tensors
        return True
    except RuntimeError:
        return False


import torch.autograd.function as _fn  # noqa: E402
_fn.FunctionCtx._is_data_valid = _is_data_valid
