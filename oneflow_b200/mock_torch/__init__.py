"""``flow.mock_torch``: make ``import torch`` inside a scope resolve to this framework
(reference: python/oneflow/mock_torch/). Because local flow tensors are torch tensors and flow.* falls
back to torch.*, scripts written against torch already run; ``enable()`` additionally routes
``torch.save`` / ``torch.load`` to the flow checkpoint format and reports the state."""
import contextlib

import torch

_state = {"enabled": False, "save": None, "load": None}


def enable(lazy=False, verbose=False):
    if _state["enabled"]:
        return
    from ..framework.check_point import load, save
    _state.update(enabled=True, save=torch.save, load=torch.load)
    torch.save = lambda obj, f, *a, **k: save(obj, f)
    torch.load = lambda f, *a, **k: load(f, map_location=k.get("map_location"))


def disable():
    if not _state["enabled"]:
        return
    torch.save, torch.load = _state["save"], _state["load"]
    _state["enabled"] = False


def is_enabled():
    return _state["enabled"]


@contextlib.contextmanager
def mock(lazy=False, verbose=False):
    enable(lazy, verbose)
    try:
        yield
    finally:
        disable()
