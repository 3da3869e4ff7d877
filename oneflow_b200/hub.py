"""``flow.hub``: torch.hub under the flow names (reference: python/oneflow/hub.py); the cache lives under
``$ONEFLOW_HOME`` when set."""
import os as _os

from torch.hub import *  # noqa: F401,F403
import torch.hub as _hub

ENV_ONEFLOW_HOME = "ONEFLOW_HOME"
if _os.environ.get(ENV_ONEFLOW_HOME):
    _hub.set_dir(_os.path.join(_os.environ[ENV_ONEFLOW_HOME], "hub"))


def __getattr__(name):
    return getattr(_hub, name)
