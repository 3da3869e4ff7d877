"""``import oneflow as flow`` — alias of :mod:`oneflow_b200` so that scripts written for the reference
run unchanged. Sub-modules (``oneflow.nn``, ``oneflow.optim``, ...) resolve to the oneflow_b200 ones."""
import importlib
import sys

import oneflow_b200 as _impl
from oneflow_b200 import *  # noqa: F401,F403
from oneflow_b200 import __all__ as _all  # noqa: F401

__version__ = _impl.__version__

for _name in _impl._SUBMODULES:
    _mod = importlib.import_module(f"oneflow_b200.{_name}")
    sys.modules[f"oneflow.{_name}"] = _mod
    globals()[_name.split(".")[0]] = importlib.import_module(f"oneflow_b200.{_name.split('.')[0]}")

from . import _oneflow_internal  # noqa: E402,F401


def __getattr__(name):
    return getattr(_impl, name)
