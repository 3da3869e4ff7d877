"""``import oneflow as flow`` — alias of :mod:`oneflow_b200` so that scripts written for the reference
run unchanged. Every dotted import path below ``oneflow`` (``oneflow.nn``, ``oneflow.nn.utils.rnn``,
``oneflow.linalg`` ...) resolves lazily: first to the ``oneflow_b200`` module of the same path, then to a module
attribute of the package, and last to the module of the same path of the tensor substrate (``torch``), whose
functions operate on the same tensor type."""
import importlib
import importlib.abc
import importlib.machinery
import sys
import types

import oneflow_b200 as _impl
from oneflow_b200 import *  # noqa: F401,F403
from oneflow_b200 import __all__ as _all  # noqa: F401

__version__ = _impl.__version__


def _import_or_none(name):
    try:
        return importlib.import_module(name)
    except ModuleNotFoundError as e:
        if e.name and (name == e.name or name.startswith(e.name + ".")):
            return None
        raise


def _resolve(rel):
    mod = _import_or_none("oneflow_b200." + rel)
    if mod is None:
        obj = _impl
        for part in rel.split("."):
            obj = getattr(obj, part, None)
            if obj is None:
                break
        if isinstance(obj, types.ModuleType):
            mod = obj
    if mod is None:
        mod = _import_or_none("torch." + rel)
    if mod is not None and mod.__name__.startswith("oneflow_b200") and not hasattr(mod, "__path__"):
        mod.__path__ = []          # lets ``import oneflow.a.b.c`` descend through a plain module
    return mod


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("oneflow.") or fullname == "oneflow.__main__":
            return None
        mod = _resolve(fullname[len("oneflow."):])
        if mod is None:
            return None
        # a real package stays one (``python -m oneflow.<package>`` then looks for its __main__)
        return importlib.machinery.ModuleSpec(fullname, self, is_package=bool(getattr(mod, "__path__", None)))

    def create_module(self, spec):
        return _resolve(spec.name[len("oneflow."):])

    def exec_module(self, module):
        pass

    def get_code(self, fullname):
        """For ``python -m oneflow.<package>``: the code object of the module this name stands for."""
        mod = _resolve(fullname[len("oneflow."):])
        loader = getattr(getattr(mod, "__spec__", None), "loader", None)
        return loader.get_code(mod.__name__) if loader is not None and hasattr(loader, "get_code") else None


sys.meta_path.insert(0, _AliasFinder())    # ahead of the path finder: one module object per file, under both names

for _name in _impl._SUBMODULES:
    _mod = _resolve(_name)
    sys.modules[f"oneflow.{_name}"] = _mod
    globals()[_name.split(".")[0]] = importlib.import_module(f"oneflow_b200.{_name.split('.')[0]}")

from . import _oneflow_internal  # noqa: E402,F401


def __getattr__(name):
    return getattr(_impl, name)
