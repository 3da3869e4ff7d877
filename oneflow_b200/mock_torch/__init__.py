"""``flow.mock_torch``: make ``import torch`` inside a scope resolve to this framework
(reference: python/oneflow/mock_torch/). Because local flow tensors are torch tensors and flow.* falls
back to torch.*, scripts written against torch already run; ``enable()`` additionally routes
``torch.save`` / ``torch.load`` to the flow checkpoint format and reports the state."""
import contextlib
import importlib
import sys
import types

import torch

_state = {"enabled": False, "save": None, "load": None}


# ------------------------------------------------------------------------------------------------ the two module sets
# While the mock is on, ``import torch`` / ``import torch.nn`` / ``from torch import nn`` in user code give views of
# this framework's modules (named ``oneflow`` / ``oneflow.nn``); switching off puts the library's own modules back.
# Only names that user code imported under the mock are shadowed in ``sys.modules``: PyTorch, the substrate of this
# framework, keeps finding its own sub-modules. Module-valued globals of the calling scope are switched as well, as
# the reference does (python/oneflow/mock_torch/mock_importer.py, ``enable`` / ``disable`` and ``_ModeState``).
_NAME_MAP = {"torch": "oneflow"}
_displaced = {}      # real modules taken out of sys.modules while the mock is on
_views = {}          # mock-side modules by the name they are imported under ("torch.nn" -> view of oneflow.nn)
_opts = {"lazy": False, "verbose": False}


_resolving = {"active": False}


@contextlib.contextmanager
def _real_imports():
    """Imports made while a view resolves a name must see the library's own modules (this framework falls back to
    them): the displaced modules are put back for the duration and the mock finder steps aside."""
    if _resolving["active"]:
        yield
        return
    _resolving["active"] = True
    shadow = {name: sys.modules.get(name) for name in _displaced}
    sys.modules.update(_displaced)
    try:
        yield
    finally:
        for name, prev in shadow.items():
            if prev is None:
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = prev
        _resolving["active"] = False


def _import_ours(shown):
    with _real_imports():
        return importlib.import_module(shown)


def _target_name(fullname, name_map=None):
    head, _, rest = fullname.partition(".")
    to = (name_map or _NAME_MAP).get(head)
    if to is None:
        return None
    return to + ("." + rest if rest else "")


class _View(types.ModuleType):
    """One of this framework's modules under the name user code expects: ``__name__`` / ``__package__`` read
    ``oneflow...``, attribute reads and writes go to the module behind it, sub-modules come back as views, and a
    missing name is a :class:`DummyModule` in lazy mode."""

    def __init__(self, target, shown):
        super().__init__(shown)
        self.__dict__.update(_target=target, __package__=shown, __path__=[], __file__=getattr(target, "__file__", None))

    def __setattr__(self, name, value):
        setattr(self.__dict__["_target"], name, value)

    def __dir__(self):
        return dir(self.__dict__["_target"])

    def __getattr__(self, name):
        target, shown = self.__dict__["_target"], self.__name__
        try:
            value = getattr(target, name)
        except AttributeError:
            try:
                value = _import_ours(shown + "." + name)
            except ImportError:
                if name.startswith("__") and name.endswith("__"):
                    raise AttributeError(name) from None
                if _opts["lazy"]:
                    if _opts["verbose"]:
                        print(f"{shown}.{name} is not found in oneflow, use dummy object as fallback.")
                    return DummyModule(shown + "." + name, _opts["verbose"])
                raise AttributeError(f"module '{shown}' has no attribute '{name}'") from None
        if isinstance(value, types.ModuleType) and not isinstance(value, (_View, DummyModule)) \
                and value.__name__.split(".")[0] in ("oneflow", "oneflow_b200", "flowvision"):
            return _view_of(value, shown + "." + name)
        return value


def _view_of(target, shown):
    v = _views.get(shown)
    if v is None or v.__dict__["_target"] is not target:
        v = _views[shown] = _View(target, shown)
    return v


class _MockFinder:
    """Meta-path finder of the mock: ``torch[.x.y]`` -> a view of ``oneflow[.x.y]``."""

    def __init__(self):
        self.name_map = dict(_NAME_MAP)

    def find_spec(self, fullname, path=None, target=None):
        shown = _target_name(fullname, self.name_map)
        if shown is None or not _state["enabled"] or _resolving["active"]:
            return None
        import importlib.machinery
        return importlib.machinery.ModuleSpec(fullname, self, is_package=True)

    def create_module(self, spec):
        shown = _target_name(spec.name, self.name_map)
        try:
            return _view_of(_import_ours(shown), shown)
        except ImportError:
            if _opts["lazy"]:
                if _opts["verbose"]:
                    print(f"{shown} is not found in oneflow, use dummy object as fallback.")
                return DummyModule(shown, _opts["verbose"])
            raise ModuleNotFoundError(f"{shown} is not implemented", name=spec.name) from None

    def exec_module(self, module):
        pass


_finder = _MockFinder()


def _is_ours(name, name_map):
    return name.partition(".")[0] in name_map


def _switch_globals(scope, to_mock):
    if scope is None:
        return
    for key, val in list(scope.items()):
        if not isinstance(val, types.ModuleType):
            continue
        if to_mock and not isinstance(val, (_View, DummyModule)) and _is_ours(val.__name__, _finder.name_map):
            shown = _target_name(val.__name__, _finder.name_map)
            try:
                scope[key] = _view_of(_import_ours(shown), shown)
            except ImportError:
                pass
        elif not to_mock and isinstance(val, _View):
            back = {v: k for k, v in _finder.name_map.items()}
            head, _, rest = val.__name__.partition(".")
            real = back.get(head, head) + ("." + rest if rest else "")
            mod = _displaced.get(real) or sys.modules.get(real)
            if mod is not None and not isinstance(mod, _View):
                scope[key] = mod


def _enable(lazy=False, verbose=False, extra_dict=None, scope=None):
    import os
    if os.getenv("ONEFLOW_DISABLE_MOCK_TORCH") == "1":
        return
    _opts.update(lazy=lazy, verbose=verbose)
    _finder.name_map = dict(_NAME_MAP, **(extra_dict or {}))
    if not _state["enabled"]:
        from ..framework.check_point import load, save
        _state.update(enabled=True, save=torch.save, load=torch.load)
        torch.save = lambda obj, f, *a, **k: save(obj, f)
        torch.load = lambda f, *a, **k: load(f, map_location=k.get("map_location"))
        if _finder not in sys.meta_path:
            sys.meta_path.insert(0, _finder)
        # the library's modules leave sys.modules (imports made under the mock get views; the views themselves
        # resolve names with the real modules back in place), what was imported under the mock before returns
        for name in [n for n in sys.modules if _is_ours(n, _finder.name_map)]:
            if not isinstance(sys.modules[name], (_View, DummyModule)):
                _displaced[name] = sys.modules.pop(name)
        sys.modules.update(_views_by_import)
    _switch_globals(scope, True)


def _disable(scope=None):
    if _state["enabled"]:
        torch.save, torch.load = _state["save"], _state["load"]
        _state["enabled"] = False
        for name, mod in list(sys.modules.items()):
            if isinstance(mod, (_View, DummyModule)) and _is_ours(name, _finder.name_map):
                _views_by_import[name] = sys.modules.pop(name)
        sys.modules.update(_displaced)
        _displaced.clear()
    _switch_globals(scope, False)


_views_by_import = {}    # what user code imported under the mock, by import name; re-installed on the next enable


def _caller_globals():
    f = sys._getframe(2)
    return f.f_globals if f is not None else None


class enable:
    """``mock_torch.enable()`` switches the mock on at once; used as ``with mock_torch.enable():`` it is switched
    back on leaving the block. ``lazy``: names this framework lacks become dummy objects instead of errors;
    ``extra_dict``: further package renames, e.g. ``{"torchvision": "flowvision"}``
    (reference: python/oneflow/mock_torch/mock_importer.py, class ``enable``)."""

    def __init__(self, lazy=False, verbose=False, extra_dict=None, main_pkg=None, mock_version=None,
                 required_dependencies=(), *, _scope=None):
        self._was = _state["enabled"]
        self._prev = dict(_opts)
        self._scope = _scope if _scope is not None else _caller_globals()
        _enable(lazy, verbose, extra_dict, self._scope)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if not self._was:
            _disable(self._scope)
        else:
            _opts.update(self._prev)
        return False


class disable:
    """The inverse of :class:`enable`: off at once, restored on leaving a ``with`` block."""

    def __init__(self, *, _scope=None):
        self._was = _state["enabled"]
        self._prev = dict(_opts)
        self._scope = _scope if _scope is not None else _caller_globals()
        _disable(self._scope)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if self._was:
            _enable(self._prev["lazy"], self._prev["verbose"], None, self._scope)
        return False


def is_enabled():
    return _state["enabled"]


@contextlib.contextmanager
def mock(lazy=False, verbose=False):
    with enable(lazy, verbose, _scope={}):
        yield


# ------------------------------------------------------------------------------------------------ helper objects
import importlib  # noqa: E402
import types  # noqa: E402


class DummyModule(types.ModuleType):
    """Stand-in for a name that does not exist: every attribute, item and call yields another dummy, it is falsy,
    empty when iterated and usable as a base class — so optional code paths of third-party packages import
    (reference: python/oneflow/mock_torch/mock_modules.py:61-118)."""

    def __init__(self, name, verbose=False):
        super().__init__(name)
        self.__dict__["_verbose"] = verbose

    def _say(self, what):
        if self.__dict__.get("_verbose"):
            print(f'"{self.__name__}" is a dummy object, and {what}.')

    def __getattr__(self, name):
        self._say(f'its attr "{name}" is accessed')
        if name in ("__path__", "__file__"):
            return None
        if name == "__all__":
            return []
        if name == "__mro_entries__":
            return lambda bases: ()
        return DummyModule(self.__name__ + "." + name, self.__dict__.get("_verbose", False))

    def __getitem__(self, item):
        self._say(f"`{self.__name__}[{item}]` is called")
        if isinstance(item, int):
            raise IndexError
        return DummyModule(f"{self.__name__}[{item}]", self.__dict__.get("_verbose", False))

    def __call__(self, *args, **kwargs):
        self._say("it is called")
        return DummyModule(self.__name__ + "()", self.__dict__.get("_verbose", False))

    def __bool__(self):
        return False

    def __instancecheck__(self, obj):
        return False

    def __subclasscheck__(self, cls):
        return False

    def __len__(self):
        return 0

    def __iter__(self):
        return iter(())

    def __enter__(self):
        raise RuntimeError(f'"{self.__name__}" is a dummy object, and does not support "with" statement.')

    def __exit__(self, *exc):
        return False


class ModuleWrapper(types.ModuleType):
    """A module view whose attribute writes reach the wrapped module and whose missing attributes become
    :class:`DummyModule` objects when ``lazy`` (reference: python/oneflow/mock_torch/mock_importer.py:60-91)."""

    def __init__(self, module, lazy=False, verbose=False):
        super().__init__(module.__name__)
        self.__dict__.update(module=module, _lazy=lazy, _verbose=verbose)

    def __setattr__(self, name, value):
        setattr(self.__dict__["module"], name, value)

    def __getattr__(self, name):
        mod = self.__dict__["module"]
        if not hasattr(mod, name):
            if name == "__path__":
                return None
            if name == "__all__":
                return [a for a in dir(mod) if not a.startswith("_")]
            full = mod.__name__ + "." + name
            if self.__dict__["_lazy"]:
                return DummyModule(full, self.__dict__["_verbose"])
            raise AttributeError(full + " is not implemented")
        attr = getattr(mod, name)
        if isinstance(attr, types.ModuleType):
            return ModuleWrapper(attr, self.__dict__["_lazy"], self.__dict__["_verbose"])
        return attr


class DynamicMockModule(types.ModuleType):
    """A third-party package imported with the mock active; ``hijack(name, obj)`` overrides single attributes
    afterwards (reference: python/oneflow/mock_torch/dyn_mock_mod.py:25-100)."""

    def __init__(self, pkg_name, obj_entity, main_pkg_enable):
        super().__init__(pkg_name)
        self.__dict__.update(_pkg_name=pkg_name, _obj_entity=obj_entity, _main_pkg_enable=main_pkg_enable, _intercept_dict={})

    def __repr__(self):
        return f"<DynamicMockModule {self._pkg_name} {self._obj_entity}>"

    def hijack(self, module_name, obj):
        self._intercept_dict[module_name] = obj

    @classmethod
    def from_package(cls, main_pkg, *, lazy=True, verbose=False, extra_dict=None, required_dependencies=()):
        def main_pkg_enable():
            return mock(lazy=lazy, verbose=verbose)

        with main_pkg_enable():
            entity = importlib.import_module(main_pkg)
        return cls(main_pkg, entity, main_pkg_enable)

    def __getattr__(self, name):
        if name in self._intercept_dict:
            return self._intercept_dict[name]
        with self._main_pkg_enable():
            if hasattr(self._obj_entity, name):
                return getattr(self._obj_entity, name)
            try:
                return importlib.import_module(f"{self._obj_entity.__name__}.{name}")
            except ModuleNotFoundError:
                raise AttributeError(f"{self._pkg_name} has no attribute {name!r}") from None

    def __all__(self):
        with self._main_pkg_enable():
            return dir(self._obj_entity)
