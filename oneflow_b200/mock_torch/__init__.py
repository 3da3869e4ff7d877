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

    def __len__(self):
        return 0

    def __iter__(self):
        return iter(())

    def __enter__(self):
        raise RuntimeError(f'"{self.__name__}" is a dummy object and cannot be used as a context manager')

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
