"""Build-time state of ``nn.Graph``: whether code currently runs inside a graph's ``build``
(reference: python/oneflow/framework/graph_build_util.py, ``lazy_mode``)."""
import contextlib


class _LazyMode:
    """``lazy_mode.is_enabled()`` is True inside ``nn.Graph.build`` (and inside ``lazy_mode.guard(True)``)."""

    def __init__(self):
        self._forced = []

    def is_enabled(self):
        if self._forced:
            return self._forced[-1]
        from ..nn.graph.graph import Graph
        return Graph._nesting > 0

    @contextlib.contextmanager
    def guard(self, mode=True):
        self._forced.append(bool(mode))
        try:
            yield
        finally:
            self._forced.pop()


lazy_mode = _LazyMode()


@contextlib.contextmanager
def graph_build_context(config_proto=None, session=None):
    with lazy_mode.guard(True):
        yield
