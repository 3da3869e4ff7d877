"""The process's one implicit session (reference: python/oneflow/framework/session_context.py)."""
import itertools

_ids = itertools.count(1)


class Session:
    def __init__(self):
        self.id = next(_ids)
        self.is_running = True
        self.resource = {}

    def TryInit(self):
        return self

    def TryClose(self):
        self.is_running = False


_default = None


def GetDefaultSession():
    global _default
    if _default is None:
        _default = Session()
    return _default


def NewDefaultSession(*args, **kwargs):
    global _default
    _default = Session()
    return _default


def TryCloseDefaultSession():
    if _default is not None:
        _default.TryClose()
