"""``oneflow._oneflow_internal._C``: the functional namespace under its extension-module path."""
import oneflow_b200._C as _impl


def __getattr__(name):
    return getattr(_impl, name)


def __dir__():
    return dir(_impl)
