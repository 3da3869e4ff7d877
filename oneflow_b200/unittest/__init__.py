"""``flow.unittest``: helpers test suites written for the reference rely on — ``TestCase``, the
``skip_unless_<n>n<d>d`` decorators driven by the launcher's environment, ``register_test_cases`` and the dataset
directory (reference: python/oneflow/unittest/__init__.py:16-30, python/oneflow/framework/unittest.py:37-222)."""
import importlib.util
import os
import unittest as _unittest

from . import env  # noqa: F401
from .env import device_num, node_size

TestCase = _unittest.TestCase
MLIRTestCase = _unittest.TestCase       # no MLIR pipeline exists here; such cases run as plain test cases


def dataset_dir(sub_dir=None):
    base = os.getenv("ONEFLOW_TEST_DATASET_DIR") or "/dataset"
    return base if sub_dir is None else os.path.join(base, sub_dir)


def num_nodes_required(num_nodes):
    def decorator(f):
        f.__oneflow_test_case_num_nodes_required__ = num_nodes
        return f
    return decorator


def _num_nodes_of(func):
    return getattr(func, "__oneflow_test_case_num_nodes_required__", 1)


def register_test_cases(scope, directory, filter_by_num_nodes, base_class=_unittest.TestCase):
    """Loads every ``test*.py`` of ``directory`` and publishes its ``test*`` functions whose node requirement passes
    ``filter_by_num_nodes`` as methods of a TestCase class named after the file, in ``scope``."""
    for f in sorted(os.listdir(directory)):
        path = os.path.join(directory, f)
        if not (os.path.isfile(path) and f.endswith(".py") and f.startswith("test")):
            continue
        name = f[:-3]
        spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        methods = {k: getattr(module, k) for k in dir(module)
                   if k.startswith("test") and callable(getattr(module, k)) and filter_by_num_nodes(_num_nodes_of(getattr(module, k)))}
        scope[name] = type(name, (base_class,), methods)


def skip_unless(n, d):
    """Run only under a launch of ``n`` nodes with ``d`` devices each (``ONEFLOW_TEST_NODE_NUM`` /
    ``ONEFLOW_TEST_DEVICE_NUM``, both 1 by default)."""
    if node_size() == n and device_num() == d:
        return lambda func: func
    return _unittest.skip(f"only runs when node_size is {n} and device_num is {d}")


def skip_unless_1n1d():
    return skip_unless(1, 1)


def skip_unless_1n2d():
    return skip_unless(1, 2)


def skip_unless_1n4d():
    return skip_unless(1, 4)


def skip_unless_2n1d():
    return skip_unless(2, 1)


def skip_unless_2n2d():
    return skip_unless(2, 2)


def skip_unless_2n4d():
    return skip_unless(2, 4)
