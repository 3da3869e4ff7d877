"""The test helpers under their other import path (reference: python/oneflow/framework/unittest.py, re-exported there as
``oneflow.unittest``): TestCase, ``skip_unless_1n1d`` and friends, ``register_test_cases``."""
from ..unittest import *  # noqa: F401,F403
from ..unittest import TestCase, register_test_cases, skip_unless, skip_unless_1n1d, skip_unless_1n2d, skip_unless_1n4d  # noqa: F401
