"""Side-by-side testing against PyTorch: ``torch`` here is a *dual* namespace — every attribute, call and operator is
carried out once on real PyTorch objects and once on this framework's (``oneflow``) objects, on equal inputs, and
``@autotest`` compares all results (and, after a backward pass with one shared random output gradient, the gradients
of every input tensor and module parameter).  Interface of the reference's harness
(python/oneflow/test_utils/automated_test_util/: ``autotest``, ``globaltest``, ``random_tensor``, ``random``,
``random_device``, ``oneof``, ``constant``, ``nothing``, placements and sbp generators), so its test files run
against this framework unchanged.

Because local flow tensors are torch tensors, the two sides differ exactly where this framework puts its own code
in the path: the ``flow.*`` / ``flow.nn.*`` / ``flow._C`` wrappers, global tensors with their SBP dispatch and
boxing, and the CUDA kernels behind them.
"""
import os  # noqa: F401  (test files written for the reference rely on ``os`` arriving with the star import)

from .generators import *  # noqa: F401,F403,E402
from .dual import *  # noqa: F401,F403,E402
from .dual import profile, torch  # noqa: F401,E402
