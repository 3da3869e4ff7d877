"""Import path of the dual-object module under the reference's file name
(python/oneflow/test_utils/automated_test_util/torch_flow_dual_object.py)."""
from .dual import *  # noqa: F401,F403
from .dual import (DualObject, GetDualObject, _trace, check_equality, check_tensor_equality, torch, torch_original)  # noqa: F401
