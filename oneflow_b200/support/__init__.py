"""Small helpers the reference keeps under ``oneflow.support`` (python/oneflow/support/env_var_util.py and friends)."""
from . import env_var_util  # noqa: F401
