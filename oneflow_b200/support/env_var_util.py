"""Typed reads of environment variables (reference: python/oneflow/support/env_var_util.py)."""
import os


def parse_boolean_from_env(name, default):
    """``default`` when the variable is unset; else true for 1 / true / yes / on (any case), false for 0 / false / no / off."""
    raw = os.getenv(name)
    if raw is None:
        return bool(default)
    v = raw.strip().lower()
    if v in ("1", "true", "yes", "on"):
        return True
    if v in ("0", "false", "no", "off", ""):
        return False
    raise ValueError(f"environment variable {name}={raw!r} is not a boolean")


def parse_integer_from_env(name, default):
    raw = os.getenv(name)
    return int(default) if raw is None else int(raw)
