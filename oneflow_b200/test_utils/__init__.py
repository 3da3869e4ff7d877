"""``oneflow.test_utils``: what test suites written for the reference import (argument grids, the torch / flow
side-by-side checker)."""
