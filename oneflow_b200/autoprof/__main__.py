"""python -m oneflow.autoprof script.py [...]  ->  $ONEFLOW_PROFILE_CSV (default op_prof.csv) and a summary on stdout."""
import os
import sys

from ..support.env_var_util import parse_boolean_from_env
from .util import print_summary_from_csv, profile_script, write_csv


def main(argv=None):
    scripts = list(sys.argv[1:] if argv is None else argv)
    if not scripts:
        print("usage: python -m oneflow.autoprof script.py [more scripts ...]", file=sys.stderr)
        return 2
    name = os.getenv("ONEFLOW_PROFILE_CSV", "op_prof")
    if not name.endswith(".csv"):
        name += ".csv"
    rows = []
    for s in scripts:
        rows += [(os.path.basename(s), ev) for ev in profile_script(s)]
    write_csv(rows, name)
    if parse_boolean_from_env("ONEFLOW_PROFILE_PRINT_SUMMARY", True):
        print_summary_from_csv(name)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
