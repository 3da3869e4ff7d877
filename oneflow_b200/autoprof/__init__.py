"""``python -m oneflow.autoprof script.py [more scripts ...]``: runs the scripts under ``flow.profiler`` and writes one CSV row
per operator (reference: python/oneflow/autoprof, which profiles the ``profile`` blocks of its test files into op_prof.csv)."""
from .util import profile_script, print_summary_from_csv, write_csv  # noqa: F401
