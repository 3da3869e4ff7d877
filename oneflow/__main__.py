"""``python -m oneflow`` (see oneflow_b200/__main__.py)."""
from oneflow_b200.__main__ import main

if __name__ == "__main__":
    raise SystemExit(main())
