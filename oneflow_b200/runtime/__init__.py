"""Python faces of the C++ runtime library (csrc/core -> lib/libofb_core.so)."""
from .core import (BinAllocator, ControlClient, CoreError, ControlServer, PersistentTable, RecordReader, TaskExecutor, TokenDataset,  # noqa: F401
                   balanced_split, copy_cost, slice_view, use_bin_allocator_for_torch, write_records)
