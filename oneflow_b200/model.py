"""``flow.model``: the high-level training loop (reference: python/oneflow/model.py re-exporting framework/model.py)."""
from .framework.model import (Callback, CheckpointConfig, DataModule, Model, NumpyDataModule, TrainingConfig,  # noqa: F401
                              ValidationConfig)
