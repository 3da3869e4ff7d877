"""``flow.model.Model``: a training / validation / checkpoint loop around a module that defines its own steps.

    class Net(flow.model.Model):
        def forward(self, x): ...
        def training_step(self, batch, optimizer_idx=0): return loss            # or (loss, extras...)
        def validation_step(self, batch): return metrics
        def configure_optimizers(self): return flow.optim.SGD(self.parameters(), lr=0.1)

    train = flow.model.TrainingConfig(); train.config_data(my_data_module)
    Net().fit(training_config=train, validation_config=..., checkpoint_config=..., callbacks=..., max_steps=100)

Every step index runs, in this order, the sub-loops that were configured: training (one ``training_step`` + backward + optimizer
step per configured optimizer), validation (every ``step_interval`` steps, under ``no_grad`` and ``eval``), checkpoint (load once
before the first step, save every ``step_interval`` steps).

Reference: python/oneflow/framework/model.py (Model.fit, TrainingConfig / ValidationConfig / CheckpointConfig, Callback,
DataModule / NumpyDataModule, the OOP-style train / validate / checkpoint sub-models)."""
from __future__ import annotations

import os

import numpy as np
import torch

from ..nn import Module


class DataModule(Module):
    """Produces the batch of a step: ``forward(step_idx, optimizer_idx)`` returns whatever ``training_step`` takes as ``batch``."""

    def forward(self, step_idx=0, optimizer_idx=0):
        raise NotImplementedError


class NumpyDataModule(DataModule):
    """A data module whose ``forward`` returns numpy arrays; they reach the step as tensors."""

    def __call__(self, *args):
        batch = super().__call__(*args)
        conv = lambda a: torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
        return tuple(conv(a) for a in batch) if isinstance(batch, (tuple, list)) else conv(batch)


class _Config:
    def __init__(self):
        self.data = None
        self.step_interval = 1
        self.error_msg = ""

    def config_data(self, data=None):
        self.data = data

    def config_step_interval(self, step_interval=1):
        if int(step_interval) < 1:
            raise ValueError("step_interval must be at least 1")
        self.step_interval = int(step_interval)

    def config_execution(self, exe_cfg=None):          # the function-style execution config of old releases: nothing to set here
        self.exe_cfg = exe_cfg

    def check_valid(self):
        if not isinstance(self.data, DataModule):
            self.error_msg = "the data of a config must be a DataModule (config_data)"
            return False
        return True


class TrainingConfig(_Config):
    pass


class ValidationConfig(_Config):
    pass


class CheckpointConfig:
    def __init__(self):
        self.load_dirpath = None
        self.save_dirpath = None
        self.save_step_interval = 1
        self.error_msg = ""

    def config_load(self, dirpath=None):
        self.load_dirpath = dirpath

    def config_save(self, dirpath=None, step_interval=1):
        if int(step_interval) < 1:
            raise ValueError("step_interval must be at least 1")
        self.save_dirpath, self.save_step_interval = dirpath, int(step_interval)

    def check_valid(self):
        if self.load_dirpath is None and self.save_dirpath is None:
            self.error_msg = "a checkpoint config needs a directory to load from or to save to"
            return False
        return True


class Callback:
    def on_training_step_end(self, outputs, step_idx=0, optimizer_idx=0):
        pass

    def on_validation_step_end(self, outputs, step_idx=0):
        pass


class Model(Module):
    def __init__(self, *args, **kwargs):
        super().__init__()

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def training_step(self, *args, **kwargs):
        raise NotImplementedError

    def validation_step(self, *args, **kwargs):
        raise NotImplementedError

    def configure_optimizers(self):
        raise NotImplementedError

    def method_overrided(self, method_name=None):
        return getattr(type(self), method_name) is not getattr(Model, method_name)

    def fit(self, training_config=None, validation_config=None, checkpoint_config=None, callbacks=None, max_steps=100):
        callbacks = [] if callbacks is None else (list(callbacks) if isinstance(callbacks, (list, tuple)) else [callbacks])
        for cb in callbacks:
            if not isinstance(cb, Callback):
                raise TypeError("callbacks must be Callback instances")
        for cfg, need in ((training_config, ("training_step", "configure_optimizers")), (validation_config, ("validation_step",))):
            if cfg is None:
                continue
            if not cfg.check_valid():
                raise ValueError(cfg.error_msg)
            for name in need:
                if not self.method_overrided(name):
                    raise NotImplementedError(f"model.{name}() is not defined")
        if checkpoint_config is not None and not checkpoint_config.check_valid():
            raise ValueError(checkpoint_config.error_msg)
        optimizers = []
        if training_config is not None:
            conf = self.configure_optimizers()
            optimizers = list(conf) if isinstance(conf, (list, tuple)) else [conf]
            if not optimizers or not all(hasattr(o, "step") and hasattr(o, "zero_grad") for o in optimizers):
                raise TypeError("model.configure_optimizers() must return an optimizer or a list of optimizers")
        if checkpoint_config is not None and checkpoint_config.load_dirpath is not None:
            self.load_state_dict(torch.load(os.path.join(checkpoint_config.load_dirpath, "model.pt")))
        self._max_steps = int(max_steps)
        for step_idx in range(self._max_steps):
            try:
                if training_config is not None:
                    self._train_once(training_config, optimizers, callbacks, step_idx)
                if validation_config is not None and (step_idx + 1) % validation_config.step_interval == 0:
                    self._validate_once(validation_config, callbacks, step_idx)
                if checkpoint_config is not None and checkpoint_config.save_dirpath is not None and \
                        (step_idx + 1) % checkpoint_config.save_step_interval == 0:
                    d = os.path.join(checkpoint_config.save_dirpath, f"step_{step_idx + 1}")
                    os.makedirs(d, exist_ok=True)
                    torch.save(self.state_dict(), os.path.join(d, "model.pt"))
            except Exception:
                print(f"Model step_idx {step_idx} failed.")
                raise

    def _train_once(self, cfg, optimizers, callbacks, step_idx):
        self.train()
        for optimizer_idx, opt in enumerate(optimizers):
            batch = cfg.data(step_idx, optimizer_idx)
            outputs = self.training_step(batch=batch, optimizer_idx=optimizer_idx)
            loss = outputs[0] if isinstance(outputs, tuple) and outputs else outputs
            loss.backward()
            opt.step()
            opt.zero_grad()
            for cb in callbacks:
                cb.on_training_step_end(outputs=outputs, step_idx=step_idx, optimizer_idx=optimizer_idx)

    def _validate_once(self, cfg, callbacks, step_idx):
        was_training = self.training
        self.eval()
        with torch.no_grad():
            outputs = self.validation_step(batch=cfg.data(step_idx, 0))
        self.train(was_training)
        for cb in callbacks:
            cb.on_validation_step_end(outputs=outputs, step_idx=step_idx)
