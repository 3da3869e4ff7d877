"""``oneflow.nn.optimizer.<name>``: the per-file import paths of the reference's optimizers and learning-rate
schedulers (python/oneflow/nn/optimizer/*.py), each a small module that holds the class of ``flow.optim`` /
``flow.optim.lr_scheduler`` under the same name."""
import sys as _sys
import types as _types

from ... import optim as _optim
from ...optim import lr_scheduler as _lrs

_FILES = {
    "adadelta": (_optim, ["Adadelta"]), "adagrad": (_optim, ["Adagrad"]), "adam": (_optim, ["Adam"]),
    "adamw": (_optim, ["AdamW"]), "lamb": (_optim, ["LAMB"]), "lbfgs": (_optim, ["LBFGS"]),
    "rmsprop": (_optim, ["RMSprop"]), "sgd": (_optim, ["SGD"]), "ftrl": (_optim, ["Ftrl"]), "swa_utils": (_optim.swa_utils, ["AveragedModel", "SWALR", "update_bn"]),
    "lr_scheduler": (_lrs, ["LRScheduler"]), "chained_scheduler": (_lrs, ["ChainedScheduler"]),
    "constant_lr": (_lrs, ["ConstantLR"]), "cosine_annealing_lr": (_lrs, ["CosineAnnealingLR"]),
    "cosine_annealing_warm_restarts": (_lrs, ["CosineAnnealingWarmRestarts"]), "cosine_decay_lr": (_lrs, ["CosineDecayLR"]),
    "exponential_lr": (_lrs, ["ExponentialLR"]), "lambda_lr": (_lrs, ["LambdaLR"]), "linear_lr": (_lrs, ["LinearLR"]),
    "multiplicative_lr": (_lrs, ["MultiplicativeLR"]), "multistep_lr": (_lrs, ["MultiStepLR"]),
    "polynomial_lr": (_lrs, ["PolynomialLR"]), "reduce_lr_on_plateau": (_lrs, ["ReduceLROnPlateau"]),
    "sequential_lr": (_lrs, ["SequentialLR"]), "step_lr": (_lrs, ["StepLR"]), "warmup_lr": (_lrs, ["WarmupLR", "WarmUpLR"]),
}

for _file, (_src, _names) in _FILES.items():
    _m = _types.ModuleType(f"{__name__}.{_file}")
    for _n in _names:
        setattr(_m, _n, getattr(_src, _n))
    _sys.modules[_m.__name__] = _m
    globals()[_file] = _m
del _file, _src, _names, _m, _n
