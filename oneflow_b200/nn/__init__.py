"""``flow.nn``: torch.nn's layers (Module, Linear, Conv*, norms, RNNs, losses, ...) under the flow names,
plus what the reference adds: ``Graph``, ``parallel.DistributedDataParallel``, ``FusedMLP``,
``Module.to_global / to_local``, ``utils.clip_grad_norm_`` aware of global tensors, and the few layers
torch lacks (``CombinedMarginLoss``, ``FusedBatchNorm*`` aliases, ``RMSNorm`` when missing)."""
import torch as _torch
import torch.nn as _tnn
from torch.nn import *  # noqa: F401,F403
from torch.nn import Module  # noqa: F401

import importlib as _importlib

# ``from torch.nn import *`` above bound torch's functional / init / utils / parallel / modules under these names, and
# ``from . import x`` would keep an attribute that already exists — import this package's sub-modules explicitly.
for _n in ("functional", "init", "graph", "module_ext", "parallel", "utils", "modules"):
    globals()[_n] = _importlib.import_module(__name__ + "." + _n)
del _n
from .graph import Graph  # noqa: F401
from .modules import FusedMLP, SyncBatchNorm, distributed_partial_fc_sample  # noqa: F401
from .modules.nhwc import AvgPool2d, BatchNorm2d, Conv2d, MaxPool2d  # noqa: F401  (layout by ONEFLOW_ENABLE_NHWC)
from .modules.native_layers import Embedding, LayerNorm, Linear  # noqa: F401  (forward on the native kernels)
from .modules import (AllReduce, COCOReader, CoinFlip, CropMirrorNormalize, DistributedPariticalFCSample,  # noqa: F401
                      GPTIndexedBinDataReader, OFRecordBytesDecoder, OFRecordImageDecoder, OFRecordImageDecoderRandomCrop,
                      OFRecordImageGpuDecoderRandomCropResize, OFRecordRawDecoder, OFRecordReader, QatConv1d, QatConv2d,
                      QatConv3d, QuickGELU, RawReader, RMSLayerNorm, SquareReLU)
image = _importlib.import_module(__name__ + ".image")
qat = _importlib.import_module(__name__ + ".qat")

OfrecordReader, OfrecordRawDecoder = OFRecordReader, OFRecordRawDecoder
from .extra_modules import (CombinedMarginLoss, FusedBatchNorm1d, FusedBatchNorm2d, FusedBatchNorm3d, MinMaxObserver,  # noqa: F401
                            MovingAverageMinMaxObserver, FakeQuantization, Quantization)



Parameter = _tnn.Parameter        # global tensors become parameters through torch's ``_is_param`` protocol


class _ParameterStandin:
    """What a parameter is written as inside a checkpoint: an object of the class path ``oneflow.nn.Parameter`` that
    carries the reference's tensor state (``framework.check_point`` writes the class path itself)."""
    _pickle_state = None

    def __getstate__(self):
        return self._pickle_state


_ParameterStandin.__module__, _ParameterStandin.__name__, _ParameterStandin.__qualname__ = "oneflow.nn", "Parameter", "Parameter"
module_ext.install()
GraphModule = graph.GraphModule


def __getattr__(name):
    return getattr(_tnn, name)
