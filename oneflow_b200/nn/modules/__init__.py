from .fused_mlp import FusedMLP, fused_linear_act  # noqa: F401
from .partial_fc import distributed_partial_fc_sample  # noqa: F401
from .sync_batchnorm import SyncBatchNorm  # noqa: F401
from .conv import Conv2d, conv2d  # noqa: F401
from .compat import (AllReduce, DistributedPariticalFCSample, QatConv1d, QatConv2d, QatConv3d, QuickGELU, RMSLayerNorm,  # noqa: F401
                     SquareReLU)
from .dataset import (COCOReader, CoinFlip, CropMirrorNormalize, GPTIndexedBinDataReader, ImageBatchAlign, ImageDecode,  # noqa: F401
                      ImageFlip, ImageNormalize, ImageResize, OFRecordBytesDecoder, OFRecordImageDecoder,
                      OFRecordImageDecoderRandomCrop, OFRecordImageGpuDecoderRandomCropResize, OFRecordRawDecoder,
                      OFRecordReader, RawReader, RecordBatch, TensorBufferToListOfTensors)


def __getattr__(name):
    """``oneflow.nn.modules.<file>`` for the layer files this package does not define itself: torch.nn.modules'."""
    import importlib
    try:
        return importlib.import_module(f"torch.nn.modules.{name}")
    except ModuleNotFoundError:
        raise AttributeError(f"module 'oneflow.nn.modules' has no attribute {name!r}") from None
