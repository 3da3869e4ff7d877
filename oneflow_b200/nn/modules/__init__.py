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
