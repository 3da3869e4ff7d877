"""Data-loading modules of ``flow.nn``: OFRecord / raw / COCO / Megatron-GPT readers and the record and image
decoders that follow them (reference: python/oneflow/nn/modules/dataset.py:42-1180 and the kernels under
oneflow/user/data and oneflow/user/kernels/{ofrecord_decoder,image_*,crop_mirror_normalize}*).

Layout of the pipeline here:

* a reader module owns prefetching native readers (``runtime.core.RecordReader``: a C++ thread per part file that reads
  the length-framed records ahead and keeps a shuffle buffer) and returns a :class:`RecordBatch` — the serialised
  records of one batch — per call, endlessly (epochs roll over inside the reader);
* decoder modules pick one feature out of every record (``utils.ofrecord``) and give a dense tensor, or a
  ``TensorBuffer`` (a ragged batch) of images / byte strings;
* image modules work on ``TensorBuffer`` batches of HWC uint8 tensors; ``CropMirrorNormalize`` ends the chain with
  one dense float batch, which is what gets copied to the GPU.

With ``placement`` and a ``split(0)`` sbp every rank reads its own share of the part files and of the batch, and the
dense outputs come back as global tensors made of those shards; with ``broadcast`` every rank reads the same data.
"""
from __future__ import annotations

import io
import json
import os
import struct

import numpy as np
import torch
import torch.nn as nn

from ...framework.toplevel_extra import TensorBuffer
from ...utils import ofrecord as _rec


# ------------------------------------------------------------------------------------------------ common plumbing
class RecordBatch(list):
    """The serialised OFRecords of one batch, plus where the batch lives (local device or placement / sbp)."""

    device = torch.device("cpu")
    placement = None
    sbp = None

    def like(self, other):
        self.device, self.placement, self.sbp = other.device, other.placement, other.sbp
        return self


def _seed_of(random_seed):
    return (int(random_seed) if random_seed is not None and int(random_seed) >= 0
            else int.from_bytes(os.urandom(4), "little"))


def _check_dist_args(device, placement, sbp):
    if placement is None:
        if sbp is not None:
            raise ValueError("sbp given without a placement")
        return torch.device(device) if device is not None else torch.device("cpu"), None, None
    if device is not None:
        raise ValueError("give either device or placement, not both")
    if sbp is None:
        raise ValueError("placement given without sbp")
    nd = tuple(sbp) if isinstance(sbp, (tuple, list)) else (sbp,)
    if len(nd) != len(placement.hierarchy):
        raise ValueError(f"{len(nd)} sbp entries for a {len(placement.hierarchy)}-D placement")
    return None, placement, nd


def _shard_of(placement, nd_sbp):
    """(number of data shards, index of this rank's shard): the product over the placement axes split on dim 0."""
    if placement is None:
        return 1, 0
    from ... import env
    rank = env.get_rank()
    flat = list(placement.ranks_flat)
    if rank not in flat:
        return 1, 0
    coords = np.unravel_index(flat.index(rank), placement.hierarchy)
    num, idx = 1, 0
    for axis, s in enumerate(nd_sbp):
        if getattr(s, "kind", None) == "S":
            if s.axis != 0:
                raise ValueError("data readers shard the batch dimension only: use split(0) or broadcast")
            idx = idx * placement.hierarchy[axis] + int(coords[axis])
            num *= placement.hierarchy[axis]
    return num, idx


def _emit(t, src):
    """A dense per-rank batch -> local tensor on the reader's device, or the global tensor made of the shards."""
    if src.placement is None:
        return t.to(src.device) if src.device is not None and t.device != src.device else t
    from ...framework.global_tensor import to_global
    return to_global(t, src.placement, src.sbp, sync_data=False)


class _ShardedSource(nn.Module):
    """Shared constructor logic: device / placement / sbp, the shard of this rank, the per-rank batch size."""

    def _init_dist(self, batch_size, device, placement, sbp):
        self.device, self.placement, self.sbp = _check_dist_args(device, placement, sbp)
        self.shards, self.shard = _shard_of(self.placement, self.sbp)
        if batch_size % self.shards:
            raise ValueError(f"batch size {batch_size} is not divisible by {self.shards} data shards")
        self.batch_size = batch_size
        self.local_batch = batch_size // self.shards

    def _tag(self, batch: RecordBatch):
        batch.device, batch.placement, batch.sbp = self.device, self.placement, self.sbp
        return batch


# ------------------------------------------------------------------------------------------------ OFRecord reader
class OFRecordReader(_ShardedSource):
    """Reads ``data_part_num`` part files ``<dir>/<prefix><i>`` and returns one :class:`RecordBatch` per call.
    Part files are dealt round robin to the data shards; inside a shard they are read one after the other through a
    prefetching native reader with a shuffle buffer of ``shuffle_buffer_size`` records when ``random_shuffle``;
    ``shuffle_after_epoch`` also re-orders the part files at every epoch
    (reference: python/oneflow/nn/modules/dataset.py:42-124, oneflow/user/data/ofrecord_dataset.h:38-130)."""

    def __init__(self, ofrecord_dir, batch_size=1, data_part_num=1, part_name_prefix="part-", part_name_suffix_length=-1,
                 random_shuffle=False, shuffle_buffer_size=1024, shuffle_after_epoch=False, random_seed=-1, device=None,
                 placement=None, sbp=None, name=None):
        super().__init__()
        self._init_dist(batch_size, device, placement, sbp)
        self.ofrecord_dir, self.data_part_num = ofrecord_dir, data_part_num
        self.random_shuffle, self.shuffle_buffer_size = random_shuffle, shuffle_buffer_size
        self.shuffle_after_epoch = shuffle_after_epoch
        self.seed = _seed_of(random_seed)
        fmt = "{}" if part_name_suffix_length < 0 else "{:0" + str(part_name_suffix_length) + "d}"
        files = [os.path.join(ofrecord_dir, part_name_prefix + fmt.format(i)) for i in range(data_part_num)]
        missing = [f for f in files if not os.path.isfile(f)]
        if missing:
            raise FileNotFoundError(f"OFRecord part files not found: {missing[:3]}")
        if data_part_num < self.shards:
            raise ValueError(f"{data_part_num} part files cannot feed {self.shards} data shards")
        self.files = files[self.shard::self.shards]
        self._epoch, self._order, self._cur, self._reader = 0, [], 0, None

    def _open_next(self):
        from ...runtime.core import RecordReader
        if self._reader is not None:
            self._reader.close()
            self._reader = None
        if self._cur >= len(self._order):
            order = list(range(len(self.files)))
            if self.random_shuffle and (self.shuffle_after_epoch or self._epoch == 0):
                np.random.RandomState((self.seed + self._epoch) & 0x7FFFFFFF).shuffle(order)
            elif self._order:
                order = self._order
            self._order, self._cur = order, 0
            self._epoch += 1
        path = self.files[self._order[self._cur]]
        self._cur += 1
        self._reader = RecordReader(path, prefetch=max(2 * self.local_batch, 8),
                                    shuffle_buffer=self.shuffle_buffer_size if self.random_shuffle else 0,
                                    seed=self.seed + 7919 * self._epoch + self._cur)

    def forward(self):
        out = RecordBatch()
        empty_files = 0
        while len(out) < self.local_batch:
            if self._reader is None:
                self._open_next()
            try:
                out.append(next(self._reader))
                empty_files = 0
            except StopIteration:
                self._reader.close()
                self._reader = None
                empty_files += 1
                if empty_files > len(self.files):
                    raise RuntimeError(f"no records in {self.ofrecord_dir}")
        return self._tag(out)

    def __del__(self):
        r = getattr(self, "_reader", None)
        if r is not None:
            try:
                r.close()
            except Exception:               # interpreter shutdown: the native library may already be gone
                pass


# ------------------------------------------------------------------------------------------------ record decoders
_NP_OF_TORCH = {torch.float32: np.float32, torch.float64: np.float64, torch.int32: np.int32, torch.int64: np.int64,
                torch.int8: np.int8, torch.uint8: np.uint8, torch.float16: np.float16, torch.int16: np.int16, torch.bool: np.bool_}


class OFRecordRawDecoder(nn.Module):
    """Feature ``blob_name`` of every record as a dense ``[batch, *shape]`` tensor of ``dtype``.  A feature shorter
    than ``shape`` needs ``dim1_varying_length`` (it is zero padded); a longer one needs ``truncate``
    (reference: python/oneflow/nn/modules/dataset.py:127-165, oneflow/user/kernels/ofrecord_decoder_kernels.cpp)."""

    def __init__(self, blob_name, shape, dtype, dim1_varying_length=False, truncate=False, auto_zero_padding=False, name=None):
        super().__init__()
        self.blob_name, self.shape, self.dtype = blob_name, tuple(int(s) for s in shape), dtype
        self.dim1_varying_length, self.truncate = dim1_varying_length, truncate or auto_zero_padding

    def forward(self, input):
        n = int(np.prod(self.shape)) if self.shape else 1
        npdt = _NP_OF_TORCH.get(self.dtype, np.float32)
        out = np.zeros((len(input), n), dtype=npdt)
        for i, rec in enumerate(input):
            kind, vals = _rec.decode_feature(rec, self.blob_name)
            if kind == "bytes":
                vals = np.frombuffer(b"".join(vals), dtype=npdt)
            if vals.size > n:
                if not self.truncate:
                    raise ValueError(f"feature {self.blob_name!r} has {vals.size} values, more than shape {self.shape}")
                vals = vals[:n]
            elif vals.size < n and not (self.dim1_varying_length or self.truncate):
                raise ValueError(f"feature {self.blob_name!r} has {vals.size} values, fewer than shape {self.shape}")
            out[i, :vals.size] = vals
        return _emit(torch.from_numpy(out.reshape((len(input),) + self.shape)).to(self.dtype), input)


class OFRecordBytesDecoder(nn.Module):
    """Feature ``blob_name`` of every record as raw bytes: a ``TensorBuffer`` of 1-D uint8 tensors
    (reference: python/oneflow/nn/modules/dataset.py:963-1020)."""

    def __init__(self, blob_name, name=None):
        super().__init__()
        self.blob_name = blob_name

    def forward(self, input):
        out = []
        for rec in input:
            kind, vals = _rec.decode_feature(rec, self.blob_name)
            if kind != "bytes":
                raise TypeError(f"feature {self.blob_name!r} is a {kind}_list, not a bytes_list")
            out.append(torch.frombuffer(bytearray(vals[0]), dtype=torch.uint8))
        return TensorBuffer(out)


def _decode_image(data: bytes, color_space: str):
    from PIL import Image
    img = Image.open(io.BytesIO(data))
    cs = color_space.upper()
    if cs == "GRAY":
        return np.array(img.convert("L"))[:, :, None]
    arr = np.array(img.convert("RGB"))
    return arr[:, :, ::-1].copy() if cs == "BGR" else arr


def _random_crop_window(h, w, rng, area, ratio, attempts):
    """Random-resized-crop window (x, y, cw, ch): area fraction and aspect ratio drawn uniformly (the ratio in log
    space), ``attempts`` tries, then the largest centred window with a clamped aspect ratio."""
    for _ in range(attempts):
        target = h * w * rng.uniform(area[0], area[1])
        r = np.exp(rng.uniform(np.log(ratio[0]), np.log(ratio[1])))
        cw, ch = int(round(np.sqrt(target * r))), int(round(np.sqrt(target / r)))
        if 0 < cw <= w and 0 < ch <= h:
            return rng.randint(0, w - cw + 1), rng.randint(0, h - ch + 1), cw, ch
    r = w / h
    if r < ratio[0]:
        cw, ch = w, int(round(w / ratio[0]))
    elif r > ratio[1]:
        cw, ch = int(round(h * ratio[1])), h
    else:
        cw, ch = w, h
    return (w - cw) // 2, (h - ch) // 2, cw, ch


class OFRecordImageDecoder(nn.Module):
    """Decodes the encoded image (JPEG / PNG / ...) stored in feature ``blob_name`` of every record into an HWC uint8
    tensor, channels in ``color_space`` order (reference: python/oneflow/nn/modules/dataset.py:467-480)."""

    def __init__(self, blob_name, color_space="BGR"):
        super().__init__()
        self.blob_name, self.color_space = blob_name, color_space

    def _bytes(self, rec):
        kind, vals = _rec.decode_feature(rec, self.blob_name)
        if kind != "bytes" or not vals:
            raise TypeError(f"feature {self.blob_name!r} holds no encoded image")
        return vals[0]

    def forward(self, input):
        return TensorBuffer([torch.from_numpy(_decode_image(self._bytes(r), self.color_space)) for r in input])


class OFRecordImageDecoderRandomCrop(OFRecordImageDecoder):
    """Decode, then keep a random window of relative area ``random_area`` and aspect ratio ``random_aspect_ratio``
    (reference: python/oneflow/nn/modules/dataset.py:428-464, oneflow/user/image/random_crop_generator.cpp)."""

    def __init__(self, blob_name, color_space="BGR", num_attempts=10, random_seed=None, random_area=(0.08, 1.0),
                 random_aspect_ratio=(0.75, 1.333333)):
        super().__init__(blob_name, color_space)
        self.num_attempts, self.random_area, self.random_aspect_ratio = num_attempts, tuple(random_area), tuple(random_aspect_ratio)
        self.rng = np.random.RandomState(_seed_of(random_seed) & 0x7FFFFFFF)

    def forward(self, input):
        out = []
        for r in input:
            img = _decode_image(self._bytes(r), self.color_space)
            x, y, cw, ch = _random_crop_window(img.shape[0], img.shape[1], self.rng, self.random_area,
                                               self.random_aspect_ratio, self.num_attempts)
            out.append(torch.from_numpy(np.ascontiguousarray(img[y:y + ch, x:x + cw])))
        return TensorBuffer(out)


def _resize_hwc(img: torch.Tensor, h: int, w: int, interpolation="bilinear"):
    mode = {"auto": "bilinear", "bilinear": "bilinear", "nearest_neighbor": "nearest", "nearest": "nearest", "bicubic": "bicubic",
            "area": "area"}[interpolation]
    x = img.permute(2, 0, 1)[None].float()
    kw = {} if mode in ("nearest", "area") else {"align_corners": False}
    y = torch.nn.functional.interpolate(x, size=(h, w), mode=mode, **kw)
    if img.dtype == torch.uint8:
        y = y.round().clamp_(0, 255)
    return y[0].permute(1, 2, 0).to(img.dtype).contiguous()


class OFRecordImageGpuDecoderRandomCropResize(nn.Module):
    """Decode + random crop + resize to ``target_width`` x ``target_height`` in one module; takes the byte buffers of
    :class:`OFRecordBytesDecoder` and returns one dense uint8 ``[batch, H, W, 3]`` RGB tensor.  The reference decodes
    with nvJPEG inside ``nn.Graph`` only; here decoding runs on host threads, the resize on the batch's device
    (reference: python/oneflow/nn/modules/dataset.py:483-550)."""

    def __init__(self, target_width, target_height, num_attempts=10, seed=0, random_area=(0.08, 1.0),
                 random_aspect_ratio=(0.75, 1.333333), num_workers=3, warmup_size=6400, max_num_pixels=67108864):
        super().__init__()
        if len(random_area) != 2 or len(random_aspect_ratio) != 2:
            raise ValueError("random_area and random_aspect_ratio are (min, max) pairs")
        self.target_width, self.target_height, self.num_attempts = target_width, target_height, num_attempts
        self.random_area, self.random_aspect_ratio = tuple(random_area), tuple(random_aspect_ratio)
        self.num_workers, self.max_num_pixels = max(int(num_workers), 1), max_num_pixels
        self.rng = np.random.RandomState(int(seed) & 0x7FFFFFFF)
        self._pool = None

    def _one(self, args):
        data, seed = args
        img = _decode_image(bytes(data.numpy().tobytes()), "RGB")
        if img.shape[0] * img.shape[1] > self.max_num_pixels:
            raise ValueError(f"image of {img.shape[0]}x{img.shape[1]} pixels exceeds max_num_pixels")
        x, y, cw, ch = _random_crop_window(img.shape[0], img.shape[1], np.random.RandomState(seed), self.random_area,
                                           self.random_aspect_ratio, self.num_attempts)
        return _resize_hwc(torch.from_numpy(np.ascontiguousarray(img[y:y + ch, x:x + cw])), self.target_height, self.target_width)

    def forward(self, input):
        from concurrent.futures import ThreadPoolExecutor
        if self._pool is None:
            self._pool = ThreadPoolExecutor(self.num_workers)
        seeds = self.rng.randint(0, 2 ** 31 - 1, size=len(input.tensors))
        return torch.stack(list(self._pool.map(self._one, zip(input.tensors, seeds))))


# ------------------------------------------------------------------------------------------------ image ops
class ImageDecode(nn.Module):
    """Byte buffers -> HWC image tensors (reference: python/oneflow/nn/modules/dataset.py:842-852)."""

    def __init__(self, dtype=torch.uint8, color_space="BGR"):
        super().__init__()
        self.dtype, self.color_space = dtype, color_space

    def forward(self, input):
        return TensorBuffer([torch.from_numpy(_decode_image(t.numpy().tobytes(), self.color_space)).to(self.dtype)
                             for t in input.tensors])


class ImageResize(nn.Module):
    """Resize every image of a buffer.  Fixed mode: ``target_size=(width, height)`` -> dense ``[batch, h, w, c]`` tensor
    and the per-image ``(w_scale, h_scale)``.  ``keep_aspect_ratio``: ``target_size`` is the length of the shorter (or
    longer) side, bounded by ``min_size`` / ``max_size`` of the other side; returns the resized buffer, scales and the
    new ``(w, h)`` sizes (reference: python/oneflow/nn/modules/dataset.py:584-733,
    oneflow/user/kernels/image_resize_kernels.cpp)."""

    def __init__(self, target_size=None, min_size=None, max_size=None, keep_aspect_ratio=False, resize_side="shorter",
                 channels=3, dtype=None, interpolation_type="auto", name=None, color_space=None, interp_type=None,
                 resize_shorter=0, resize_x=0, resize_y=0):
        super().__init__()
        if color_space is not None:
            channels = 1 if color_space.upper() == "GRAY" else 3
        if interp_type is not None:
            interpolation_type = {"Linear": "bilinear", "NN": "nearest_neighbor", "Cubic": "bicubic"}[interp_type]
        if resize_x > 0 and resize_y > 0:
            target_size, keep_aspect_ratio = (resize_x, resize_y), False
        if resize_shorter > 0:
            target_size, keep_aspect_ratio, resize_side = resize_shorter, True, "shorter"
        self.channels, self.interpolation_type, self.keep_aspect_ratio = channels, interpolation_type, keep_aspect_ratio
        if keep_aspect_ratio:
            if not isinstance(target_size, int):
                raise ValueError("target_size must be an int when keep_aspect_ratio is True")
            if resize_side not in ("shorter", "longer"):
                raise ValueError('resize_side must be "shorter" or "longer"')
            self.target_size, self.min_size, self.max_size = target_size, min_size or 0, max_size or 0
            self.resize_longer = resize_side == "longer"
        else:
            if not isinstance(target_size, (list, tuple)) or len(target_size) != 2 or not all(isinstance(s, int) for s in target_size):
                raise ValueError("target_size must be (width, height) when keep_aspect_ratio is False")
            self.target_w, self.target_h = target_size
            self.dtype = dtype if dtype is not None else torch.uint8

    def _aspect_size(self, h, w):
        short, long = (min(h, w), max(h, w))
        if self.resize_longer:
            new_long = self.target_size
            new_short = int(round(short * new_long / long))
            if self.min_size and new_short < self.min_size:
                new_short, new_long = self.min_size, int(round(long * self.min_size / short))
        else:
            new_short = self.target_size
            new_long = int(round(long * new_short / short))
            if self.max_size and new_long > self.max_size:
                new_long, new_short = self.max_size, int(round(short * self.max_size / long))
        return (new_short, new_long) if h <= w else (new_long, new_short)

    def forward(self, input):
        imgs = input.tensors
        if self.keep_aspect_ratio:
            out, scale, size = [], [], []
            for im in imgs:
                nh, nw = self._aspect_size(im.shape[0], im.shape[1])
                out.append(_resize_hwc(im, nh, nw, self.interpolation_type))
                scale.append([nw / im.shape[1], nh / im.shape[0]])
                size.append([nw, nh])
            return TensorBuffer(out), torch.tensor(scale, dtype=torch.float32), torch.tensor(size, dtype=torch.int32)
        out = torch.stack([_resize_hwc(im, self.target_h, self.target_w, self.interpolation_type).to(self.dtype) for im in imgs])
        scale = torch.tensor([[self.target_w / im.shape[1], self.target_h / im.shape[0]] for im in imgs], dtype=torch.float32)
        return out, scale, None


class ImageFlip(nn.Module):
    """Flip each image by its code: 0 none, 1 horizontal, 2 vertical, 3 both
    (reference: python/oneflow/nn/modules/dataset.py:784-839, image_object_preprocess_kernels.cpp:26-52)."""

    def forward(self, images, flip_code):
        codes = (torch.as_tensor(flip_code).reshape(-1).tolist() if not isinstance(flip_code, int)
                 else [flip_code] * len(images.tensors))
        out = []
        for im, c in zip(images.tensors, codes):
            dims = [d for d, bit in ((1, 1), (0, 2)) if int(c) & bit]
            out.append(torch.flip(im, dims) if dims else im)
        return TensorBuffer(out)


class ImageNormalize(nn.Module):
    """``(x - mean) / std`` per channel on every image of a buffer, result float32
    (reference: python/oneflow/nn/modules/dataset.py:855-865)."""

    def __init__(self, std, mean):
        super().__init__()
        self.std, self.mean = torch.tensor(std, dtype=torch.float32), torch.tensor(mean, dtype=torch.float32)

    def forward(self, input):
        return TensorBuffer([(im.float() - self.mean) / self.std for im in input.tensors])


class ImageBatchAlign(nn.Module):
    """Pads the images of a buffer (top-left aligned, zeros) to the largest height and width of the batch rounded up
    to ``alignment`` and stacks them into ``[batch, H, W, C]``
    (reference: python/oneflow/nn/modules/dataset.py:942-960, oneflow/user/kernels/image_batch_align_kernel.cpp)."""

    def __init__(self, shape, dtype, alignment):
        super().__init__()
        self.shape, self.dtype, self.alignment = tuple(shape), dtype, int(alignment)

    def forward(self, input):
        imgs = input.tensors
        a = self.alignment
        H = -(-max(i.shape[0] for i in imgs) // a) * a
        W = -(-max(i.shape[1] for i in imgs) // a) * a
        C = imgs[0].shape[2]
        out = torch.zeros((len(imgs), H, W, C), dtype=self.dtype)
        for n, im in enumerate(imgs):
            if im.shape[2] != C:
                raise ValueError("images of one batch must have the same number of channels")
            out[n, :im.shape[0], :im.shape[1]] = im.to(self.dtype)
        return out


class TensorBufferToListOfTensors(nn.Module):
    """The entries of a buffer as a list of tensors reshaped / cast to ``out_shapes`` / ``out_dtypes``
    (reference: python/oneflow/nn/modules/dataset.py:553-581)."""

    def __init__(self, out_shapes, out_dtypes, out_num=1, dynamic_out=False):
        super().__init__()
        self.out_shapes, self.out_dtypes, self.dynamic_out = out_shapes, out_dtypes, dynamic_out

    def forward(self, input):
        out = []
        for i, t in enumerate(input.tensors):
            dt = self.out_dtypes[i] if isinstance(self.out_dtypes, (list, tuple)) else self.out_dtypes
            t = t.to(dt)
            if not self.dynamic_out:
                shape = tuple(self.out_shapes[i])
                pad = torch.zeros(shape, dtype=dt)
                pad.reshape(-1)[:t.numel()] = t.reshape(-1)[:pad.numel()]
                t = pad
            out.append(t)
        return out


class CoinFlip(_ShardedSource):
    """A batch of independent 0/1 draws with P(1) = ``probability`` as int8 ``[batch]`` — the mirror flags of
    :class:`CropMirrorNormalize` (reference: python/oneflow/nn/modules/dataset.py:168-261)."""

    def __init__(self, batch_size=1, random_seed=None, probability=0.5, device=None, placement=None, sbp=None):
        super().__init__()
        self._init_dist(batch_size, device, placement, sbp)
        self.probability = float(probability)
        self.gen = torch.Generator().manual_seed((_seed_of(random_seed) + 104729 * self.shard) & 0x7FFFFFFF)

    def forward(self):
        flags = (torch.rand(self.local_batch, generator=self.gen) < self.probability).to(torch.int8)
        return _emit(flags, self)


class CropMirrorNormalize(nn.Module):
    """Crop (``crop_h`` x ``crop_w`` at the relative position ``crop_pos_*`` of the free range; 0 keeps the full side),
    mirror where the per-image flag is set, normalise per channel and lay the batch out as float NCHW (NHWC when the
    environment variable ``ONEFLOW_ENABLE_NHWC`` is 1).  Input: a uint8 ``[batch, H, W, C]`` tensor or a buffer of
    equally sized HWC images (reference: python/oneflow/nn/modules/dataset.py:264-425,
    oneflow/user/kernels/crop_mirror_normalize_kernel.cu).  One fused pass over the batch on the device the input
    lives on: a dense input already on the GPU is cropped, flipped and normalised there."""

    def __init__(self, color_space="BGR", output_layout="NCHW", crop_h=0, crop_w=0, crop_pos_y=0.5, crop_pos_x=0.5,
                 mean=(0.0,), std=(1.0,), output_dtype=torch.float32):
        super().__init__()
        self.color_space = color_space
        self.output_layout = "NHWC" if os.getenv("ONEFLOW_ENABLE_NHWC") == "1" else "NCHW"
        self.crop_h, self.crop_w, self.crop_pos_y, self.crop_pos_x = crop_h, crop_w, crop_pos_y, crop_pos_x
        self.mean, self.std, self.output_dtype = list(mean), list(std), output_dtype

    def forward(self, input, mirror=None):
        src = None
        if isinstance(input, TensorBuffer):
            imgs = input.tensors
            if any(i.shape != imgs[0].shape for i in imgs):
                ch, cw = self.crop_h or min(i.shape[0] for i in imgs), self.crop_w or min(i.shape[1] for i in imgs)
                imgs = [self._crop(i, ch, cw) for i in imgs]
            x = torch.stack(imgs)
        else:
            from ...framework.global_tensor import GlobalTensor
            if isinstance(input, GlobalTensor):
                src, x = input, input.to_local()
            else:
                x = input
            if x.dtype != torch.uint8:
                raise NotImplementedError(f"CropMirrorNormalize does not take {x.dtype} input")
        x = self._crop(x, self.crop_h or x.shape[-3], self.crop_w or x.shape[-2])
        C = x.shape[-1]
        mean = torch.tensor(self.mean if len(self.mean) == C else self.mean * C, dtype=torch.float32, device=x.device)
        std = torch.tensor(self.std if len(self.std) == C else self.std * C, dtype=torch.float32, device=x.device)
        y = (x.float() - mean) / std
        if mirror is not None:
            m = mirror.to_local() if hasattr(mirror, "to_local") and not isinstance(mirror, torch.Tensor) else mirror
            m = torch.as_tensor(m).to(x.device).bool().reshape(-1, 1, 1, 1)
            y = torch.where(m, y.flip(2), y)
        if self.output_layout == "NCHW":
            y = y.permute(0, 3, 1, 2)
        y = y.contiguous().to(self.output_dtype)
        if src is not None:
            from ...framework.global_tensor import to_global
            return to_global(y, src.placement, src.sbp, sync_data=False)
        return y

    def _crop(self, x, ch, cw):
        H, W = x.shape[-3], x.shape[-2]
        if ch > H or cw > W:
            raise ValueError(f"crop {ch}x{cw} is larger than the image {H}x{W}")
        y0, x0 = int(round((H - ch) * self.crop_pos_y)), int(round((W - cw) * self.crop_pos_x))
        return x[..., y0:y0 + ch, x0:x0 + cw, :]


# ------------------------------------------------------------------------------------------------ raw reader
class RawReader(_ShardedSource):
    """Fixed-size binary samples: every file is a flat array of ``shape`` x ``dtype`` records, memory mapped.  Shuffling
    permutes blocks of ``shuffle_block_size`` consecutive samples (0: one block per batch) so that reads stay
    sequential inside a block (reference: python/oneflow/nn/modules/dataset.py:1104-1160,
    oneflow/user/kernels/raw_reader_kernel.cpp)."""

    def __init__(self, files, shape, dtype, batch_size, random_shuffle=True, shuffle_block_size=0, random_seed=None,
                 placement=None, sbp=None):
        super().__init__()
        self._init_dist(batch_size, None, placement, sbp)
        self.files, self.shape, self.dtype = list(files), tuple(int(s) for s in shape), dtype
        self.shuffle, self.random_seed = bool(random_shuffle), _seed_of(random_seed)
        npdt = np.dtype(_NP_OF_TORCH[dtype])
        self._sample_elems = int(np.prod(self.shape)) if self.shape else 1
        self._maps, counts = [], []
        for f in self.files:
            size = os.path.getsize(f)
            n = size // (self._sample_elems * npdt.itemsize)
            if n == 0:
                continue
            self._maps.append(np.memmap(f, dtype=npdt, mode="r", shape=(n, self._sample_elems)))
            counts.append(n)
        self._starts = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        self.num_samples = int(self._starts[-1])
        if self.num_samples < batch_size:
            raise ValueError(f"{self.num_samples} samples in the files, fewer than one batch of {batch_size}")
        self.shuffle_block_size = int(shuffle_block_size) if shuffle_block_size > 0 else batch_size
        self._epoch, self._pos, self._order = 0, 0, None

    def _new_epoch(self):
        idx = np.arange(self.num_samples, dtype=np.int64)
        if self.shuffle:
            bs = self.shuffle_block_size
            nblocks = -(-self.num_samples // bs)
            perm = np.random.RandomState((self.random_seed + self._epoch) & 0x7FFFFFFF).permutation(nblocks)
            idx = np.concatenate([idx[b * bs:(b + 1) * bs] for b in perm])
        self._order, self._pos = idx, 0
        self._epoch += 1

    def forward(self):
        if self._order is None or self._pos + self.batch_size > self.num_samples:
            self._new_epoch()                                   # a ragged tail is dropped, as the reference does
        lo = self._pos + self.shard * self.local_batch
        ids = self._order[lo:lo + self.local_batch]
        self._pos += self.batch_size
        out = np.empty((self.local_batch, self._sample_elems), dtype=self._maps[0].dtype)
        which = np.searchsorted(self._starts, ids, side="right") - 1
        for f in np.unique(which):
            sel = which == f
            out[sel] = self._maps[f][ids[sel] - self._starts[f]]
        return _emit(torch.from_numpy(out.reshape((self.local_batch,) + self.shape)), self)


# ------------------------------------------------------------------------------------------------ Megatron GPT reader
_MEGATRON_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}


class MegatronIndexedDataset:
    """A Megatron ``.idx`` / ``.bin`` pair: the index holds, per sentence, its length and byte address, and the
    document boundaries; the data file is memory mapped (reference: oneflow/user/data/gpt_dataset.cpp:79-118)."""

    MAGIC = b"MMIDIDX\x00\x00"

    def __init__(self, prefix):
        with open(prefix + ".idx", "rb") as f:
            if f.read(9) != self.MAGIC:
                raise ValueError(f"{prefix}.idx is not a Megatron index file")
            (self.version,) = struct.unpack("<Q", f.read(8))
            (code,) = struct.unpack("<B", f.read(1))
            n_sizes, n_docs = struct.unpack("<QQ", f.read(16))
            self.sizes = np.frombuffer(f.read(4 * n_sizes), dtype=np.int32)
            self.addresses = np.frombuffer(f.read(8 * n_sizes), dtype=np.int64)
            self.doc_offsets = np.frombuffer(f.read(8 * n_docs), dtype=np.int64)
        self.dtype = np.dtype(_MEGATRON_DTYPES[code])
        self.data = np.memmap(prefix + ".bin", dtype=self.dtype, mode="r")

    @staticmethod
    def write(prefix, docs, dtype=np.uint16):
        """Writes documents (token arrays, one sentence per document) in this format."""
        code = {v: k for k, v in _MEGATRON_DTYPES.items()}[np.dtype(dtype).type]
        sizes = np.array([len(d) for d in docs], dtype=np.int32)
        addresses = np.concatenate([[0], np.cumsum(sizes[:-1].astype(np.int64) * np.dtype(dtype).itemsize)]).astype(np.int64)
        with open(prefix + ".bin", "wb") as f:
            for d in docs:
                f.write(np.asarray(d, dtype=dtype).tobytes())
        with open(prefix + ".idx", "wb") as f:
            f.write(MegatronIndexedDataset.MAGIC + struct.pack("<Q", 1) + struct.pack("<B", code))
            f.write(struct.pack("<QQ", len(docs), len(docs) + 1))
            f.write(sizes.tobytes() + addresses.tobytes() + np.arange(len(docs) + 1, dtype=np.int64).tobytes())


class GPTIndexedBinDataReader(_ShardedSource):
    """Token samples of ``seq_length + 1`` from a Megatron indexed dataset: the documents of the chosen split are
    repeated for as many epochs as ``num_samples`` needs, concatenated (each epoch's document order shuffled), cut
    every ``seq_length`` tokens with one token of overlap, and the samples are shuffled; a trailing partial epoch is
    shuffled apart when it is short (reference: python/oneflow/nn/modules/dataset.py:1023-1101,
    oneflow/user/data/gpt_dataset.cpp:31-245).  Sample starts come from one cumulative sum over the document lengths
    rather than a walk per sample."""

    def __init__(self, data_file_prefix, seq_length, num_samples, batch_size, dtype=torch.int64, shuffle=True,
                 random_seed=None, split_sizes=None, split_index=None, device=None, placement=None, sbp=None):
        super().__init__()
        self._init_dist(batch_size, device, placement, sbp)
        self.seq_length, self.num_samples, self.dtype = int(seq_length), int(num_samples), dtype
        self.shuffle, self.random_seed = bool(shuffle), _seed_of(random_seed)
        split_sizes = tuple(split_sizes) if split_sizes is not None else (1,)
        split_index = 0 if split_index is None else int(split_index)
        if split_index >= len(split_sizes):
            raise ValueError(f"split index {split_index} is out of range, split_sizes {split_sizes}")
        self.index = MegatronIndexedDataset(data_file_prefix)
        rng = np.random.RandomState(self.random_seed & 0x7FFFFFFF)
        ndocs = len(self.index.doc_offsets) - 1
        total = float(sum(split_sizes))
        bounds = np.concatenate([[0], np.cumsum([int(np.rint(np.float32(s / total) * ndocs)) for s in split_sizes])])
        docs = np.arange(bounds[split_index], min(bounds[split_index + 1], ndocs), dtype=np.int64)
        doc_len = np.add.reduceat(self.index.sizes.astype(np.int64), self.index.doc_offsets[:-1])[docs] if len(docs) else np.zeros(0, np.int64)
        tokens_per_epoch = int(doc_len.sum())
        if tokens_per_epoch <= 1:
            raise ValueError("the chosen split holds no tokens")
        L, N = self.seq_length, self.num_samples
        epochs = int(np.ceil((N * L + 1) / tokens_per_epoch))
        complete = epochs
        if epochs > 1:
            per_epoch = (tokens_per_epoch - 1) // L
            last = N - ((epochs - 1) * tokens_per_epoch - 1) // L
            complete = epochs - 1 if last < int(0.8 * per_epoch) else epochs
        order = []
        for span in ([complete] if complete == epochs else [complete, 1]):
            o = np.tile(docs, span)
            if self.shuffle:
                rng.shuffle(o)
            order.append(o)
        self._doc_order = np.concatenate(order)
        self._doc_start = self.index.addresses[self.index.doc_offsets[:-1]] // self.index.dtype.itemsize   # first token of a doc
        lens = np.add.reduceat(self.index.sizes.astype(np.int64), self.index.doc_offsets[:-1])[self._doc_order]
        self._cum = np.concatenate([[0], np.cumsum(lens)])
        total_samples = (epochs * tokens_per_epoch - 1) // L
        sh = np.arange(total_samples, dtype=np.int64)
        if self.shuffle:
            first = (complete * tokens_per_epoch - 1) // L
            rng.shuffle(sh[:first])
            if complete != epochs:
                rng.shuffle(sh[first:])
        self._shuffle_idx, self._cursor = sh, 0

    def sample(self, i):
        """Tokens ``[i * seq_length, i * seq_length + seq_length]`` of the concatenated stream, across documents."""
        lo, hi = i * self.seq_length, i * self.seq_length + self.seq_length + 1
        d = int(np.searchsorted(self._cum, lo, side="right") - 1)
        parts, pos = [], lo
        while pos < hi:
            take = int(min(hi, self._cum[d + 1]) - pos)
            s = int(self._doc_start[self._doc_order[d]] + (pos - self._cum[d]))
            parts.append(self.index.data[s:s + take])
            pos += take
            d += 1
        return np.concatenate(parts)

    def forward(self):
        n = len(self._shuffle_idx)
        out = np.empty((self.local_batch, self.seq_length + 1), dtype=np.int64)
        base = self._cursor + self.shard * self.local_batch
        for b in range(self.local_batch):
            out[b] = self.sample(int(self._shuffle_idx[(base + b) % n]))
        self._cursor = (self._cursor + self.batch_size) % n
        return _emit(torch.from_numpy(out).to(self.dtype), self)


# ------------------------------------------------------------------------------------------------ COCO reader
class COCOReader(_ShardedSource):
    """COCO detection data: per batch the encoded image bytes (decode with :class:`ImageDecode`), image ids, image
    sizes ``(h, w)``, ground-truth boxes as xyxy clipped to the image, contiguous labels (1-based, by ascending
    category id), polygon points and their ``(point, polygon, object)`` indices.  Crowd objects are skipped; images
    without usable annotations can be dropped; ``group_by_aspect_ratio`` fills a batch with images of one orientation
    (reference: python/oneflow/nn/modules/dataset.py:868-939, oneflow/user/data/coco_data_reader.{h,cpp})."""

    def __init__(self, annotation_file, image_dir, batch_size, shuffle=True, random_seed=None, group_by_aspect_ratio=True,
                 remove_images_without_annotations=True, stride_partition=True, device=None, placement=None, sbp=None):
        super().__init__()
        self._init_dist(batch_size, device, placement, sbp)
        self.image_dir, self.shuffle, self.group = image_dir, bool(shuffle), bool(group_by_aspect_ratio)
        self.rng = np.random.RandomState(_seed_of(random_seed) & 0x7FFFFFFF)
        with open(annotation_file) as f:
            meta = json.load(f)
        self.images = {im["id"]: im for im in meta["images"]}
        self.annos = {i: [] for i in self.images}
        for a in meta["annotations"]:
            if a.get("iscrowd", 0) == 1 or a["image_id"] not in self.annos:
                continue
            self.annos[a["image_id"]].append(a)
        self.cat = {c: i + 1 for i, c in enumerate(sorted(c["id"] for c in meta["categories"]))}
        ids = sorted(self.images)
        if remove_images_without_annotations:
            ids = [i for i in ids if self._valid(i)]
        # partition over the data shards: strided or contiguous
        ids = ids[self.shard::self.shards] if stride_partition else \
            ids[len(ids) * self.shard // self.shards:len(ids) * (self.shard + 1) // self.shards]
        if not ids:
            raise ValueError("no images left for this rank")
        self.ids, self._queue = ids, []

    def _valid(self, image_id):
        annos = self.annos[image_id]
        if not annos:
            return False
        return any(a["bbox"][2] > 1 and a["bbox"][3] > 1 for a in annos)

    def _refill(self):
        order = list(self.ids)
        if self.shuffle:
            self.rng.shuffle(order)
        self._queue.extend(order)

    def _take(self):
        while len(self._queue) < self.local_batch:
            self._refill()
        if not self.group:
            batch, self._queue = self._queue[:self.local_batch], self._queue[self.local_batch:]
            return batch
        wide = lambda i: self.images[i]["width"] >= self.images[i]["height"]  # noqa: E731
        want = wide(self._queue[0])
        batch, rest = [], []
        for pos, i in enumerate(self._queue):
            if len(batch) < self.local_batch and wide(i) == want:
                batch.append(i)
            else:
                rest.append(i)
            if len(batch) == self.local_batch:
                rest.extend(self._queue[pos + 1:])
                break
        self._queue = rest
        if len(batch) < self.local_batch:            # not enough of this orientation queued yet: top up next epoch
            self._refill()
            self._queue = batch + self._queue
            return self._take()
        return batch

    def forward(self):
        batch = self._take()
        image, bbox, label, segm, segm_index = [], [], [], [], []
        for i in batch:
            info = self.images[i]
            with open(os.path.join(self.image_dir, info["file_name"]), "rb") as f:
                image.append(torch.frombuffer(bytearray(f.read()), dtype=torch.uint8))
            W, H = float(info["width"]), float(info["height"])
            boxes, labels, pts, idx = [], [], [], []
            obj = 0
            for a in self.annos[i]:
                l, t, w, h = (float(v) for v in a["bbox"])
                r, b = l + max(w - 1, 0), t + max(h - 1, 0)
                l, r = min(max(l, 0), W - 1), min(max(r, 0), W - 1)
                t, b = min(max(t, 0), H - 1), min(max(b, 0), H - 1)
                if not (r > l and b > t):
                    continue
                boxes.append([l, t, r, b])
                labels.append(self.cat[a["category_id"]])
                if isinstance(a.get("segmentation"), list):
                    for p, poly in enumerate(a["segmentation"]):
                        for k in range(len(poly) // 2):
                            pts.append([poly[2 * k], poly[2 * k + 1]])
                            idx.append([k, p, obj])
                obj += 1
            bbox.append(torch.tensor(boxes, dtype=torch.float32).reshape(-1, 4))
            label.append(torch.tensor(labels, dtype=torch.int32))
            segm.append(torch.tensor(pts, dtype=torch.float32).reshape(-1, 2))
            segm_index.append(torch.tensor(idx, dtype=torch.int32).reshape(-1, 3))
        image_id = _emit(torch.tensor(batch, dtype=torch.int64), self)
        image_size = _emit(torch.tensor([[self.images[i]["height"], self.images[i]["width"]] for i in batch], dtype=torch.int32), self)
        return (TensorBuffer(image), image_id, image_size, TensorBuffer(bbox), TensorBuffer(label), TensorBuffer(segm),
                TensorBuffer(segm_index))


# ------------------------------------------------------------------------------------------------ functional spellings
def raw_decoder(input_record, blob_name, shape, dtype, dim1_varying_length=False, truncate=False, auto_zero_padding=False,
                name=None):
    return OFRecordRawDecoder(blob_name, shape, dtype, dim1_varying_length, truncate or auto_zero_padding)(input_record)


def get_ofrecord_handle(ofrecord_dir, batch_size=1, data_part_num=1, part_name_prefix="part-", part_name_suffix_length=-1,
                        random_shuffle=False, shuffle_buffer_size=1024, shuffle_after_epoch=False, name=None):
    return OFRecordReader(ofrecord_dir, batch_size, data_part_num, part_name_prefix, part_name_suffix_length,
                          random_shuffle, shuffle_buffer_size, shuffle_after_epoch)()


def tensor_buffer_to_list_of_tensors(tensor, out_shapes, out_dtypes):
    return TensorBufferToListOfTensors([list(s) for s in out_shapes], out_dtypes, len(out_shapes))(tensor)
