"""MNIST as numpy batches (reference: python/oneflow/experimental/load_mnist.py, which downloads ``mnist.npz``).

There is no download here: ``data_dir`` must hold ``mnist.npz`` (keys x_train, y_train, x_test, y_test, as distributed by
Keras) or the four IDX files of the original distribution (optionally gzip-compressed). Returns
``(train_images, train_labels), (test_images, test_labels)`` as lists of batches: images float32 [batch, 1, 28, 28] scaled
to [0, 1], labels int32 [batch]; a trailing partial batch is dropped, as in the reference."""
from __future__ import annotations

import gzip
import os
import struct

import numpy as np

_IDX = {"x_train": "train-images-idx3-ubyte", "y_train": "train-labels-idx1-ubyte", "x_test": "t10k-images-idx3-ubyte",
        "y_test": "t10k-labels-idx1-ubyte"}


def _read_idx(path):
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        raw = f.read()
    _zero, dtype, ndim = struct.unpack(">HBB", raw[:4])
    if dtype != 0x08:
        raise ValueError(f"{path}: not an unsigned-byte IDX file")
    dims = struct.unpack(">" + "I" * ndim, raw[4:4 + 4 * ndim])
    return np.frombuffer(raw, dtype=np.uint8, offset=4 + 4 * ndim).reshape(dims)


def _find(data_dir):
    npz = os.path.join(data_dir, "mnist.npz")
    if os.path.exists(npz):
        with np.load(npz) as z:
            return {k: z[k] for k in _IDX}
    out = {}
    for key, stem in _IDX.items():
        for name in (stem, stem + ".gz"):
            if os.path.exists(os.path.join(data_dir, name)):
                out[key] = _read_idx(os.path.join(data_dir, name))
                break
        else:
            raise FileNotFoundError(f"no MNIST files under {data_dir}: put mnist.npz or the four IDX files there (nothing is downloaded)")
    return out


def load_mnist(train_batch_size=100, test_batch_size=100, data_dir="./mnist_data", **_unused):
    data = _find(data_dir)

    def batches(images, labels, bs):
        n = images.shape[0] // bs * bs
        x = (images[:n].astype(np.float32) / 255.0).reshape(-1, bs, 1, 28, 28)
        y = labels[:n].astype(np.int32).reshape(-1, bs)
        return list(x), list(y)

    return batches(data["x_train"], data["y_train"], train_batch_size), batches(data["x_test"], data["y_test"], test_batch_size)
