"""OFRecord codec: the record format of the reference's datasets, without a protobuf runtime.

An OFRecord is the protobuf message ``OFRecord { map<string, Feature> feature = 1; }`` where a ``Feature`` holds one
of ``bytes_list = 1``, ``float_list = 2``, ``double_list = 3``, ``int32_list = 4``, ``int64_list = 5`` and every list
is ``repeated value = 1`` (packed for the numeric kinds) — reference: oneflow/core/record/record.proto:4-37.
A dataset file is a sequence of ``[int64 little-endian length][serialised OFRecord]`` frames
(reference: oneflow/user/data/ofrecord_dataset.h:94-100), which is the framing of ``runtime.core.RecordReader``.

Numeric lists decode into numpy arrays with vectorised varint decoding, so a record of a few thousand ids costs a
handful of numpy calls rather than a Python loop per element.
"""
from __future__ import annotations

import struct

import numpy as np

_KIND_OF_FIELD = {1: "bytes", 2: "float", 3: "double", 4: "int32", 5: "int64"}
_FIELD_OF_KIND = {v: k for k, v in _KIND_OF_FIELD.items()}


# ------------------------------------------------------------------------------------------------ wire helpers
def _put_varint(out: bytearray, v: int):
    v &= (1 << 64) - 1
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)


def _get_varint(buf, pos):
    result = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if b < 0x80:
            return result, pos
        shift += 7
        if shift > 63:
            raise ValueError("malformed varint")


def _len_delimited(out: bytearray, field: int, payload: bytes):
    _put_varint(out, (field << 3) | 2)
    _put_varint(out, len(payload))
    out += payload


def _fields(buf):
    """Yields (field number, wire type, value) over one message; value is an int, or a memoryview for type 2."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _get_varint(buf, pos)
        field, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _get_varint(buf, pos)
        elif wt == 2:
            n, pos = _get_varint(buf, pos)
            v = buf[pos:pos + n]
            pos += n
        elif wt == 5:
            v = buf[pos:pos + 4]
            pos += 4
        elif wt == 1:
            v = buf[pos:pos + 8]
            pos += 8
        else:
            raise ValueError(f"unsupported wire type {wt}")
        if pos > end:
            raise ValueError("truncated record")
        yield field, wt, v


def _unpack_varints(payload) -> np.ndarray:
    """All varints of a packed field as uint64."""
    b = np.frombuffer(payload, dtype=np.uint8)
    if b.size == 0:
        return np.empty(0, dtype=np.uint64)
    ends = np.flatnonzero(b < 0x80)
    if ends.size == 0 or ends[-1] != b.size - 1:
        raise ValueError("malformed packed varints")
    starts = np.concatenate([[0], ends[:-1] + 1])
    shift = (np.arange(b.size) - np.repeat(starts, ends - starts + 1)) * 7
    if shift.max() > 63:
        raise ValueError("malformed packed varints")
    terms = (b & 0x7F).astype(np.uint64) << shift.astype(np.uint64)
    return np.add.reduceat(terms, starts)


# ------------------------------------------------------------------------------------------------ encode
def _encode_list(kind: str, values) -> bytes:
    out = bytearray()
    if kind == "bytes":
        for v in values:
            _len_delimited(out, 1, v.encode() if isinstance(v, str) else bytes(v))
    elif kind == "float":
        _len_delimited(out, 1, np.asarray(values, dtype="<f4").tobytes())
    elif kind == "double":
        _len_delimited(out, 1, np.asarray(values, dtype="<f8").tobytes())
    else:
        packed = bytearray()
        for v in np.asarray(values, dtype=np.int64).reshape(-1).tolist():
            _put_varint(packed, v)
        _len_delimited(out, 1, bytes(packed))
    return bytes(out)


def _infer_kind(value):
    if isinstance(value, (bytes, bytearray, str)):
        return "bytes", [value]
    if isinstance(value, (list, tuple)) and value and isinstance(value[0], (bytes, bytearray, str)):
        return "bytes", list(value)
    arr = np.asarray(value)
    if arr.dtype == np.float64:
        return "double", arr.reshape(-1)
    if arr.dtype.kind == "f":
        return "float", arr.reshape(-1)
    if arr.dtype in (np.int64, np.uint64):
        return "int64", arr.reshape(-1)
    if arr.dtype.kind in "iub":
        return "int32", arr.reshape(-1)
    raise TypeError(f"cannot store {arr.dtype} in an OFRecord feature")


def encode_ofrecord(features: dict) -> bytes:
    """``{name: value}`` -> serialised OFRecord.  A value is bytes / str / a list of them (bytes_list), or an array:
    float32 -> float_list, float64 -> double_list, int64 -> int64_list, other integers -> int32_list;
    ``(kind, values)`` forces the kind."""
    out = bytearray()
    for name, value in features.items():
        if isinstance(value, tuple) and len(value) == 2 and value[0] in _FIELD_OF_KIND:
            kind, vals = value
        else:
            kind, vals = _infer_kind(value)
        feature = bytearray()
        _len_delimited(feature, _FIELD_OF_KIND[kind], _encode_list(kind, vals))
        entry = bytearray()
        _len_delimited(entry, 1, name.encode())
        _len_delimited(entry, 2, bytes(feature))
        _len_delimited(out, 1, bytes(entry))
    return bytes(out)


# ------------------------------------------------------------------------------------------------ decode
def _decode_list(kind: str, msg):
    if kind == "bytes":
        return [bytes(v) for f, wt, v in _fields(msg) if f == 1 and wt == 2]
    chunks = []
    for f, wt, v in _fields(msg):
        if f != 1:
            continue
        if kind == "float":
            chunks.append(np.frombuffer(v, dtype="<f4"))
        elif kind == "double":
            chunks.append(np.frombuffer(v, dtype="<f8"))
        else:
            u = _unpack_varints(v) if wt == 2 else np.array([v], dtype=np.uint64)
            chunks.append(u.view(np.int64) if kind == "int64" else u.view(np.int64).astype(np.int32))
    if not chunks:
        return np.empty(0, dtype={"float": np.float32, "double": np.float64, "int32": np.int32, "int64": np.int64}[kind])
    return chunks[0] if len(chunks) == 1 else np.concatenate(chunks)


def decode_feature(record: bytes, name: str):
    """``(kind, values)`` of one feature of a serialised OFRecord, skipping the others; KeyError when absent."""
    want = name.encode()
    for f, wt, entry in _fields(memoryview(record)):
        if f != 1 or wt != 2:
            continue
        key = feat = None
        for ef, ewt, ev in _fields(entry):
            if ef == 1:
                key = bytes(ev)
            elif ef == 2:
                feat = ev
        if key == want:
            for ff, fwt, fv in _fields(feat if feat is not None else b""):
                if ff in _KIND_OF_FIELD and fwt == 2:
                    return _KIND_OF_FIELD[ff], _decode_list(_KIND_OF_FIELD[ff], fv)
            raise ValueError(f"feature {name!r} has no value")
    raise KeyError(name)


def decode_ofrecord(record: bytes) -> dict:
    """Serialised OFRecord -> ``{name: (kind, values)}``."""
    out = {}
    for f, wt, entry in _fields(memoryview(record)):
        if f != 1 or wt != 2:
            continue
        key, feat = None, b""
        for ef, ewt, ev in _fields(entry):
            if ef == 1:
                key = bytes(ev).decode()
            elif ef == 2:
                feat = ev
        for ff, fwt, fv in _fields(feat):
            if ff in _KIND_OF_FIELD and fwt == 2:
                out[key] = (_KIND_OF_FIELD[ff], _decode_list(_KIND_OF_FIELD[ff], fv))
    return out


# ------------------------------------------------------------------------------------------------ files
def write_ofrecord_file(path, records):
    """Writes feature dicts (or already serialised records) as one OFRecord part file."""
    with open(path, "wb") as f:
        for r in records:
            blob = r if isinstance(r, (bytes, bytearray)) else encode_ofrecord(r)
            f.write(struct.pack("<q", len(blob)))
            f.write(blob)


def read_ofrecord_file(path):
    """All serialised records of one part file (for tools and tests; training uses the prefetching reader)."""
    out = []
    with open(path, "rb") as f:
        while True:
            head = f.read(8)
            if len(head) < 8:
                return out
            (n,) = struct.unpack("<q", head)
            out.append(f.read(n))
