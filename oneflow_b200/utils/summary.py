"""Event-file summaries (scalars, histograms, text) readable by TensorBoard, written without any dependency:
records are framed as TFRecords (length, masked CRC-32C, payload, masked CRC-32C) and the Event / Summary messages
are protobuf-encoded by hand.

Reference: oneflow/user/summary/{event_writer_helper,events_writer,histogram,summary_converter}.cpp, the
``summary_write_*`` ops, and python/oneflow/utils/tensorboard (SummaryWriter: add_scalar / add_histogram / add_text)."""
from __future__ import annotations

import os
import socket
import struct
import time

import numpy as np

# ------------------------------------------------------------------------------------------------ crc32c (Castagnoli)
_TABLE = []
for _i in range(256):
    _c = _i
    for _ in range(8):
        _c = (_c >> 1) ^ 0x82F63B78 if _c & 1 else _c >> 1
    _TABLE.append(_c)


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


# ------------------------------------------------------------------------------------------------ protobuf encoding
def _varint(n: int) -> bytes:
    out = bytearray()
    n &= (1 << 64) - 1
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _key(field, wire):
    return _varint((field << 3) | wire)


def _f_double(field, v):
    return _key(field, 1) + struct.pack("<d", float(v))


def _f_float(field, v):
    return _key(field, 5) + struct.pack("<f", float(v))


def _f_int(field, v):
    return _key(field, 0) + _varint(int(v))


def _f_bytes(field, b):
    return _key(field, 2) + _varint(len(b)) + b


def _packed_doubles(field, values):
    body = b"".join(struct.pack("<d", float(v)) for v in values)
    return _f_bytes(field, body)


def _event(step, summary_value=None, file_version=None, wall_time=None):
    msg = _f_double(1, time.time() if wall_time is None else wall_time) + _f_int(2, step)
    if file_version is not None:
        msg += _f_bytes(3, file_version.encode())
    if summary_value is not None:
        msg += _f_bytes(5, _f_bytes(1, summary_value))      # Event.summary { repeated Value value = 1 }
    return msg


class SummaryWriter:
    def __init__(self, log_dir="runs", filename_suffix=""):
        os.makedirs(log_dir, exist_ok=True)
        name = f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}.{os.getpid()}{filename_suffix}"
        self.path = os.path.join(log_dir, name)
        self._f = open(self.path, "ab")
        self._write(_event(0, file_version="brain.Event:2"))

    def _write(self, payload: bytes):
        header = struct.pack("<Q", len(payload))
        self._f.write(header + struct.pack("<I", _masked(header)) + payload + struct.pack("<I", _masked(payload)))

    def add_scalar(self, tag, value, global_step=0, walltime=None):
        v = _f_bytes(1, tag.encode()) + _f_float(2, float(value))             # Value { tag = 1, simple_value = 2 }
        self._write(_event(global_step, v, wall_time=walltime))

    def add_histogram(self, tag, values, global_step=0, bins=30, walltime=None):
        a = np.asarray(values.detach().cpu().float().numpy() if hasattr(values, "detach") else values, dtype=np.float64).ravel()
        counts, edges = np.histogram(a, bins=bins)
        histo = (_f_double(1, a.min()) + _f_double(2, a.max()) + _f_double(3, a.size) + _f_double(4, a.sum()) +
                 _f_double(5, (a * a).sum()) + _packed_doubles(6, edges[1:]) + _packed_doubles(7, counts))
        v = _f_bytes(1, tag.encode()) + _f_bytes(5, histo)                    # Value.histo = 5
        self._write(_event(global_step, v, wall_time=walltime))

    def add_text(self, tag, text, global_step=0, walltime=None):
        tensor = _f_int(1, 7) + _f_bytes(8, text.encode())                   # TensorProto { dtype = DT_STRING, string_val = 8 }
        meta = _f_bytes(1, _f_bytes(1, b"text"))                             # SummaryMetadata.plugin_data.plugin_name
        v = _f_bytes(1, tag.encode()) + _f_bytes(8, tensor) + _f_bytes(9, meta)
        self._write(_event(global_step, v, wall_time=walltime))

    def flush(self):
        self._f.flush()

    def close(self):
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def read_events(path):
    """Parses an event file written above: yields (step, tag, simple_value or None). Checks every CRC."""
    def read_varint(buf, pos):
        shift = val = 0
        while True:
            b = buf[pos]
            pos += 1
            val |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                return val, pos

    def fields(buf):
        pos = 0
        while pos < len(buf):
            key, pos = read_varint(buf, pos)
            f, wire = key >> 3, key & 7
            if wire == 0:
                v, pos = read_varint(buf, pos)
            elif wire == 1:
                v, pos = buf[pos:pos + 8], pos + 8
            elif wire == 5:
                v, pos = buf[pos:pos + 4], pos + 4
            else:
                n, pos = read_varint(buf, pos)
                v, pos = buf[pos:pos + n], pos + n
            yield f, wire, v

    with open(path, "rb") as f:
        data = f.read()
    pos = 0
    while pos < len(data):
        header = data[pos:pos + 8]
        (n,) = struct.unpack("<Q", header)
        assert struct.unpack("<I", data[pos + 8:pos + 12])[0] == _masked(header), "corrupt record header"
        payload = data[pos + 12:pos + 12 + n]
        assert struct.unpack("<I", data[pos + 12 + n:pos + 16 + n])[0] == _masked(payload), "corrupt record payload"
        pos += 16 + n
        step, summary = 0, None
        for fnum, wire, v in fields(payload):
            if fnum == 2 and wire == 0:
                step = v
            elif fnum == 5:
                summary = v
        if summary is None:
            continue
        for fnum, _, value in fields(summary):
            if fnum != 1:
                continue
            tag, simple = None, None
            for vf, vw, vv in fields(value):
                if vf == 1:
                    tag = vv.decode()
                elif vf == 2 and vw == 5:
                    simple = struct.unpack("<f", vv)[0]
            yield step, tag, simple
