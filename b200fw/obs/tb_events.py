"""TensorBoard scalar event files without the ``tensorboard`` package.

The run directory of the reference contains a ``tensorboard/`` folder written through
``torch.utils.tensorboard.SummaryWriter`` (orchestrator: src/orchestrator/colocate_orchestrator.py:389-399;
``MetricsCollector.export_to_tensorboard``: src/utils/metrics.py:180-203) and a helper that prints
``train/loss`` back out of it (``_plot_loss.py:1-20``).  Only scalars are ever logged, and the on-disk format
for those is small: a TFRecord stream (length, masked CRC-32C of the length, payload, masked CRC-32C of the
payload) whose payloads are ``Event`` protocol buffers.  ``EventFileWriter`` writes exactly that, so the
files open in TensorBoard, and ``read_scalars`` parses them back, so nothing here needs the package.

Wire layout used (proto field numbers):

    Event   { double wall_time = 1; int64 step = 2; string file_version = 3; Summary summary = 5; }
    Summary { repeated Value value = 1; }
    Value   { string tag = 1; float simple_value = 2; }
"""
from __future__ import annotations

import os
import socket
import struct
import time
from typing import Dict, Iterator, List, Tuple

__all__ = ["EventFileWriter", "read_scalars", "open_writer"]


def _crc_table() -> List[int]:
    poly, table = 0x82F63B78, []            # CRC-32C (Castagnoli), reflected
    for i in range(256):
        c = i
        for _ in range(8):
            c = (c >> 1) ^ poly if c & 1 else c >> 1
        table.append(c)
    return table


_TABLE = _crc_table()


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _len_field(field: int, payload: bytes) -> bytes:
    return _varint((field << 3) | 2) + _varint(len(payload)) + payload


def _encode_event(wall_time: float, step: int = 0, file_version: str = "", scalar: Tuple[str, float] = None) -> bytes:
    ev = b"\x09" + struct.pack("<d", wall_time)
    if step:
        ev += b"\x10" + _varint(step)
    if file_version:
        ev += _len_field(3, file_version.encode())
    if scalar is not None:
        tag, val = scalar
        value = _len_field(1, tag.encode()) + b"\x15" + struct.pack("<f", float(val))
        ev += _len_field(5, _len_field(1, value))
    return ev


class EventFileWriter:
    """The subset of ``SummaryWriter`` the framework uses: ``add_scalar``, ``flush``, ``close``."""
    _serial = 0

    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self.log_dir = log_dir
        EventFileWriter._serial += 1        # two writers of one process in the same second get distinct files
        name = f"events.out.tfevents.{int(time.time()):010d}.{socket.gethostname()}.{os.getpid()}.{self._serial}"
        self.path = os.path.join(log_dir, name)
        self._f = open(self.path, "wb")
        self._record(_encode_event(time.time(), file_version="brain.Event:2"))
        self._f.flush()

    def _record(self, payload: bytes):
        head = struct.pack("<Q", len(payload))
        self._f.write(head + struct.pack("<I", _masked_crc(head)) + payload + struct.pack("<I", _masked_crc(payload)))

    def add_scalar(self, tag: str, scalar_value, global_step: int = 0, walltime: float = None):
        if self._f is None:
            raise ValueError("writer is closed")
        self._record(_encode_event(walltime if walltime is not None else time.time(), int(global_step or 0),
                                   scalar=(tag, float(scalar_value))))

    def flush(self):
        if self._f is not None:
            self._f.flush()

    def close(self):
        if self._f is not None:
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def open_writer(log_dir: str):
    """``SummaryWriter`` when the ``tensorboard`` package is importable, else the built-in writer."""
    try:
        from torch.utils.tensorboard import SummaryWriter
        return SummaryWriter(log_dir)
    except Exception:  # noqa: BLE001 - optional dependency
        return EventFileWriter(log_dir)


# ---- reading ----------------------------------------------------------------------------------------
def _records(path: str) -> Iterator[bytes]:
    with open(path, "rb") as f:
        while True:
            head = f.read(8)
            if len(head) < 8:
                return
            (n,) = struct.unpack("<Q", head)
            (crc,) = struct.unpack("<I", f.read(4))
            if crc != _masked_crc(head):
                raise ValueError(f"{path}: corrupt record header")
            payload = f.read(n)
            tail = f.read(4)
            if len(payload) < n or len(tail) < 4:
                return                      # a writer was cut off mid-record: keep what is complete
            if struct.unpack("<I", tail)[0] != _masked_crc(payload):
                raise ValueError(f"{path}: corrupt record payload")
            yield payload


def _fields(buf: bytes) -> Iterator[Tuple[int, int, object]]:
    i, n = 0, len(buf)
    while i < n:
        key, shift = 0, 0
        while True:
            b = buf[i]
            i += 1
            key |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                break
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, shift = 0, 0
            while True:
                b = buf[i]
                i += 1
                v |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            yield field, wire, v
        elif wire == 1:
            yield field, wire, buf[i:i + 8]
            i += 8
        elif wire == 2:
            ln, shift = 0, 0
            while True:
                b = buf[i]
                i += 1
                ln |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            yield field, wire, buf[i:i + ln]
            i += ln
        elif wire == 5:
            yield field, wire, buf[i:i + 4]
            i += 4
        else:
            raise ValueError(f"unsupported wire type {wire}")


def read_scalars(log_dir_or_file: str) -> Dict[str, List[Tuple[int, float, float]]]:
    """``{tag: [(step, value, wall_time), ...]}`` from one event file or every event file of a folder."""
    if os.path.isdir(log_dir_or_file):
        files = sorted(os.path.join(log_dir_or_file, f) for f in os.listdir(log_dir_or_file) if "tfevents" in f)
    else:
        files = [log_dir_or_file]
    out: Dict[str, List[Tuple[int, float, float]]] = {}
    for path in files:
        for rec in _records(path):
            wall, step, summaries = 0.0, 0, []
            for field, wire, v in _fields(rec):
                if field == 1 and wire == 1:
                    (wall,) = struct.unpack("<d", v)
                elif field == 2 and wire == 0:
                    step = v if v < (1 << 63) else v - (1 << 64)
                elif field == 5 and wire == 2:
                    summaries.append(v)
            for s in summaries:
                for field, wire, value in _fields(s):
                    if field != 1 or wire != 2:
                        continue
                    tag, val = None, None
                    for f2, w2, v2 in _fields(value):
                        if f2 == 1 and w2 == 2:
                            tag = v2.decode()
                        elif f2 == 2 and w2 == 5:
                            (val,) = struct.unpack("<f", v2)
                    if tag is not None and val is not None:
                        out.setdefault(tag, []).append((step, val, wall))
    for series in out.values():
        series.sort(key=lambda t: (t[0], t[2]))
    return out
