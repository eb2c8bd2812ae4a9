"""The .vlt weight container and the int8 weight-only quantiser, in numpy.

The file format is the reference's (engine/src/weights.rs:37-74 reads it, tools/convert.py:117-152
documents and writes it): a 32-byte header, one 128-byte record per tensor, then a data region that
starts and ends on 16 KiB boundaries with every tensor on a 256-byte boundary. Here the header and the
record are numpy structured types and a file is laid out up front as a table of offsets, then filled
through a memory map. bf16 tensors are carried as uint16 bit patterns in a `Bf16` wrapper, since numpy
has no bf16. The quantiser is tools/convert.py:41-56's arithmetic, bit for bit.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

DATA_ALIGN = 16384
TENSOR_ALIGN = 256
F32, BF16, I8 = 0, 1, 2
MAGIC = b"VIOLETTO"
VERSION = 1

HEADER = np.dtype([("magic", "S8"), ("version", "<u4"), ("count", "<u4"), ("data_offset", "<u8"), ("reserved", "<u4", (2,))])
RECORD = np.dtype([("name", "S64"), ("dtype", "<u4"), ("ndim", "<u4"), ("shape", "<u4", (4,)), ("offset", "<u8"), ("nbytes", "<u8"), ("reserved", "V24")])
assert HEADER.itemsize == 32 and RECORD.itemsize == 128
_STORAGE = {F32: np.dtype("<f4"), BF16: np.dtype("<u2"), I8: np.dtype("i1")}


class Bf16:
    """A bf16 tensor as its uint16 bit patterns."""

    def __init__(self, bits: np.ndarray):
        self.bits = np.ascontiguousarray(bits, np.uint16)

    @staticmethod
    def from_f32(x: np.ndarray) -> "Bf16":
        return Bf16(to_bf16(x))

    def f32(self) -> np.ndarray:
        return from_bf16(self.bits)

    @property
    def shape(self):
        return self.bits.shape


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even (finite inputs), as torch's .to(bfloat16) and kernels.metal:22-27."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def from_bf16(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _up(x: int, align: int) -> int:
    return (x + align - 1) // align * align


def _storage(name: str, t) -> tuple[int, np.ndarray]:
    """A tensor's dtype code and the array that holds its bytes."""
    if isinstance(t, Bf16):
        code, raw = BF16, t.bits
    else:
        raw = np.ascontiguousarray(t)
        codes = [c for c, dt in _STORAGE.items() if c != BF16 and raw.dtype == dt]
        if not codes:
            raise TypeError(f"{name}: a .vlt tensor is float32, int8 or Bf16, not {raw.dtype}")
        code = codes[0]
    if raw.ndim > 4:
        raise ValueError(f"{name}: more than 4 dimensions")
    if len(name.encode()) >= 64:
        raise ValueError(f"{name}: name longer than 63 bytes")
    return code, raw


def layout(tensors: dict) -> tuple[np.ndarray, np.ndarray, list]:
    """The header, the record table and the tensors' storage arrays of a file holding `tensors`, in their order."""
    stored = [_storage(name, t) for name, t in tensors.items()]
    table = np.zeros(len(stored), RECORD)
    at = 0
    for rec, name, (code, raw) in zip(table, tensors, stored):
        at = _up(at, TENSOR_ALIGN)
        rec["name"], rec["dtype"], rec["ndim"] = name.encode(), code, raw.ndim
        rec["shape"][:raw.ndim] = raw.shape
        rec["offset"], rec["nbytes"] = at, raw.nbytes
        at += raw.nbytes
    header = np.zeros(1, HEADER)
    header["magic"], header["version"], header["count"] = MAGIC, VERSION, len(stored)
    header["data_offset"] = _up(HEADER.itemsize + table.nbytes, DATA_ALIGN)
    return header, table, [raw for _, raw in stored]


def write(path, tensors: dict) -> None:
    """Writes `tensors` (name -> float32 / int8 array or Bf16) as a weight file."""
    header, table, arrays = layout(tensors)
    data_offset = int(header["data_offset"][0])
    end = int(table["offset"][-1] + table["nbytes"][-1]) if len(table) else 0
    total = data_offset + _up(end, DATA_ALIGN)
    out = np.memmap(path, dtype=np.uint8, mode="w+", shape=(total,))  # a new file of that size, zero-filled
    out[:HEADER.itemsize] = header.view(np.uint8)
    out[HEADER.itemsize:HEADER.itemsize + table.nbytes] = table.view(np.uint8)
    for rec, raw in zip(table, arrays):
        lo = data_offset + int(rec["offset"])
        out[lo:lo + raw.nbytes] = raw.reshape(-1).view(np.uint8)
    out.flush()
    del out


def read(path) -> dict:
    """Every tensor of a weight file: name -> array (float32, int8) or Bf16."""
    blob = np.memmap(path, dtype=np.uint8, mode="r")
    if blob.size < HEADER.itemsize:
        raise ValueError(f"{path}: not a version-1 violetto weight file")
    header = blob[:HEADER.itemsize].view(HEADER)[0]
    if header["magic"] != MAGIC or header["version"] != VERSION:
        raise ValueError(f"{path}: not a version-1 violetto weight file")
    table = blob[HEADER.itemsize:HEADER.itemsize + int(header["count"]) * RECORD.itemsize].view(RECORD)
    base = int(header["data_offset"])
    out = {}
    for rec in table:
        lo = base + int(rec["offset"])
        arr = np.array(blob[lo:lo + int(rec["nbytes"])]).view(_STORAGE[int(rec["dtype"])]).reshape(tuple(int(x) for x in rec["shape"][:int(rec["ndim"])]))
        out[rec["name"].decode()] = Bf16(arr) if int(rec["dtype"]) == BF16 else arr
    return out


def quantize(w: np.ndarray, group: int) -> tuple[np.ndarray, Bf16]:
    """Symmetric int8 over groups of `group` consecutive k with one bf16 scale per group (tools/convert.py:41-50):
    scale = bf16(absmax / 127), q = the weight over its scale rounded half to even and clamped to +-127, 0 where the
    scale is 0."""
    w = np.ascontiguousarray(w, np.float32)
    rows, k = w.shape
    grouped = w.reshape(rows, k // group, group)
    scale_bits = to_bf16(np.abs(grouped).max(axis=2) / np.float32(127))
    scale = from_bf16(scale_bits)[:, :, None]
    ratio = np.zeros_like(grouped)
    np.divide(grouped, scale, out=ratio, where=scale > 0)
    q = np.rint(ratio)
    np.clip(q, -127, 127, out=q)
    return q.astype(np.int8).reshape(rows, k), Bf16(scale_bits)


def dequantize(q: np.ndarray, s: Bf16) -> np.ndarray:
    """The fp32 weights of an int8 matrix (tools/convert.py:53-56): exact, an int8 times a bf16 fits in fp32."""
    rows, k = q.shape
    groups = s.shape[1]
    return (q.astype(np.float32).reshape(rows, groups, k // groups) * s.f32()[:, :, None]).reshape(rows, k)
