"""The .vlt weight container and the int8 weight-only quantiser, in numpy.

Same bytes as the reference's converter writes (tools/convert.py:117-165 `write`/`read`,
:41-56 `quantize`/`dequantize`) and its engine reads (engine/src/weights.rs:37-74). bf16
tensors are carried as uint16 bit patterns in a `Bf16` wrapper, since numpy has no bf16.
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np

DATA_ALIGN = 16384
TENSOR_ALIGN = 256
F32, BF16, I8 = 0, 1, 2


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


def _code_and_raw(t) -> tuple[int, np.ndarray]:
    if isinstance(t, Bf16):
        return BF16, t.bits
    t = np.ascontiguousarray(t)
    if t.dtype == np.float32:
        return F32, t
    if t.dtype == np.int8:
        return I8, t
    raise TypeError(f"a .vlt tensor is float32, int8 or Bf16, not {t.dtype}")


def write(path, tensors: dict) -> None:
    """tools/convert.py:117-152: 32-byte header, 128-byte records, tensors 256-byte aligned
    in a data region that starts and ends on 16 KiB boundaries."""
    records, blobs, offset = [], [], 0
    for name, t in tensors.items():
        code, raw = _code_and_raw(t)
        if raw.ndim > 4:
            raise ValueError(f"{name}: more than 4 dimensions")
        offset = -(-offset // TENSOR_ALIGN) * TENSOR_ALIGN
        name_b = name.encode()
        if len(name_b) >= 64:
            raise ValueError(f"{name}: name longer than 63 bytes")
        shape = list(raw.shape) + [0] * (4 - raw.ndim)
        records.append(struct.pack("<64sII4IQQ24x", name_b, code, raw.ndim, *shape, offset, raw.nbytes))
        blobs.append((offset, raw))
        offset += raw.nbytes
    header_len = 32 + 128 * len(records)
    data_offset = -(-header_len // DATA_ALIGN) * DATA_ALIGN
    total = data_offset + -(-offset // DATA_ALIGN) * DATA_ALIGN
    with open(path, "wb") as fh:
        fh.write(struct.pack("<8sIIQII", b"VIOLETTO", 1, len(records), data_offset, 0, 0))
        fh.writelines(records)
        for off, raw in blobs:
            fh.seek(data_offset + off)
            fh.write(raw.tobytes() if raw.nbytes < (1 << 28) else memoryview(raw).cast("B"))
        fh.truncate(total)


def read(path) -> dict:
    """Every tensor of a weight file (tools/convert.py:155-167)."""
    data = Path(path).read_bytes()
    magic, version, n, data_offset, _, _ = struct.unpack_from("<8sIIQII", data, 0)
    if magic != b"VIOLETTO" or version != 1:
        raise ValueError(f"{path}: not a version-1 violetto weight file")
    out = {}
    for i in range(n):
        name_b, code, ndim, *rest = struct.unpack_from("<64sII4IQQ24x", data, 32 + 128 * i)
        shape, (offset, nbytes) = rest[:ndim], rest[4:]
        raw = data[data_offset + offset:data_offset + offset + nbytes]
        dt = {F32: np.float32, BF16: np.uint16, I8: np.int8}[code]
        arr = np.frombuffer(raw, dtype=dt).reshape(shape).copy()
        out[name_b.rstrip(b"\0").decode()] = Bf16(arr) if code == BF16 else arr
    return out


def quantize(w: np.ndarray, group: int) -> tuple[np.ndarray, Bf16]:
    """tools/convert.py:41-50: symmetric int8 over groups of `group` consecutive k, one bf16
    scale per group (absmax / 127 rounded to nearest), q = round-half-even(w / scale)
    clamped to +-127, 0 where the scale is 0."""
    w = np.ascontiguousarray(w, np.float32)
    m, k = w.shape
    g = w.reshape(m, k // group, group)
    s = to_bf16(np.abs(g).max(-1) / np.float32(127))
    sf = from_bf16(s)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(sf > 0, g / sf, np.float32(0))
    q = np.clip(np.rint(q), -127, 127).astype(np.int8)
    return q.reshape(m, k), Bf16(s)


def dequantize(q: np.ndarray, s: Bf16) -> np.ndarray:
    """tools/convert.py:53-56: exact in fp32."""
    m, k = q.shape
    return (q.astype(np.float32).reshape(m, s.shape[1], -1) * s.f32()[..., None]).reshape(m, k)
