"""``lapid_quant``'s surface over the C ABI (crates/lapid-quant/src/lib.rs:27-160).

``layout`` is host arithmetic; ``quantize`` / ``dequantize`` / ``from_ggml_blocks`` run CUDA kernels
on a :class:`lapid_b200.Backend` and move host arrays through device buffers.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from . import _lib

GROUP = 32
ALIGN = 256


class Format(enum.IntEnum):
    """Formats this backend implements; values are lapid-c's dtype codes."""
    Int8 = 4   # GGUF Q8_0 in lapid's plane layout
    Int4 = 5   # GGUF Q4_0's nibbles in lapid's plane layout
    Q4K = 6
    Q5K = 7
    Q6K = 8

    def block_elems(self) -> int:
        return 32 if self in (Format.Int8, Format.Int4) else 256

    def block_bytes(self) -> int:
        return {Format.Int8: 0, Format.Int4: 0, Format.Q4K: 144, Format.Q5K: 176, Format.Q6K: 210}[self]

    def is_aos(self) -> bool:
        return self.block_bytes() != 0


@dataclass(frozen=True)
class Layout:
    rows: int
    cols: int
    qs_offset: int
    qs_bytes: int
    scales_offset: int
    scales_bytes: int
    total: int


def layout(fmt: int, rows: int, cols: int) -> Layout:
    out = _lib.LayoutC()
    _lib.check(_lib.lib().lapid_b200_quant_layout(int(fmt), rows, cols, C.byref(out)))
    return Layout(*[int(getattr(out, f)) for f, _ in _lib.LayoutC._fields_])


def quantize(backend, fmt: int, data: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Row-major f32 ``[rows, cols]`` -> ``layout(..).total`` bytes (quantized on the device)."""
    data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
    l = layout(fmt, rows, cols)
    src = backend.upload(data)
    dst = backend.alloc(l.total)
    backend.quantize_into(fmt, src, rows, cols, dst)
    return dst.download()


def dequantize(backend, fmt: int, qbytes: np.ndarray, rows: int, cols: int) -> np.ndarray:
    qbytes = np.ascontiguousarray(qbytes, dtype=np.uint8)
    src = backend.upload(qbytes)
    dst = backend.alloc(rows * cols * 4)
    backend.dequantize_into(fmt, src, rows, cols, dst)
    return dst.download().view(np.float32).reshape(rows, cols)


def from_ggml_blocks(backend, fmt: int, blocks: np.ndarray, rows: int, cols: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    l = layout(fmt, rows, cols)
    src = backend.upload(blocks)
    dst = backend.alloc(l.total)
    _lib.check(_lib.lib().lapid_b200_from_ggml_blocks(backend._h, int(fmt), src._h, blocks.size, rows, cols, dst._h))
    return dst.download()
