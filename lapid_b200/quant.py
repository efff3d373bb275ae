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
    MXFP4 = 9  # ggml block_mxfp4: 32 elements in 17 bytes
    # ggml's grid-based i-quants, blocks kept as in GGUF (crates/lapid-quant/src/lib.rs:43-51); no quantizer here
    Iq2Xxs = 10
    Iq2S = 11
    Iq3Xxs = 12
    Iq2Xs = 13

    def block_elems(self) -> int:
        return 32 if self in (Format.Int8, Format.Int4, Format.MXFP4) else 256

    def block_bytes(self) -> int:
        return {Format.Int8: 0, Format.Int4: 0, Format.Q4K: 144, Format.Q5K: 176, Format.Q6K: 210, Format.MXFP4: 17,
                Format.Iq2Xxs: 66, Format.Iq2Xs: 74, Format.Iq2S: 82, Format.Iq3Xxs: 98}[self]

    def is_iquant(self) -> bool:
        return self in (Format.Iq2Xxs, Format.Iq2Xs, Format.Iq2S, Format.Iq3Xxs)

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


def from_ggml_blocks_into(backend, fmt: int, src, src_bytes: int, rows: int, cols: int, dst) -> None:
    """``from_ggml_blocks`` between two device buffers: ``src_bytes`` of GGUF blocks in ``src`` -> lapid layout in ``dst``."""
    _lib.check(_lib.lib().lapid_b200_from_ggml_blocks(backend._h, int(fmt), src._h, src_bytes, rows, cols, dst._h))


def from_ggml_blocks(backend, fmt: int, blocks: np.ndarray, rows: int, cols: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    l = layout(fmt, rows, cols)
    src = backend.upload(blocks)
    dst = backend.alloc(l.total)
    _lib.check(_lib.lib().lapid_b200_from_ggml_blocks(backend._h, int(fmt), src._h, blocks.size, rows, cols, dst._h))
    return dst.download()


# ---- the quantized activation operand of the decode path (lapid_b200_quantize_activations / lapid_b200_act_layout)
ACT_PLANES, ACT_RECORDS, ACT_TILES = 0, 1, 2
_REC = 336


def _up256(x: int) -> int:
    return (x + 255) // 256 * 256


def act_bytes(act_layout: int, rows: int, k: int) -> int:
    """Bytes of ``rows`` quantized activation rows of ``k`` elements in ``act_layout``."""
    if act_layout == ACT_PLANES:
        return _up256(rows * k) + 2 * _up256(rows * (k // 32) * 4)
    if act_layout == ACT_RECORDS:
        return rows * (k // 256) * _REC
    return (k // 256) * (256 * rows + 512)


def quantize_activations(backend, x: np.ndarray, rows: int, k: int, act_layout: int) -> np.ndarray:
    """The raw operand bytes for f32 ``x [rows, k]`` (``quantize_row_sums``, crates/lapid-cpu/src/matmul/quant.rs:30-89)."""
    src = backend.upload(np.ascontiguousarray(x, dtype=np.float32).reshape(-1))
    dst = backend.upload(np.zeros(act_bytes(act_layout, rows, k), np.uint8))
    backend.quantize_activations(src, rows, k, act_layout, dst)
    return dst.download()


def unpack_activations(act_layout: int, raw: np.ndarray, rows: int, k: int):
    """``(q int8 [rows, k], d f32 [rows, k/32], bs f32 [rows, k/32])`` from the raw bytes of an operand in
    ``act_layout``: planes; 336-byte records, one per (row, 256-block): 4 x [64 quants | d d bs bs], 16 pad; or
    tiles, one per 256-block: ``[sub-block 8][row][32]`` quants, then f32 d as
    ``[sub-block pair 4][row pair 4][sub-block & 1][row & 1]`` and the same for bs."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    kg, nblk = k // 32, k // 256
    q = np.zeros((rows, k), np.int8)
    d = np.zeros((rows, kg), np.float32)
    bs = np.zeros((rows, kg), np.float32)
    if act_layout == ACT_PLANES:
        p0, p1 = _up256(rows * k), _up256(rows * kg * 4)
        q[:] = raw[:rows * k].view(np.int8).reshape(rows, k)
        d[:] = raw[p0:p0 + rows * kg * 4].view(np.float32).reshape(rows, kg)
        bs[:] = raw[p0 + p1:p0 + p1 + rows * kg * 4].view(np.float32).reshape(rows, kg)
    elif act_layout == ACT_RECORDS:
        rec = raw[:rows * nblk * _REC].reshape(rows, nblk, _REC)
        for p in range(4):
            part = rec[:, :, 80 * p:80 * p + 80]
            for h in range(2):
                g = 2 * p + h
                q.reshape(rows, nblk, 8, 32)[:, :, g, :] = part[:, :, 32 * h:32 * h + 32].view(np.int8)
                d.reshape(rows, nblk, 8)[:, :, g] = np.ascontiguousarray(part[:, :, 64 + 4 * h:68 + 4 * h]).view(np.float32)[:, :, 0]
                bs.reshape(rows, nblk, 8)[:, :, g] = np.ascontiguousarray(part[:, :, 72 + 4 * h:76 + 4 * h]).view(np.float32)[:, :, 0]
    else:
        ab = 256 * rows + 512
        blk = raw[:nblk * ab].reshape(nblk, ab)
        qs = blk[:, :256 * rows].view(np.int8).reshape(nblk, 8, rows, 32)
        q.reshape(rows, nblk, 8, 32)[:] = qs.transpose(2, 0, 1, 3)
        sc = np.ascontiguousarray(blk[:, 256 * rows:]).view(np.float32).reshape(nblk, 2, 4, 4, 2, 2)  # [d | bs][sub-block pair][row pair][sub-block & 1][row & 1]
        for r in range(rows):
            d.reshape(rows, nblk, 8)[r] = sc[:, 0, :, r >> 1, :, r & 1].reshape(nblk, 8)
            bs.reshape(rows, nblk, 8)[r] = sc[:, 1, :, r >> 1, :, r & 1].reshape(nblk, 8)
    return q, d, bs
