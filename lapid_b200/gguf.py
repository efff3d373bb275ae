"""GGUF tensor table reader: real model tensors into lapid-quant layout on the device.

The counterpart, for this path only, of the reference's GGUF reader and its "keep the blocks" import
(crates/lapid-convert/src/gguf.rs:1-12 container layout, :177-215 `write_ggml_tensor`): K-quant blocks
(Q4_K, Q5_K, Q6_K), MXFP4 blocks and the i-quants (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS) are kept byte for byte, Q8_0 and Q4_0 blocks are repacked losslessly into lapid's
Int8 / Int4 planes (`lapid_quant::from_ggml_blocks`, crates/lapid-quant/src/imp.rs:171-200, here
`lapid_b200_from_ggml_blocks` on the device), F32 / F16 tensors are handed over as they are. Nothing is
dequantized and nothing is re-quantized.

Container (little endian, versions 2 and 3)::

    "GGUF" | u32 version | u64 n_tensors | u64 n_kv
    n_kv x      (string key, u32 value_type, value)
    n_tensors x (string name, u32 n_dims, n_dims x u64 ne, u32 ggml_type, u64 offset)
    pad to general.alignment (default 32) | tensor data (offsets relative to here)

Strings are ``u64 len`` + UTF-8 bytes, arrays ``u32 elem_type, u64 len, elems``; ``ne[0]`` is the
fastest-varying dimension, so the row-major shape is ``ne`` reversed.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from .backend import DType

MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32
_MAX_COUNT = 1 << 20
_MAX_STRING = 1 << 30
_MAX_DIMS = 4

# ggml type id -> (name, elements per block, bytes per block)
GGML_TYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
    8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 40), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144),
    13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292), 16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74),
    18: ("IQ3_XXS", 256, 98), 22: ("IQ2_S", 256, 82), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8),
    28: ("F64", 1, 8), 30: ("BF16", 1, 2), 39: ("MXFP4", 32, 17),
}
# ggml type -> the lapid dtype this backend keeps it in (crates/lapid-convert/src/ggml.rs `lapid_format`)
LAPID_DTYPE = {"Q8_0": DType.Int8, "Q4_0": DType.Int4, "Q4_K": DType.Q4K, "Q5_K": DType.Q5K, "Q6_K": DType.Q6K, "MXFP4": DType.MXFP4,
               "IQ2_XXS": DType.Iq2Xxs, "IQ2_XS": DType.Iq2Xs, "IQ2_S": DType.Iq2S, "IQ3_XXS": DType.Iq3Xxs,
               "F32": DType.F32, "F16": DType.F16, "BF16": DType.BF16}


class GgufError(ValueError):
    """A malformed or unsupported file; ``code`` follows the reference's error codes."""

    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code


@dataclass(frozen=True)
class GgufTensor:
    name: str
    shape: Tuple[int, ...]   # row-major (ne reversed)
    ggml_type: int
    type_name: str
    offset: int              # absolute byte offset in the file
    nbytes: int

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class _Cursor:
    def __init__(self, buf):
        self.b, self.pos = buf, 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > len(self.b):
            raise GgufError("invalid_gguf", f"truncated file: need {n} bytes at offset {self.pos}, file has {len(self.b)}")
        out = self.b[self.pos:self.pos + n]
        self.pos += n
        return out

    def num(self, fmt: str):
        return struct.unpack("<" + fmt, self.take(struct.calcsize("<" + fmt)))[0]

    def string(self) -> str:
        n = self.num("Q")
        if n > _MAX_STRING:
            raise GgufError("invalid_gguf", f"string of {n} bytes at offset {self.pos}")
        return bytes(self.take(n)).decode("utf-8", errors="replace")


_SCALARS = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}


def _value(c: _Cursor, vt: int, depth: int = 0) -> Any:
    if vt in _SCALARS:
        return c.num(_SCALARS[vt])
    if vt == 8:
        return c.string()
    if vt == 9:
        if depth > 2:
            raise GgufError("invalid_gguf", "arrays nested too deeply")
        et, n = c.num("I"), c.num("Q")
        if n > (1 << 28):
            raise GgufError("invalid_gguf", f"array of {n} elements")
        if et in _SCALARS and et != 7:   # numeric arrays in one piece
            code = _SCALARS[et]
            return np.frombuffer(c.take(n * struct.calcsize("<" + code)), dtype="<" + {"B": "u1", "b": "i1", "H": "u2", "h": "i2", "I": "u4",
                                 "i": "i4", "f": "f4", "Q": "u8", "q": "i8", "d": "f8"}[code]).tolist()
        return [_value(c, et, depth + 1) for _ in range(n)]
    raise GgufError("invalid_gguf", f"unknown metadata value type {vt}")


class GgufFile:
    """The metadata and the tensor table of a GGUF file; tensor bytes are served from a memory map."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        c = _Cursor(self._map)
        if bytes(c.take(4)) != MAGIC:
            raise GgufError("invalid_gguf", f"{path}: not a GGUF file")
        self.version = c.num("I")
        if self.version not in (2, 3):
            raise GgufError("unsupported_gguf_version", f"{path}: version {self.version} (2 and 3 are read)")
        n_tensors, n_kv = c.num("Q"), c.num("Q")
        if n_tensors > _MAX_COUNT or n_kv > _MAX_COUNT:
            raise GgufError("invalid_gguf", f"{path}: {n_tensors} tensors, {n_kv} metadata entries")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = _value(c, c.num("I"))
        infos = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.num("I")
            if nd > _MAX_DIMS:
                raise GgufError("invalid_gguf", f"tensor {name!r}: {nd} dimensions")
            ne = [c.num("Q") for _ in range(nd)]
            infos.append((name, ne, c.num("I"), c.num("Q")))
        align = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT)) or DEFAULT_ALIGNMENT
        self.alignment = align
        self.data_offset = (c.pos + align - 1) // align * align
        self.tensors: List[GgufTensor] = []
        for name, ne, gt, off in infos:
            if gt not in GGML_TYPES:
                raise GgufError("unsupported_gguf_type", f"tensor {name!r}: ggml type {gt}")
            tname, be, bb = GGML_TYPES[gt]
            numel = 1
            for e in ne:
                numel *= e
            if ne and ne[0] % be:
                raise GgufError("invalid_gguf", f"tensor {name!r}: ne[0] = {ne[0]} is not a multiple of the {tname} block ({be})")
            nbytes = numel // be * bb
            absolute = self.data_offset + off
            if off % align or absolute + nbytes > len(self._map):
                raise GgufError("invalid_gguf", f"tensor {name!r}: data [{absolute}, {absolute + nbytes}) is misaligned or outside the file")
            self.tensors.append(GgufTensor(name, tuple(reversed(ne)), gt, tname, absolute, nbytes))

    # ---- access
    def tensor(self, name: str) -> Optional[GgufTensor]:
        for t in self.tensors:
            if t.name == name:
                return t
        return None

    def tensor_data(self, t: GgufTensor) -> np.ndarray:
        """The raw (ggml-encoded) bytes of a tensor, zero copy."""
        return np.frombuffer(self._map, dtype=np.uint8, count=t.nbytes, offset=t.offset)

    def architecture(self) -> Optional[str]:
        v = self.metadata.get("general.architecture")
        return v if isinstance(v, str) else None

    def close(self) -> None:
        try:
            self._map.close()
        finally:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        try:
            self.close()
        except BufferError:   # a numpy view of the map is still alive; the map goes with it
            pass

    # ---- onto the device
    def load(self, backend, name: str):
        """Tensor ``name`` as a device buffer in the layout the launches read: ``(buffer, dtype, shape)``.

        2-D tensors are one lapid-quant matrix ``[rows, cols]``; 3-D tensors are expert stacks ``[e, rows, cols]``
        of ``e`` matrices, each ``layout(rows, cols).total`` bytes (what a MatMulId launch reads). K-quant blocks
        are kept as they are, Q8_0 / Q4_0 become Int8 / Int4 planes, F32 / F16 / BF16 are uploaded unchanged.
        Other ggml types fail with ``unsupported_gguf_type``: this path holds no dequantizer for them."""
        from . import quant
        t = self.tensor(name)
        if t is None:
            raise GgufError("not_found", f"{self.path}: no tensor {name!r}")
        if t.type_name not in LAPID_DTYPE:
            raise GgufError("unsupported_gguf_type", f"tensor {name!r}: {t.type_name} is not kept by this backend")
        dtype = LAPID_DTYPE[t.type_name]
        data = self.tensor_data(t)
        if dtype in (DType.F32, DType.F16, DType.BF16):
            return backend.upload(data), dtype, t.shape
        if len(t.shape) not in (2, 3):
            raise GgufError("shape_mismatch", f"tensor {name!r}: a quantized tensor must be 2-D or a 3-D expert stack, got {t.shape}")
        rows, cols = t.shape[-2], t.shape[-1]
        experts = t.shape[0] if len(t.shape) == 3 else 1
        one = quant.layout(dtype, rows, cols).total
        per = t.nbytes // experts
        dst = backend.alloc(experts * one)
        if experts == 1:
            quant.from_ggml_blocks_into(backend, dtype, backend.upload(data), per, rows, cols, dst)
            return dst, dtype, t.shape
        src = backend.upload(data)
        for e in range(experts):   # each expert's matrix on its own: the padding between them is part of the layout
            piece = backend.wrap(dst.device_ptr + e * one, one, keep=dst)
            part = backend.wrap(src.device_ptr + e * per, per, keep=src) if (e * per) % 16 == 0 else backend.upload(data[e * per:(e + 1) * per])
            quant.from_ggml_blocks_into(backend, dtype, part, per, rows, cols, piece)
        return dst, dtype, t.shape
