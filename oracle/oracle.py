"""ctypes front end of the CPU oracle (``lapid_oracle.c``). TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline legs import this module; the
shipped package never does. Two builds of the same C source exist:

* the parity copy (``-O2 -ffp-contract=off``, portable ISA), built by ``make -C oracle`` /
  ``build()`` and shipped next to the source;
* the timed copy (``-O3 -march=native``), compiled on first use on the machine that runs it
  (``load(fast=True)``), because ``-march=native`` code must not travel between hosts.

Function names follow the reference's: ``layout``, ``quantize``, ``dequantize``,
``from_ggml_blocks`` (crates/lapid-quant/src/lib.rs:97-160), ``quantize_row_sums``
(crates/lapid-cpu/src/matmul/quant.rs:30) and ``matmul`` (crates/lapid-cpu/src/matmul/mod.rs:165).
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import tempfile
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "lapid_oracle.c")

# dtype codes shared with crates/lapid-c/src/lib.rs:37-60
INT8, INT4, Q4_K, Q5_K, Q6_K, MXFP4 = 4, 5, 6, 7, 8, 9
IQ2_XXS, IQ2_S, IQ3_XXS, IQ2_XS = 10, 11, 12, 13
IQUANTS = (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS)
FORMATS = {"int8": INT8, "int4": INT4, "q4_k": Q4_K, "q5_k": Q5_K, "q6_k": Q6_K, "mxfp4": MXFP4,
           "iq2_xxs": IQ2_XXS, "iq2_xs": IQ2_XS, "iq2_s": IQ2_S, "iq3_xxs": IQ3_XXS}
BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210, MXFP4: 17, IQ2_XXS: 66, IQ2_XS: 74, IQ2_S: 82, IQ3_XXS: 98}
# The i-quant codebooks: the reference's own fixture (crates/lapid-quant/tests/fixtures/iquant/grids.bin), kept with the
# other golden files of the tests.
IQ_GRIDS = os.path.join(os.path.dirname(HERE), "tests", "golden", "iquant", "grids.bin")

ERRORS = {1: "invalid_launch", 2: "shape_mismatch", 3: "out_of_bounds", 4: "unsupported_dtype"}


class OracleError(RuntimeError):
    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code


class _View(C.Structure):
    _fields_ = [("offset", C.c_size_t), ("batch_stride", C.c_size_t), ("row_stride", C.c_size_t)]


@dataclass(frozen=True)
class Layout:
    rows: int
    cols: int
    qs_offset: int
    qs_bytes: int
    scales_offset: int
    scales_bytes: int
    total: int


def _compile(out: str, flags: list[str]) -> None:
    cmd = ["gcc", "-std=c11", *flags, "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared",
           "-o", out, SRC, "-lm"]
    subprocess.run(cmd, check=True, capture_output=True)


def build() -> str:
    """Build the portable parity copy beside the source and return its path."""
    out = os.path.join(HERE, "liblapid_oracle.so")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(SRC):
        _compile(out, ["-O2"])
    return out


def _build_native() -> str:
    with open(SRC, "rb") as f:
        tag = hashlib.sha1(f.read()).hexdigest()[:12]
    try:
        with open("/proc/cpuinfo") as f:
            flags = next((l for l in f if l.startswith("flags")), "")
        tag += hashlib.sha1(flags.encode()).hexdigest()[:8]
    except OSError:
        pass
    out = os.path.join(tempfile.gettempdir(), f"liblapid_oracle_native_{tag}.so")
    if not os.path.exists(out):
        tmp = out + f".{os.getpid()}"
        _compile(tmp, ["-O3", "-march=native"])
        os.replace(tmp, out)
    return out


class Oracle:
    def __init__(self, path: str):
        lib = C.CDLL(path)
        self.lib = lib
        self.path = path
        sz = C.c_size_t
        lib.lo_f32_to_f16.restype = C.c_uint16
        lib.lo_f32_to_f16.argtypes = [C.c_float]
        lib.lo_f16_to_f32.restype = C.c_float
        lib.lo_f16_to_f32.argtypes = [C.c_uint16]
        lib.lo_nearest_int.restype = C.c_int
        lib.lo_nearest_int.argtypes = [C.c_float]
        lib.lo_layout.argtypes = [C.c_int, sz, sz, C.POINTER(sz)]
        lib.lo_quantize.argtypes = [C.c_int, C.c_void_p, sz, sz, C.c_void_p]
        lib.lo_dequantize.argtypes = [C.c_int, C.c_void_p, sz, sz, C.c_void_p]
        lib.lo_dequantize_row.argtypes = [C.c_int, C.c_void_p, sz, sz, sz, C.c_void_p]
        lib.lo_from_ggml_blocks.argtypes = [C.c_int, C.c_void_p, sz, sz, sz, C.c_void_p]
        lib.lo_quantize_row_sums.argtypes = [C.c_void_p, sz, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.lo_quantize_row_sums.restype = None
        lib.lo_quantize_q4k_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_quantize_q6k_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_dequantize_q4k_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_dequantize_q6k_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_quantize_q5k_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_dequantize_q5k_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_quantize_mxfp4_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_dequantize_mxfp4_block.argtypes = [C.c_void_p, C.c_void_p]
        lib.lo_mxfp4_from_e2m1_pairs.argtypes = [C.c_void_p, C.c_void_p, sz, sz, C.c_void_p]
        lib.lo_mxfp4_from_e2m1_pairs.restype = None
        lib.lo_set_iq_grids.argtypes = [C.c_void_p]
        lib.lo_set_iq_grids.restype = None
        lib.lo_dequantize_iq_block.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
        if os.path.exists(IQ_GRIDS):
            grids = np.fromfile(IQ_GRIDS, dtype=np.uint8)
            assert grids.size == 15488
            lib.lo_set_iq_grids(grids.ctypes.data)
        lib.lo_matmul.argtypes = [C.c_int, C.c_void_p, sz, _View, C.c_void_p, sz, sz, sz, C.c_void_p, C.c_void_p, sz,
                                  _View, sz, sz, sz, sz, C.c_int, C.c_int, C.POINTER(C.c_int)]
        lib.lo_num_threads.restype = C.c_int
        lib.lo_set_num_threads.argtypes = [C.c_int]

    # ---- scalar helpers
    def f32_to_f16_bits(self, v: float) -> int:
        return int(self.lib.lo_f32_to_f16(C.c_float(v)))

    def f16_bits_to_f32(self, h: int) -> float:
        return float(self.lib.lo_f16_to_f32(C.c_uint16(h)))

    def nearest_int(self, v: float) -> int:
        return int(self.lib.lo_nearest_int(C.c_float(v)))

    def num_threads(self) -> int:
        return int(self.lib.lo_num_threads())

    def set_num_threads(self, n: int) -> None:
        self.lib.lo_set_num_threads(int(n))

    # ---- lapid-quant surface
    def layout(self, fmt: int, rows: int, cols: int) -> Layout:
        out = (C.c_size_t * 5)()
        if self.lib.lo_layout(fmt, rows, cols, out) != 0:
            raise OracleError("invalid_launch", f"format {fmt}: cols {cols} is not a multiple of the block length")
        return Layout(rows, cols, *[int(x) for x in out])

    def quantize(self, fmt: int, data: np.ndarray, rows: int, cols: int) -> np.ndarray:
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        if data.size != rows * cols:
            raise OracleError("shape_mismatch", f"quantize: data has {data.size} elements, expected {rows}x{cols}")
        l = self.layout(fmt, rows, cols)
        out = np.empty(l.total, dtype=np.uint8)
        if self.lib.lo_quantize(fmt, data.ctypes.data, rows, cols, out.ctypes.data) != 0:
            raise OracleError("invalid_launch", "quantize: bad format or shape")
        return out

    def dequantize(self, fmt: int, qbytes: np.ndarray, rows: int, cols: int) -> np.ndarray:
        qbytes = np.ascontiguousarray(qbytes, dtype=np.uint8)
        l = self.layout(fmt, rows, cols)
        if qbytes.size < l.scales_offset + l.scales_bytes:
            raise OracleError("out_of_bounds", f"dequantize: buffer too small ({qbytes.size} < {l.total})")
        out = np.empty((rows, cols), dtype=np.float32)
        if self.lib.lo_dequantize(fmt, qbytes.ctypes.data, rows, cols, out.ctypes.data) != 0:
            raise OracleError("invalid_launch", "dequantize: bad format or shape")
        return out

    def from_ggml_blocks(self, fmt: int, blocks: np.ndarray, rows: int, cols: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        l = self.layout(fmt, rows, cols)
        out = np.empty(l.total, dtype=np.uint8)
        rc = self.lib.lo_from_ggml_blocks(fmt, blocks.ctypes.data, blocks.size, rows, cols, out.ctypes.data)
        if rc == -2:
            raise OracleError("shape_mismatch", f"from_ggml_blocks: got {blocks.size} bytes for [{rows}, {cols}]")
        if rc != 0:
            raise OracleError("invalid_launch", "from_ggml_blocks: bad format or shape")
        return out

    def quantize_block(self, fmt: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        assert x.size == (32 if fmt == MXFP4 else 256)
        out = np.empty(BLOCK_BYTES[fmt], dtype=np.uint8)
        {Q4_K: self.lib.lo_quantize_q4k_block, Q5_K: self.lib.lo_quantize_q5k_block,
         Q6_K: self.lib.lo_quantize_q6k_block, MXFP4: self.lib.lo_quantize_mxfp4_block}[fmt](x.ctypes.data, out.ctypes.data)
        return out

    def dequantize_block(self, fmt: int, b: np.ndarray) -> np.ndarray:
        b = np.ascontiguousarray(b, dtype=np.uint8)
        out = np.empty(32 if fmt == MXFP4 else 256, dtype=np.float32)
        if fmt in IQUANTS:
            if self.lib.lo_dequantize_iq_block(fmt, b.ctypes.data, out.ctypes.data) != 0:
                raise OracleError("unsupported_dtype", "i-quant codebooks not loaded")
            return out
        {Q4_K: self.lib.lo_dequantize_q4k_block, Q5_K: self.lib.lo_dequantize_q5k_block,
         Q6_K: self.lib.lo_dequantize_q6k_block, MXFP4: self.lib.lo_dequantize_mxfp4_block}[fmt](b.ctypes.data, out.ctypes.data)
        return out

    def mxfp4_from_e2m1_pairs(self, packed: np.ndarray, scales: np.ndarray, rows: int, cols: int) -> np.ndarray:
        """`from_e2m1_pairs` (crates/lapid-quant/src/mxfp4.rs:61-84): torch-style packed e2m1 pairs + e8m0 scales -> MXFP4 blocks."""
        packed = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
        scales = np.ascontiguousarray(scales, dtype=np.uint8).reshape(-1)
        assert cols % 32 == 0 and packed.size == rows * cols // 2 and scales.size == rows * cols // 32
        out = np.empty(rows * cols // 32 * 17, dtype=np.uint8)
        self.lib.lo_mxfp4_from_e2m1_pairs(packed.ctypes.data, scales.ctypes.data, C.c_size_t(rows), C.c_size_t(cols), out.ctypes.data)
        return out

    # ---- lapid-cpu surface
    def quantize_row_sums(self, x: np.ndarray, want_bs: bool = True):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        k = x.size
        assert k % 32 == 0
        q = np.empty(k, dtype=np.int8)
        s = np.empty(k // 32, dtype=np.float32)
        bs = np.empty(k // 32, dtype=np.float32) if want_bs else None
        self.lib.lo_quantize_row_sums(x.ctypes.data, k, q.ctypes.data, s.ctypes.data, bs.ctypes.data if want_bs else None)
        return q, s, bs

    def matmul(self, fmt: int, a: np.ndarray, w: np.ndarray, n: int, k: int, *, batch: int = 1, m: int | None = None,
               a_view: tuple[int, int, int] | None = None, out: np.ndarray | None = None,
               out_view: tuple[int, int, int] | None = None, bias: np.ndarray | None = None,
               w_shape: tuple[int, int] | None = None, force_f32_act: bool = False, fma: bool = True):
        """Run one MatMul launch with a quantized, transposed B. Returns ``(out, path)``; ``path`` is
        "int8_act" or "f32_act". Views are ``(offset, batch_stride, row_stride)`` in elements."""
        a = np.ascontiguousarray(a, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        flat = a.reshape(-1)
        if m is None:
            m = flat.size // (batch * k) if k else 0
        av = a_view or (0, m * k, k)
        ov = out_view or (0, m * n, n)
        if out is None:
            out = np.zeros(batch * m * n, dtype=np.float32)
        oflat = out.reshape(-1)
        assert oflat.flags.c_contiguous and oflat.dtype == np.float32
        if bias is not None:
            bias = np.ascontiguousarray(bias, dtype=np.float32)
        wr, wc = w_shape or (n, k)
        path = C.c_int(-1)
        rc = self.lib.lo_matmul(fmt, flat.ctypes.data, flat.size, _View(*av), w.ctypes.data, w.size, wr, wc,
                                bias.ctypes.data if bias is not None else None, oflat.ctypes.data, oflat.size,
                                _View(*ov), batch, m, n, k, int(force_f32_act), int(fma), C.byref(path))
        if rc != 0:
            raise OracleError(ERRORS.get(rc, "backend"), f"matmul [{batch},{m},{n},{k}] format {fmt}")
        return out, {0: "int8_act", 1: "f32_act"}.get(path.value, "none")


    def matmul_id(self, fmt: int, x: np.ndarray, w: np.ndarray, ids: np.ndarray, t: int, r: int, e: int, n: int, k: int):
        """``Kernel::MatMulId`` as lapid-cpu runs it (crates/lapid-cpu/src/moe.rs:21-120): the (token, slot)
        pairs are grouped by expert, every used expert runs ONE ordinary matmul over its gathered token
        rows -- with float activations for every expert when t > 8 (:107-109), else by its own row count
        -- and the result rows are scattered back. ``w`` is the stack of ``e`` matrices, ``layout(n, k).total``
        bytes each. Returns out [t, r, n]."""
        out = np.zeros((t * r, n), dtype=np.float32)
        if t * r * n == 0:
            return out.reshape(t, r, n)
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)[: t * k].reshape(t, k)
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        if ids.size < t * r:
            raise OracleError("out_of_bounds", "matmul_id: ids too small")
        by_expert: list[list[int]] = [[] for _ in range(e)]
        for i, ex in enumerate(ids[: t * r]):
            if ex < 0 or ex >= e:
                raise OracleError("index_out_of_range", f"matmul_id: expert id {ex} at position {i} out of range for {e} experts")
            by_expert[int(ex)].append(i)
        one = self.layout(fmt, n, k).total
        w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
        if w.size < e * one:
            raise OracleError("out_of_bounds", "matmul_id: expert stack too small")
        for ex, rows in enumerate(by_expert):
            if not rows:
                continue
            a = x[[i // r for i in rows]]
            res, _ = self.matmul(fmt, a, w[ex * one:(ex + 1) * one], n, k, m=len(rows), force_f32_act=t > 8)
            out[rows] = res.reshape(len(rows), n)
        return out.reshape(t, r, n)


_cache: dict[bool, Oracle] = {}


def epilogue(words, acc: np.ndarray, extra: np.ndarray | None = None) -> np.ndarray:
    """The reference's epilogue expression (`Epilogue::apply`, crates/lapid-cpu/src/matmul/mod.rs:133-161, over the
    expression type of crates/lapid-compiler/src/ir.rs:94-111, f32 nodes) evaluated element by element: `words` is the
    postfix program of the C ABI (one word per node, op | arg << 8; 2 = constant, followed by its bits), Load(0) = `acc`,
    Load(1) = `extra`. Every node is one f32 numpy operation (lapid-cpu has polynomial exp / erf of its own: a few ulp
    from these)."""
    f = np.float32
    acc = np.asarray(acc, f)
    st, i = [], 0
    un = {16: np.negative, 17: np.exp, 18: np.log, 19: np.sqrt, 20: lambda x: f(1) / np.sqrt(x), 21: lambda x: f(1) / x, 22: np.sin,
          23: np.cos, 24: np.tanh, 26: np.abs}
    bi = {32: np.add, 33: np.subtract, 34: np.multiply, 35: np.divide, 36: np.maximum, 37: np.minimum, 38: np.power,
          39: lambda a, b: (a < b).astype(f), 40: lambda a, b: (a == b).astype(f)}
    with np.errstate(all="ignore"):
        while i < len(words):
            w = int(words[i]); op, arg = w & 0xff, w >> 8
            if op == 1:
                st.append(acc if arg == 0 else np.broadcast_to(np.asarray(extra, f), acc.shape))
            elif op == 2:
                i += 1
                st.append(np.full(acc.shape, np.uint32(words[i]).view(f), f))
            elif op == 25:
                import math
                st.append(np.vectorize(math.erf, otypes=[np.float64])(st.pop().astype(np.float64)).astype(f))
            elif op in un:
                st.append(un[op](st.pop()).astype(f))
            elif op in bi:
                b = st.pop(); a = st.pop()
                st.append(bi[op](a, b).astype(f))
            elif op == 48:
                b = st.pop(); a = st.pop(); c = st.pop()
                st.append(np.where(c != 0, a, b).astype(f))
            else:
                raise OracleError("unsupported", f"epilogue node {op}")
            i += 1
    if len(st) != 1:
        raise OracleError("invalid_launch", f"epilogue expression leaves {len(st)} values")
    return st[0]


def load(fast: bool = False) -> Oracle:
    """The parity copy by default; ``fast=True`` compiles and loads the timed ``-march=native`` copy."""
    if fast not in _cache:
        _cache[fast] = Oracle(_build_native() if fast else build())
    return _cache[fast]


# ---------------------------------------------------------------------------------------------
# Seeded synthetic inputs shared by the oracle side and the GPU side of every parity test: a
# counter-based generator, so any slice can be produced independently and identically anywhere.
# value(seed, i) = std * sqrt(-2 ln u1) * cos(2 pi u2), with (u1, u2) from splitmix64(seed * 2^40 + i).
def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def normal(seed: int, n: int, std: float = 1.0, start: int = 0) -> np.ndarray:
    """``n`` float32 draws of N(0, std) for counters ``start .. start + n``."""
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + n, dtype=np.uint64) + (np.uint64(seed) << np.uint64(40))
        h = _splitmix64(idx)
    u1 = ((h >> np.uint64(40)).astype(np.float64) + 1.0) / 16777217.0   # (0, 1)
    u2 = ((h >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) / 16777216.0
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).astype(np.float32)
