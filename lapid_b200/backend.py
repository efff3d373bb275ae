"""Python mirror of the reference's backend interface for the quantized-matmul path.

Names and argument meanings follow ``lapid_compiler`` (crates/lapid-compiler/src/backend.rs:8-63,
crates/lapid-compiler/src/ir.rs:226-282, :483-488); every method is a thin call into the C ABI.
Errors are :class:`lapid_b200.LapidError` carrying the reference's error codes ("invalid_launch",
"shape_mismatch", "out_of_bounds", "buffer_aliasing", "unsupported_dtype", ...).
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import check


class DType(enum.IntEnum):
    """crates/lapid-tensor/src/dtype.rs:15-55, numbered as lapid-c does (crates/lapid-c/src/lib.rs:37-60)."""
    F32 = 0
    F16 = 1
    BF16 = 2
    I32 = 3
    Int8 = 4
    Int4 = 5
    Q4K = 6
    Q5K = 7
    Q6K = 8
    MXFP4 = 9
    Iq2Xxs = 10
    Iq2S = 11
    Iq3Xxs = 12
    Iq2Xs = 13
    ACT_Q8 = 100  # not a lapid dtype: an activation operand quantized by its producer (LAPID_B200_DTYPE_ACT_Q8)


class Epilogue(enum.IntEnum):
    """Epilogue kinds: none, ``Load(0) + Load(1)``, or an expression (:class:`Expr`) over the accumulator and extras[0]."""
    NONE = 0
    ADD = 1
    EXPR = 2


@dataclass(frozen=True)
class MatView:
    """ir.rs:249-261 -- element offsets and strides."""
    offset: int = 0
    batch_stride: int = 0
    row_stride: int = 0

    @staticmethod
    def contiguous(rows: int, cols: int) -> "MatView":
        return MatView(0, rows * cols, cols)


@dataclass(frozen=True)
class View:
    """View of an epilogue extra over [batch, m, n]."""
    offset: int = 0
    strides: tuple = (0, 0, 1)


class Expr:
    """The f32 part of the reference's epilogue expression type (crates/lapid-compiler/src/ir.rs:94-111) as a
    postfix program for ``LAPID_B200_EPILOGUE_EXPR``: ``Expr.load(0)`` is the accumulator, ``Expr.load(1)`` extras[0];
    unary nodes are methods (``neg exp log sqrt rsqrt recip sin cos tanh erf abs``, crates/lapid-tensor/src/op.rs:11-23),
    binary ones operators and methods (``+ - * /``, ``max min pow lt eq``), ``Expr.where(cond, a, b)``; Python numbers
    become constants. ``Expr.silu(x)`` and ``Expr.gelu_tanh(x)`` build what lapid-nn's activations build
    (crates/lapid-nn/src/ops.rs:12-30)."""
    _UN = {"neg": 16, "exp": 17, "log": 18, "sqrt": 19, "rsqrt": 20, "recip": 21, "sin": 22, "cos": 23, "tanh": 24, "erf": 25, "abs": 26}
    _BIN = {"add": 32, "sub": 33, "mul": 34, "div": 35, "max": 36, "min": 37, "pow": 38, "lt": 39, "eq": 40}

    def __init__(self, words):
        self.words = tuple(int(w) for w in words)

    @staticmethod
    def load(i: int) -> "Expr":
        return Expr([1 | (i << 8)])

    @staticmethod
    def const(v: float) -> "Expr":
        return Expr([2, int(np.float32(v).view(np.uint32))])

    @staticmethod
    def _of(v) -> "Expr":
        return v if isinstance(v, Expr) else Expr.const(v)

    def _un(self, name):
        return Expr(self.words + (Expr._UN[name],))

    def _bin(self, name, other, swap=False):
        a, b = (Expr._of(other), self) if swap else (self, Expr._of(other))
        return Expr(a.words + b.words + (Expr._BIN[name],))

    @staticmethod
    def where(cond, a, b) -> "Expr":
        return Expr(Expr._of(cond).words + Expr._of(a).words + Expr._of(b).words + (48,))

    @staticmethod
    def sigmoid(x: "Expr") -> "Expr":
        return (x.neg().exp() + 1.0).recip()

    @staticmethod
    def silu(x: "Expr") -> "Expr":
        return x * Expr.sigmoid(x)

    @staticmethod
    def gelu_tanh(x: "Expr") -> "Expr":
        inner = (x * x * x * 0.044715 + x) * 0.7978845608028654
        return x * 0.5 * (inner.tanh() + 1.0)

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __truediv__(self, o): return self._bin("div", o)
    def __rtruediv__(self, o): return self._bin("div", o, True)
    def __neg__(self): return self._un("neg")
    def max(self, o): return self._bin("max", o)
    def min(self, o): return self._bin("min", o)
    def pow(self, o): return self._bin("pow", o)
    def lt(self, o): return self._bin("lt", o)
    def eq(self, o): return self._bin("eq", o)

    def reads_extra(self) -> bool:
        i, n = 0, len(self.words)
        while i < n:
            w = self.words[i]
            if (w & 0xff) == 1 and (w >> 8) == 1:
                return True
            i += 2 if (w & 0xff) == 2 else 1
        return False


for _name in Expr._UN:
    setattr(Expr, _name, (lambda nm: lambda self: self._un(nm))(_name))


@dataclass(frozen=True)
class MatMulSpec:
    """ir.rs:239-247. ``epilogue`` is an :class:`Epilogue`; with ``Epilogue.EXPR`` the expression is ``expr``."""
    a_dtype: DType = DType.F32
    b_dtype: DType = DType.Q4K
    b_transposed: bool = True
    extra_dtypes: tuple = ()
    out_dtype: DType = DType.F32
    epilogue: Epilogue = Epilogue.NONE
    expr: Optional[Expr] = None


@dataclass(frozen=True)
class MatMulDims:
    """ir.rs:263-274."""
    batch: int
    m: int
    n: int
    k: int
    a: MatView
    b: MatView
    out: MatView
    extra_views: tuple = ()


@dataclass(frozen=True)
class Launch:
    """ir.rs:483-488 with ``kernel = Kernel::MatMul(spec, dims)``; inputs/output are BufIds."""
    spec: MatMulSpec
    dims: MatMulDims
    inputs: tuple
    output: int
    kind: int = 2  # LAPID_B200_KERNEL_MATMUL

    def to_c(self) -> _lib.LaunchC:
        s, d = self.spec, self.dims
        c = _lib.LaunchC()
        c.kind = self.kind
        c.a_dtype, c.b_dtype, c.out_dtype = int(s.a_dtype), int(s.b_dtype), int(s.out_dtype)
        c.b_transposed = int(bool(s.b_transposed))
        c.epilogue = int(s.epilogue)
        if s.expr is not None:
            if len(s.expr.words) > 24:
                raise _lib.LapidError(8, "unsupported", f"an epilogue expression of {len(s.expr.words)} words (at most 24)")
            c.n_expr = len(s.expr.words)
            for i, w in enumerate(s.expr.words):
                c.expr[i] = w
        c.extra_dtype = int(s.extra_dtypes[0]) if s.extra_dtypes else 0
        c.n_inputs = len(self.inputs)
        c.batch, c.m, c.n, c.k = d.batch, d.m, d.n, d.k
        for name, v in (("a", d.a), ("b", d.b), ("out", d.out)):
            mv = getattr(c, name)
            mv.offset, mv.batch_stride, mv.row_stride = v.offset, v.batch_stride, v.row_stride
        if d.extra_views:
            ev = d.extra_views[0]
            c.extra.offset = ev.offset
            for i in range(3):
                c.extra.strides[i] = ev.strides[i]
        if len(self.inputs) > 3:
            raise _lib.LapidError(8, "invalid_launch", f"expected at most 3 inputs, got {len(self.inputs)}")
        for i, b in enumerate(self.inputs):
            c.inputs[i] = b
        c.output = self.output
        return c


def matmul_launch(b_dtype: DType, m: int, n: int, k: int, *, batch: int = 1, a_row_stride: Optional[int] = None,
                  inputs=(0, 1), output=2, bias_input: Optional[int] = None, out: Optional[MatView] = None,
                  a_quantized: bool = False, a_dtype: DType = DType.F32, expr: Optional[Expr] = None, extra_input: Optional[int] = None,
                  extra_view: Optional[View] = None, a: Optional[MatView] = None) -> Launch:
    """The launch lapid lowers ``x.matmul_t(w)`` to: contiguous A (or padded rows), quantized
    transposed B, contiguous f32 output (the `mm` helper of kbench_tests.rs:86-107).
    ``a_quantized``: input 0 is the quantized operand a producer wrote for this launch (``Backend.act_layout``);
    ``a_dtype``: F32, F16 or BF16 activations (widened exactly to f32 as they are read, like lapid-cpu's ``load_contig``);
    ``expr``: an epilogue expression; when it loads extras[0], ``extra_input`` is that buffer and ``extra_view`` its view
    over [batch, m, n] (default: a contiguous [m, n] array); ``a``: the view of A inside its buffer (default: at the start)."""
    rs = a_row_stride if a_row_stride is not None else k
    if expr is not None:
        has = expr.reads_extra()
        spec = MatMulSpec(a_dtype=DType.ACT_Q8 if a_quantized else DType(a_dtype), b_dtype=DType(b_dtype), extra_dtypes=(DType.F32,) if has else (),
                          epilogue=Epilogue.EXPR, expr=expr)
        dims = MatMulDims(batch, m, n, k, a=a or MatView(0, m * rs, rs), b=MatView(0, 0, k), out=out or MatView.contiguous(m, n),
                          extra_views=((extra_view or View(0, (m * n, n, 1)),) if has else ()))
        return Launch(spec, dims, tuple(inputs) + ((extra_input,) if has else ()), output)
    spec = MatMulSpec(a_dtype=DType.ACT_Q8 if a_quantized else DType(a_dtype), b_dtype=DType(b_dtype), extra_dtypes=(DType.F32,) if bias_input is not None else (),
                      epilogue=Epilogue.ADD if bias_input is not None else Epilogue.NONE)
    dims = MatMulDims(batch, m, n, k, a=a or MatView(0, m * rs, rs), b=MatView(0, 0, k), out=out or MatView.contiguous(m, n),
                      extra_views=(View(0, (0, 0, 1)),) if bias_input is not None else ())
    ins = tuple(inputs) + ((bias_input,) if bias_input is not None else ())
    return Launch(spec, dims, ins, output)


def gather_launch(table_dtype: DType, rows: int, cols: int, count: int, *, inputs=(0, 1), output=2) -> Launch:
    """``Kernel::Gather`` (ir.rs:284-300): ``out[i, :] = dequant(table[ids[i], :])`` for a table of
    ``rows x cols`` (f32 or a lapid-quant matrix) and ``count`` i32 indices; inputs = (table, indices)."""
    spec = MatMulSpec(b_dtype=DType(table_dtype))
    dims = MatMulDims(1, count, cols, rows, a=MatView(), b=MatView(), out=MatView.contiguous(count, cols))
    return Launch(spec, dims, tuple(inputs), output, kind=3)


def matmul_id_launch(w_dtype: DType, t: int, r: int, e: int, n: int, k: int, *, inputs=(0, 1, 2), output=3) -> Launch:
    """``Kernel::MatMulId`` (ir.rs:425-443): ``out[t, s, :] = W[ids[t, s]] @ x[t]`` over a stack of ``e``
    quantized matrices ``[n, k]`` (each ``layout(n, k).total`` bytes); inputs = (x f32 [t, k], w, ids i32 [t, r]),
    output f32 [t, r, n]."""
    spec = MatMulSpec(b_dtype=DType(w_dtype))
    dims = MatMulDims(r, t, n, k, a=MatView.contiguous(t, k), b=MatView(0, e, k), out=MatView.contiguous(t * r, n))
    return Launch(spec, dims, tuple(inputs), output, kind=4)


class Buffer:
    """``DeviceData``: a reference-counted device buffer handle."""

    def __init__(self, backend: "Backend", handle: int, keep=None):
        self.backend = backend
        self._h = C.c_void_p(handle)
        self._keep = keep  # whatever owns wrapped memory (e.g. a torch tensor)

    @property
    def nbytes(self) -> int:
        return int(_lib.lib().lapid_b200_buffer_size(self._h))

    @property
    def device_ptr(self) -> int:
        return int(_lib.lib().lapid_b200_buffer_device_ptr(self._h) or 0)

    def write(self, offset: int, data) -> None:
        self.backend.write(self, offset, data)

    def download(self, nbytes: Optional[int] = None) -> np.ndarray:
        return self.backend.download(self, nbytes)

    def free(self) -> None:
        if self._h:
            _lib.lib().lapid_b200_buffer_free(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _host_bytes(data) -> np.ndarray:
    arr = np.ascontiguousarray(data)
    return arr.reshape(-1).view(np.uint8)


class Backend:
    """``impl Backend`` for one B200. ``Backend(0)`` opens CUDA device 0."""

    def __init__(self, ordinal: int = 0):
        h = C.c_void_p()
        check(_lib.lib().lapid_b200_check_abi(1))
        check(_lib.lib().lapid_b200_device_open(ordinal, C.byref(h)))
        self._h = h
        self.ordinal = ordinal

    def name(self) -> str:
        return "b200"

    def device_name(self) -> str:
        buf = C.create_string_buffer(256)
        check(_lib.lib().lapid_b200_device_name(self._h, buf, 256))
        return buf.value.decode()

    def set_option(self, key: str, value: str) -> None:
        check(_lib.lib().lapid_b200_device_set_option(self._h, key.encode(), str(value).encode()))

    def set_stream(self, cuda_stream: int) -> None:
        check(_lib.lib().lapid_b200_device_set_stream(self._h, C.c_void_p(cuda_stream or None)))

    def synchronize(self) -> None:
        check(_lib.lib().lapid_b200_device_synchronize(self._h))

    # ---- buffers
    def alloc(self, nbytes: int) -> Buffer:
        h = C.c_void_p()
        check(_lib.lib().lapid_b200_alloc(self._h, nbytes, C.byref(h)))
        return Buffer(self, h.value)

    def upload(self, data) -> Buffer:
        b = _host_bytes(data)
        h = C.c_void_p()
        check(_lib.lib().lapid_b200_upload(self._h, b.ctypes.data, b.size, C.byref(h)))
        return Buffer(self, h.value)

    def wrap(self, device_ptr: int, nbytes: int, keep=None) -> Buffer:
        h = C.c_void_p()
        check(_lib.lib().lapid_b200_wrap(self._h, C.c_void_p(device_ptr), nbytes, C.byref(h)))
        return Buffer(self, h.value, keep)

    def wrap_tensor(self, t) -> Buffer:
        """A buffer over a contiguous CUDA torch tensor's memory (kept alive by the buffer)."""
        assert t.is_cuda and t.is_contiguous()
        return self.wrap(t.data_ptr(), t.numel() * t.element_size(), keep=t)

    def write(self, buf: Buffer, offset: int, data) -> None:
        b = _host_bytes(data)
        check(_lib.lib().lapid_b200_write(buf._h, offset, b.ctypes.data, b.size))

    def write_ptr(self, buf: Buffer, offset: int, host_ptr: int, nbytes: int) -> None:
        check(_lib.lib().lapid_b200_write(buf._h, offset, C.c_void_p(host_ptr), nbytes))

    def download(self, buf: Buffer, nbytes: Optional[int] = None) -> np.ndarray:
        n = buf.nbytes if nbytes is None else nbytes
        out = np.empty(n, dtype=np.uint8)
        check(_lib.lib().lapid_b200_download(buf._h, out.ctypes.data, n))
        return out

    def download_ptr(self, buf: Buffer, host_ptr: int, nbytes: int) -> None:
        check(_lib.lib().lapid_b200_download(buf._h, C.c_void_p(host_ptr), nbytes))

    # ---- launches
    @staticmethod
    def _pack(launches: Sequence[Launch], buffers: Sequence[Buffer]):
        arr = (_lib.LaunchC * len(launches))(*[l.to_c() for l in launches])
        bufs = (C.c_void_p * len(buffers))(*[b._h for b in buffers])
        return arr, bufs

    def prepare(self, launches: Sequence[Launch]) -> None:
        arr = (_lib.LaunchC * len(launches))(*[l.to_c() for l in launches])
        check(_lib.lib().lapid_b200_prepare(self._h, arr, len(launches)))

    def execute(self, launches: Sequence[Launch], buffers: Sequence[Buffer]) -> None:
        arr, bufs = self._pack(launches, buffers)
        check(_lib.lib().lapid_b200_execute(self._h, arr, len(launches), bufs, len(buffers)))

    def execute_async(self, launches: Sequence[Launch], buffers: Sequence[Buffer]) -> None:
        arr, bufs = self._pack(launches, buffers)
        check(_lib.lib().lapid_b200_execute_async(self._h, arr, len(launches), bufs, len(buffers)))

    def packed_io(self, launches: Sequence[Launch], buffers: Sequence[Buffer], writes: Sequence[tuple], reads: Sequence[tuple], chunk: int = 0):
        """One step with host buffers as one pipelined call (``lapid_b200_execute_io``): ``writes`` and ``reads`` are
        ``(buffer index, byte offset, host pointer, bytes, launch index)`` -- for a write the first launch that reads what
        it brings, for a read the last launch that writes what it takes. The launches run in chunks of ``chunk`` (0: the
        library picks); uploads, launches and downloads of different chunks overlap; the result is that of all writes,
        ``execute``, all reads. Host memory should be page-locked. Returns a zero-argument callable (pre-marshalled)."""
        arr, bufs = self._pack(launches, buffers)
        mk = lambda ios: (_lib.IoC * max(1, len(ios)))(*[_lib.IoC(int(b), int(l), int(off), C.c_void_p(int(h)), int(nb)) for (b, off, h, nb, l) in ios])
        w, r = mk(writes), mk(reads)
        fn, hd, n, nb_, nw, nr = _lib.lib().lapid_b200_execute_io, self._h, len(launches), len(buffers), len(writes), len(reads)

        def run():
            check(fn(hd, arr, n, bufs, nb_, w, nw, r, nr, chunk))
        run.keep = (arr, bufs, w, r, list(buffers))
        return run

    def execute_io(self, launches: Sequence[Launch], buffers: Sequence[Buffer], writes: Sequence[tuple], reads: Sequence[tuple], chunk: int = 0) -> None:
        self.packed_io(launches, buffers, writes, reads, chunk)()

    def packed(self, launches: Sequence[Launch], buffers: Sequence[Buffer]):
        """Pre-marshalled launch arrays for hot loops: returns a zero-argument callable that
        queues the launches asynchronously (no Python-side conversion per call)."""
        arr, bufs = self._pack(launches, buffers)
        fn, h, n, nb = _lib.lib().lapid_b200_execute_async, self._h, len(launches), len(buffers)

        def run():
            check(fn(h, arr, n, bufs, nb))
        run.keep = (arr, bufs, list(buffers))
        return run

    # ---- the steps between projections (queued on the device's stream, not waited for)
    def rms_norm(self, x: Buffer, out: Buffer, rows: int, cols: int, eps: float = 1e-6, residual: Optional[Buffer] = None,
                 weight: Optional[Buffer] = None, sum_out: Optional[Buffer] = None, qact: Optional[Buffer] = None,
                 layout: int = 0) -> None:
        """``out = h * rsqrt(mean(h*h) + eps) (* weight)`` with ``h = x (+ residual)``; ``sum_out`` receives h.
        ``qact``: also written as the quantized activation operand (``act_layout``) of the launches that read ``out``."""
        h = lambda b: b._h if b is not None else None
        check(_lib.lib().lapid_b200_rms_norm_act(self._h, x._h, h(residual), h(weight), h(sum_out), out._h, rows, cols, eps,
                                                 h(qact), layout))

    def silu_mul(self, gate: Buffer, up: Buffer, out: Buffer, count: int, *, rows: int = 1, qact: Optional[Buffer] = None,
                 layout: int = 0) -> None:
        """``out = silu(gate) * up`` over ``count`` f32 (``rows`` rows of ``count // rows``); ``qact`` as in ``rms_norm``."""
        check(_lib.lib().lapid_b200_silu_mul_act(self._h, gate._h, up._h, out._h, rows, count // rows,
                                                 qact._h if qact is not None else None, layout))

    def quantize_activations(self, a: Buffer, rows: int, k: int, layout: int, qact: Buffer) -> None:
        """``quantize_row_sums`` (crates/lapid-cpu/src/matmul/quant.rs:30-89) of ``rows`` f32 rows into ``qact`` in
        ``layout`` (0 planes, 1 records, 2 tiles): the decode path's activation pre-pass as a call of its own."""
        check(_lib.lib().lapid_b200_quantize_activations(self._h, a._h, rows, k, layout, qact._h))

    def act_layout(self, launch: "Launch") -> tuple:
        """``(layout, bytes)`` of the quantized activation operand a decode launch reads (``lapid_b200_act_layout``)."""
        lay, nbytes = C.c_int32(0), C.c_uint64(0)
        c = launch.to_c()
        check(_lib.lib().lapid_b200_act_layout(self._h, C.byref(c), C.byref(lay), C.byref(nbytes)))
        return int(lay.value), int(nbytes.value)

    def take_launch_count(self) -> int:
        return int(_lib.lib().lapid_b200_take_launch_count(self._h))

    def take_profile(self) -> list:
        """``Backend::take_profile``: ``[(kind, launches, ms)]`` since the last call, by time (option ``profile`` = "1")."""
        n = C.c_size_t(0)
        check(_lib.lib().lapid_b200_take_profile(self._h, None, 0, C.byref(n)))
        arr = (_lib.ProfileEntryC * max(1, n.value))()
        check(_lib.lib().lapid_b200_take_profile(self._h, arr, len(arr), C.byref(n)))
        return [(arr[i].kind.decode(), int(arr[i].launches), float(arr[i].ms)) for i in range(n.value)]

    def decode_trace_begin(self, launches: int) -> None:
        """Record the per-CTA timeline of the next ``launches`` launches of the balanced-stream decode kernel."""
        check(_lib.lib().lapid_b200_decode_trace_begin(self._h, launches))

    def decode_trace_read(self, max_launches: int) -> np.ndarray:
        """``[launches, ctas, 16]`` uint64 (see ``lapid_b200_decode_trace_begin`` in the header for the words)."""
        n, ctas = C.c_uint32(0), C.c_uint32(0)
        check(_lib.lib().lapid_b200_decode_trace_read(self._h, None, 0, C.byref(n), C.byref(ctas)))
        rows = min(int(n.value), max_launches)
        out = np.zeros((max(rows, 1), max(int(ctas.value), 1), 16), np.uint64)
        if rows:
            check(_lib.lib().lapid_b200_decode_trace_read(self._h, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n), C.byref(ctas)))
        return out[:rows]

    # ---- lapid-quant on the device
    def quantize_into(self, fmt: int, src: Buffer, rows: int, cols: int, dst: Buffer) -> None:
        check(_lib.lib().lapid_b200_quantize(self._h, int(fmt), src._h, rows, cols, dst._h))

    def dequantize_into(self, fmt: int, src: Buffer, rows: int, cols: int, dst: Buffer) -> None:
        check(_lib.lib().lapid_b200_dequantize(self._h, int(fmt), src._h, rows, cols, dst._h))

    def close(self) -> None:
        if self._h:
            _lib.lib().lapid_b200_device_free(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
