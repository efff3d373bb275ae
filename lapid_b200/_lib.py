"""ctypes declarations for ``liblapid_b200.so``. Loading fails loudly when the library is missing:
there is no other implementation to fall back to."""
from __future__ import annotations

import ctypes as C
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def library_path() -> str:
    return os.environ.get("LAPID_B200_LIBRARY", os.path.join(HERE, "liblapid_b200.so"))


class LapidError(RuntimeError):
    """``lapid_tensor::Error``: a stable string ``code`` plus a message, and the C status."""

    def __init__(self, status: int, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.status = status
        self.code = code
        self.message = message


class MatViewC(C.Structure):
    _fields_ = [("offset", C.c_uint64), ("batch_stride", C.c_uint64), ("row_stride", C.c_uint64)]


class View3C(C.Structure):
    _fields_ = [("offset", C.c_uint64), ("strides", C.c_int64 * 3)]


class LaunchC(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("a_dtype", C.c_int32), ("b_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("b_transposed", C.c_int32), ("epilogue", C.c_int32), ("extra_dtype", C.c_int32), ("n_inputs", C.c_int32),
        ("batch", C.c_uint64), ("m", C.c_uint64), ("n", C.c_uint64), ("k", C.c_uint64),
        ("a", MatViewC), ("b", MatViewC), ("out", MatViewC), ("extra", View3C),
        ("inputs", C.c_uint32 * 3), ("output", C.c_uint32),
        ("n_expr", C.c_uint32), ("expr", C.c_uint32 * 24),
    ]


class IoC(C.Structure):
    """lapid_b200_io: one host <-> device transfer of an execute_io call."""
    _fields_ = [("buffer", C.c_uint32), ("launch", C.c_uint32), ("offset", C.c_uint64), ("host", C.c_void_p), ("bytes", C.c_uint64)]


class ProfileEntryC(C.Structure):
    _fields_ = [("kind", C.c_char * 24), ("launches", C.c_uint64), ("ms", C.c_double)]


class LayoutC(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("rows", "cols", "qs_offset", "qs_bytes", "scales_offset", "scales_bytes", "total")]


# name -> (restype, argtypes); every symbol include/lapid_b200.h declares
P = C.c_void_p
SYMBOLS = {
    "lapid_b200_abi_version": (C.c_uint32, []),
    "lapid_b200_check_abi": (C.c_int32, [C.c_uint32]),
    "lapid_b200_last_error": (C.c_char_p, []),
    "lapid_b200_device_open": (C.c_int32, [C.c_int32, C.POINTER(P)]),
    "lapid_b200_device_retain": (None, [P]),
    "lapid_b200_device_free": (None, [P]),
    "lapid_b200_device_name": (C.c_int32, [P, C.c_char_p, C.c_size_t]),
    "lapid_b200_device_set_stream": (C.c_int32, [P, P]),
    "lapid_b200_device_synchronize": (C.c_int32, [P]),
    "lapid_b200_device_set_option": (C.c_int32, [P, C.c_char_p, C.c_char_p]),
    "lapid_b200_alloc": (C.c_int32, [P, C.c_size_t, C.POINTER(P)]),
    "lapid_b200_upload": (C.c_int32, [P, P, C.c_size_t, C.POINTER(P)]),
    "lapid_b200_wrap": (C.c_int32, [P, P, C.c_size_t, C.POINTER(P)]),
    "lapid_b200_write": (C.c_int32, [P, C.c_size_t, P, C.c_size_t]),
    "lapid_b200_download": (C.c_int32, [P, P, C.c_size_t]),
    "lapid_b200_buffer_retain": (None, [P]),
    "lapid_b200_buffer_free": (None, [P]),
    "lapid_b200_buffer_size": (C.c_size_t, [P]),
    "lapid_b200_buffer_device_ptr": (P, [P]),
    "lapid_b200_prepare": (C.c_int32, [P, C.POINTER(LaunchC), C.c_size_t]),
    "lapid_b200_execute": (C.c_int32, [P, C.POINTER(LaunchC), C.c_size_t, C.POINTER(P), C.c_size_t]),
    "lapid_b200_execute_async": (C.c_int32, [P, C.POINTER(LaunchC), C.c_size_t, C.POINTER(P), C.c_size_t]),
    "lapid_b200_execute_io": (C.c_int32, [P, C.POINTER(LaunchC), C.c_size_t, C.POINTER(P), C.c_size_t, C.POINTER(IoC), C.c_size_t,
                                         C.POINTER(IoC), C.c_size_t, C.c_size_t]),
    "lapid_b200_take_launch_count": (C.c_uint64, [P]),
    "lapid_b200_take_profile": (C.c_int32, [P, C.POINTER(ProfileEntryC), C.c_size_t, C.POINTER(C.c_size_t)]),
    "lapid_b200_decode_trace_begin": (C.c_int32, [P, C.c_uint32]),
    "lapid_b200_decode_trace_read": (C.c_int32, [P, P, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "lapid_b200_quant_layout": (C.c_int32, [C.c_int32, C.c_uint64, C.c_uint64, C.POINTER(LayoutC)]),
    "lapid_b200_dequantize": (C.c_int32, [P, C.c_int32, P, C.c_uint64, C.c_uint64, P]),
    "lapid_b200_quantize": (C.c_int32, [P, C.c_int32, P, C.c_uint64, C.c_uint64, P]),
    "lapid_b200_from_ggml_blocks": (C.c_int32, [P, C.c_int32, P, C.c_uint64, C.c_uint64, C.c_uint64, P]),
    "lapid_b200_tp_comm_bytes": (C.c_uint64, [C.c_int32, C.c_uint64]),
    "lapid_b200_tp_comm_create": (C.c_int32, [P, C.c_int32, C.c_int32, C.POINTER(P), C.c_uint64, C.POINTER(P)]),
    "lapid_b200_tp_comm_free": (None, [P]),
    "lapid_b200_tp_all_reduce": (C.c_int32, [P, P, C.c_uint64, C.c_uint64]),
    "lapid_b200_tp_matmul_push": (C.c_int32, [P, P, P, C.c_size_t]),
    "lapid_b200_tp_rms_norm": (C.c_int32, [P, P, P, P, P, C.c_uint64, C.c_uint64, C.c_float]),
    "lapid_b200_rms_norm": (C.c_int32, [P, P, P, P, P, P, C.c_uint64, C.c_uint64, C.c_float]),
    "lapid_b200_silu_mul": (C.c_int32, [P, P, P, P, C.c_uint64]),
    "lapid_b200_act_layout": (C.c_int32, [P, P, C.POINTER(C.c_int32), C.POINTER(C.c_uint64)]),
    "lapid_b200_quantize_activations": (C.c_int32, [P, P, C.c_uint64, C.c_uint64, C.c_int32, P]),
    "lapid_b200_rms_norm_act": (C.c_int32, [P, P, P, P, P, P, C.c_uint64, C.c_uint64, C.c_float, P, C.c_int32]),
    "lapid_b200_tp_rms_norm_act": (C.c_int32, [P, P, P, P, P, C.c_uint64, C.c_uint64, C.c_float, P, C.c_int32]),
    "lapid_b200_silu_mul_act": (C.c_int32, [P, P, P, P, C.c_uint64, C.c_uint64, P, C.c_int32]),
    "lapid_b200_gemv_q4k_static": (C.c_int32, [C.c_int32, P, P, P, C.c_uint64, P, C.c_uint32, C.c_uint32, C.c_uint32]),
    "lapid_b200_gemv_q4k_static_status": (C.c_int32, [C.c_int32, C.POINTER(C.c_int32)]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python -m lapid_b200.build` (nvcc, sm_100a). "
                "lapid_b200 has no other implementation to fall back to.")
        l = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def abi_version() -> int:
    return int(lib().lapid_b200_abi_version())


def check(status: int) -> None:
    if status == 0:
        return
    raw = lib().lapid_b200_last_error()
    try:
        d = json.loads(raw.decode()) if raw else {}
    except (ValueError, UnicodeDecodeError):
        d = {}
    raise LapidError(status, d.get("error", "internal"), d.get("message", f"status {status}"))
