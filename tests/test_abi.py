"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares,
its host-only functions agree with the oracle, and device functions fail loudly (never fall back)
when no GPU is present."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import lapid_b200 as lp
from lapid_b200 import _lib, quant
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "lapid_b200.h")).read()
    declared = set(re.findall(r"LAPID_B200_API[^;(]*?\b(lapid_b200_\w+)\s*\(", hdr))
    assert len(declared) >= 25
    lib = C.CDLL(lp.library_path())
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    # and the Python binding declares a signature for each of them
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)


def test_abi_version_and_mismatch_error_json():
    assert lp.abi_version() == 1
    assert _lib.lib().lapid_b200_check_abi(1) == 0
    st = _lib.lib().lapid_b200_check_abi(7)
    assert st == 11  # LAPID_ERR_ABI_MISMATCH
    d = json.loads(_lib.lib().lapid_b200_last_error().decode())
    assert d["status"] == 11 and d["error"] == "abi_mismatch" and "7" in d["message"]


def test_layout_matches_oracle_and_reference_sizes(oracle):
    for fmt in (quant.Format.Int8, quant.Format.Int4, quant.Format.Q4K, quant.Format.Q5K, quant.Format.Q6K, quant.Format.MXFP4,
                quant.Format.Iq2Xxs, quant.Format.Iq2Xs, quant.Format.Iq2S, quant.Format.Iq3Xxs):
        for rows, cols in [(1, 256), (3, 512), (768, 768 if fmt.block_elems() == 32 else 1024), (4096, 4096), (14336, 4096),
                           (4096, 14336), (128256, 4096)]:
            a, b = quant.layout(fmt, rows, cols), oracle.layout(int(fmt), rows, cols)
            assert (a.qs_offset, a.qs_bytes, a.scales_offset, a.scales_bytes, a.total) == \
                   (b.qs_offset, b.qs_bytes, b.scales_offset, b.scales_bytes, b.total)
    l = quant.layout(quant.Format.Int8, 1, 32)
    assert (l.qs_bytes, l.scales_offset, l.scales_bytes, l.total) == (32, 256, 2, 512)
    l = quant.layout(quant.Format.Int4, 1, 32)
    assert (l.qs_bytes, l.scales_offset, l.scales_bytes, l.total) == (16, 256, 2, 512)
    with pytest.raises(lp.LapidError) as e:
        quant.layout(quant.Format.Q4K, 2, 128)
    assert e.value.code == "invalid_launch" and e.value.status == 8
    l = quant.layout(quant.Format.MXFP4, 2, 128)  # 8 blocks of 17 bytes (crates/lapid-quant/src/lib.rs:62-75, :108-112)
    assert (l.qs_bytes, l.scales_offset, l.scales_bytes, l.total) == (136, 136, 0, 256)
    l = quant.layout(quant.Format.Iq2Xxs, 2, 512)  # 4 blocks of 66 bytes (crates/lapid-quant/tests/iquant_golden.rs:88-99)
    assert (l.qs_bytes, l.scales_offset, l.scales_bytes, l.total) == (264, 264, 0, 512)
    assert [quant.layout(f, 1, 256).qs_bytes for f in (quant.Format.Iq2Xs, quant.Format.Iq2S, quant.Format.Iq3Xxs)] == [74, 82, 98]
    with pytest.raises(lp.LapidError) as e:
        quant.layout(14, 2, 256)  # no such dtype code
    assert e.value.code == "unsupported_dtype" and e.value.status == 3


def test_null_arguments_are_rejected_not_dereferenced():
    lib = _lib.lib()
    assert lib.lapid_b200_device_open(0, None) == 1
    assert lib.lapid_b200_alloc(None, 16, None) == 1
    assert lib.lapid_b200_execute(None, None, 0, None, 0) == 1
    assert lib.lapid_b200_buffer_size(None) == 0
    lib.lapid_b200_buffer_free(None)
    lib.lapid_b200_device_free(None)
    lib.lapid_b200_device_retain(None)


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_loud_failure_not_fallback():
    with pytest.raises(lp.LapidError) as e:
        lp.Backend(0)
    assert e.value.status == 7  # LAPID_ERR_DEVICE_UNAVAILABLE
    assert e.value.code in ("cuda_unavailable", "device_unavailable")


def test_launch_marshalling_matches_header_struct():
    l = lp.backend.matmul_launch(lp.DType.Q6K, 3, 20, 256, a_row_stride=260, bias_input=3)
    c = l.to_c()
    assert (c.kind, c.b_dtype, c.n_inputs, c.epilogue) == (2, 8, 3, 1)
    assert (c.a.row_stride, c.a.batch_stride, c.b.row_stride, c.out.row_stride) == (260, 780, 256, 20)
    assert list(c.inputs) == [0, 1, 3] and c.output == 2 and list(c.extra.strides) == [0, 0, 1]
    # struct size as a C compiler lays it out: 8 int32 + 4 u64 + 3*3 u64 + (u64 + 3 i64) + 4 u32 + (1 + 24) u32, padded to 8
    assert C.sizeof(_lib.LaunchC) == 32 + 32 + 72 + 32 + 16 + 104
    assert C.sizeof(_lib.IoC) == 32 and _lib.IoC.host.offset == 16   # lapid_b200_io: u32 buffer, u32 launch, u64 offset, void *host, u64 bytes
    # an epilogue expression: postfix words, Load(1) makes the extra the third input
    e = lp.backend.Expr.silu(lp.backend.Expr.load(0)) * lp.backend.Expr.load(1)
    c = lp.backend.matmul_launch(lp.DType.Q4K, 2, 64, 256, expr=e, extra_input=5).to_c()
    assert (c.epilogue, c.n_inputs, c.n_expr, list(c.inputs)) == (2, 3, 11, [0, 1, 5])
    assert list(c.expr)[:11] == [1, 1, 16, 17, 2, 0x3F800000, 32, 21, 34, 1 | 1 << 8, 34] and list(c.extra.strides) == [128, 64, 1]
    c = lp.backend.matmul_launch(lp.DType.Q4K, 2, 64, 256, expr=lp.backend.Expr.load(0).tanh()).to_c()
    assert (c.n_inputs, c.n_expr) == (2, 2)
