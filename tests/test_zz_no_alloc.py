"""The allocation-free decode entry point, through the C ABI, against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test. The check calls `lapid_b200_gemv_q4k_static` twice in a row with different
inputs -- the second call finds the first call's leftovers in the shared static scratch -- and
compares each result with what `lapid_b200_execute` gives for the same launch. Both paths run the
same kernels on the same quantized activations, so the tolerance is the decode tests' (2e-5 of
max(|ref|, rms)); in practice the outputs are identical. It also checks the documented limits.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _max_rel(got, ref):
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = np.sqrt((ref ** 2).mean())
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), max(rms, 1e-30))).max())


def test_static_scratch_gemv_matches_execute_twice_in_a_row():
    import torch
    import lapid_b200 as lp
    from lapid_b200 import _lib, quant
    from lapid_b200.backend import matmul_launch
    from oracle import oracle as O

    lib = _lib.lib()
    be = lp.Backend(0)
    dev = torch.device("cuda", 0)
    # first call: 3 rows, k = 4096; second call: 1 row, k = 14336 (other shape, other scratch extent)
    for seed, (rows, n, k) in enumerate([(3, 640, 4096), (1, 333, 14336)]):
        w = O.normal(700 + seed, n * k, 0.02)
        qb = quant.quantize(be, quant.Format.Q4K, w, n, k)
        a = O.normal(800 + seed, rows * k)
        wt = torch.from_numpy(qb).to(dev)
        at = torch.from_numpy(a).to(dev)
        ot = torch.full((rows * n,), -7.0, device=dev)
        torch.cuda.synchronize()
        st = lib.lapid_b200_gemv_q4k_static(0, None, C.c_void_p(at.data_ptr()), C.c_void_p(wt.data_ptr()), wt.numel(),
                                            C.c_void_p(ot.data_ptr()), rows, n, k)
        assert st == 0, lib.lapid_b200_last_error()
        torch.cuda.synchronize()
        got = ot.cpu().numpy()
        bufs = [be.upload(a), be.upload(qb), be.alloc(rows * n * 4)]
        be.execute([matmul_launch(lp.DType.Q4K, rows, n, k)], bufs)
        ref = bufs[2].download().view(np.float32)
        assert _max_rel(got, ref) <= 2e-5
        want, _ = O.load().matmul(O.Q4_K, a, qb, n, k, m=rows)
        assert _max_rel(got, want) <= 2e-5
        assert torch.cuda.current_device() == 0   # the call puts the thread's device back
    word = C.c_int32(-1)
    assert lib.lapid_b200_gemv_q4k_static_status(0, C.byref(word)) == 0 and word.value == 0   # no wait gave up

    # limits: rows * k beyond the static scratch, bad rows, bad k, short weights -- clear errors, no launch
    z = torch.zeros(16, device=dev)
    p = C.c_void_p(z.data_ptr())
    assert lib.lapid_b200_gemv_q4k_static(0, None, p, p, 1 << 30, p, 8, 4, 16384) == 9      # too_large
    assert b"too_large" in lib.lapid_b200_last_error() and b"65536" in lib.lapid_b200_last_error()
    assert lib.lapid_b200_gemv_q4k_static(0, None, p, p, 1 << 30, p, 9, 4, 256) == 8        # rows
    assert lib.lapid_b200_gemv_q4k_static(0, None, p, p, 1 << 30, p, 1, 4, 100) == 8        # k % 256
    assert lib.lapid_b200_gemv_q4k_static(0, None, p, p, 100, p, 1, 4, 256) == 10           # weights too short
    assert lib.lapid_b200_gemv_q4k_static(0, None, None, p, 1 << 30, p, 1, 4, 256) == 1     # NULL
