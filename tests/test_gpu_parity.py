"""Parity of the CUDA path against the CPU oracle, through the C ABI, on a B200.

Bars (stated here, checked below):
  * dequantized weights, quantized bytes, layout conversion ........ bit / byte exact
  * decode (batch*m <= 8, int8 activations) vs the oracle's restatement of lapid-cpu:
        max_rel <= 1e-3  where max_rel = max|got-ref| / max(|ref|, rms(ref))   (expected ~1e-6:
        the integer dot products are exact, only the order of the f32 group sums differs)
  * exact-f32 GEMM (batch*m > 8) vs the oracle's qdeq with FMA accumulation ... bit exact
Shapes are the reference's own test shapes (crates/lapid-cpu/src/matmul/matmul_tests.rs:30-139,
crates/lapid/tests/round3_ops.rs:121-151) plus the benchmark's.
"""
import numpy as np
import pytest

import lapid_b200 as lp
from lapid_b200 import quant
from lapid_b200.backend import MatView, matmul_launch
from oracle import oracle as O
from tests.refgen import make_blocks, rnd

pytestmark = pytest.mark.gpu

FMTS = [(lp.DType.Int8, "int8"), (lp.DType.Int4, "int4"), (lp.DType.Q4K, "q4_k"), (lp.DType.Q5K, "q5_k"), (lp.DType.Q6K, "q6_k"),
        (lp.DType.MXFP4, "mxfp4")]
PLANES = (lp.DType.Int8, lp.DType.Int4)   # formats with 32-element groups in plane layout
GROUP32 = PLANES + (lp.DType.MXFP4,)      # formats whose K only has to be a multiple of 32


@pytest.fixture(scope="module")
def be():
    b = lp.Backend(0)
    # the tests of the tensor-core decode kernels use small matrices: keep those on the tensor-core kernels (the
    # default routing of small Q5_K / Q6_K launches has a test of its own)
    b.set_option("gemv_small_dp4a", "0")
    return b


def max_rel(got, ref):
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = np.sqrt((ref ** 2).mean())
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), max(rms, 1e-30))).max())


def rel_l2(got, ref):
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.sqrt(((got - ref) ** 2).sum() / max((ref ** 2).sum(), 1e-30)))


def run_matmul(be, fmt, a, qb, m, n, k, *, batch=1, a_row_stride=None, bias=None, out=None, out_view=None):
    bufs = [be.upload(a), be.upload(qb)]
    out_host = np.zeros(batch * m * n, np.float32) if out is None else out
    bufs.append(be.upload(out_host))
    bias_id = None
    if bias is not None:
        bufs.append(be.upload(bias))
        bias_id = 3
    l = matmul_launch(fmt, m, n, k, batch=batch, a_row_stride=a_row_stride, bias_input=bias_id, out=out_view)
    be.prepare([l])
    be.execute([l], bufs)
    return bufs[2].download().view(np.float32)


# ------------------------------------------------------------------ lapid-quant surface
def test_device_name_and_launch_counter(be):
    assert "B200" in be.device_name() or "sm_100a" in be.device_name()
    be.take_launch_count()
    x = O.normal(1, 256)
    qb = quant.quantize(be, quant.Format.Q4K, x, 1, 256)
    assert qb.size == 256 and be.take_launch_count() == 1


@pytest.mark.parametrize("fmt,name", FMTS)
def test_golden_vectors(be, oracle, fmt, name):
    g = np.load(__file__.replace("test_gpu_parity.py", "golden/golden.npz"))
    n, k = 24, 512
    w = O.normal(10 + int(fmt), n * k, 0.02)
    assert np.array_equal(quant.quantize(be, fmt, w, n, k), g[f"w_{name}"])          # quantizer bytes
    deq = quant.dequantize(be, fmt, g[f"w_{name}"], n, k)
    assert np.array_equal(deq.view(np.uint32), g[f"deq_{name}"])                      # dequant bits
    x3 = O.normal(20, 3 * k)
    y3 = run_matmul(be, fmt, x3, g[f"w_{name}"], 3, n, k)
    assert max_rel(y3, g[f"y3_{name}"]) <= 1e-3
    assert max_rel(y3, g[f"y3_{name}"]) <= 2e-5  # what the arithmetic should actually achieve
    x12 = O.normal(21, 12 * k)
    be.set_option("gemm", "f32")
    y12 = run_matmul(be, fmt, x12, g[f"w_{name}"], 12, n, k)
    be.set_option("gemm", "tc")
    assert np.array_equal(y12.view(np.uint32), g[f"y12_{name}"].reshape(-1).view(np.uint32))
    y12t = run_matmul(be, fmt, x12, g[f"w_{name}"], 12, n, k)  # tensor cores for Q4_K, exact kernel otherwise
    assert rel_l2(y12t, g[f"y12_{name}"]) <= 4e-3 and max_rel(y12t, g[f"y12_{name}"]) <= 2e-2


@pytest.mark.parametrize("fmt,name", FMTS)
def test_dequantize_bit_exact_random_blocks(be, oracle, fmt, name):
    rows, cols = 16, 2048
    if fmt in PLANES:
        l = oracle.layout(int(fmt), rows, cols)
        rng = np.random.default_rng(3)
        qb = np.zeros(l.total, np.uint8)
        qb[:l.qs_bytes] = rng.integers(0, 256, l.qs_bytes, dtype=np.uint8)
        sc = (rng.standard_normal(rows * cols // 32) * 0.01).astype(np.float16)
        qb[l.scales_offset:l.scales_offset + l.scales_bytes] = sc.view(np.uint8)
    elif fmt == lp.DType.MXFP4:   # every byte pattern is a valid block; scale bytes include 0, 1 (denormal d) and 255
        raw = np.random.default_rng(4).integers(0, 256, rows * cols // 32 * 17, dtype=np.uint8)
        raw.reshape(-1, 17)[:6, 0] = [0, 1, 2, 127, 254, 255]
        qb = np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])
    else:
        bb, d_off, dm_off = {lp.DType.Q4K: (144, 0, 2), lp.DType.Q5K: (176, 0, 2), lp.DType.Q6K: (210, 208, None)}[fmt]
        raw = make_blocks(bb, rows * cols // 256, 7, d_off, dm_off)
        b2 = raw.reshape(-1, bb)
        ds = np.array([0.01, 0.25, 3e-5, -0.02, 6e-8, 1.5, 0.003, 7.0], np.float16).view(np.uint8).reshape(8, 2)
        for i in range(b2.shape[0]):
            b2[i, d_off:d_off + 2] = ds[i % 8]
            if dm_off is not None:
                b2[i, dm_off:dm_off + 2] = ds[(i * 3 + 1) % 8]
        qb = np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])
    want = oracle.dequantize(int(fmt), qb, rows, cols)
    got = quant.dequantize(be, fmt, qb, rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt,name", FMTS)
def test_quantize_byte_exact(be, oracle, fmt, name):
    rows, cols = 37, 1024
    x = O.normal(40 + int(fmt), rows * cols, 0.02).reshape(rows, cols)
    x[3, 256:512] = 0.0            # an all-zero super-block
    x[4, :256] = 1.0               # constants
    x[5, 0:32] = -2.5
    x[6, 17] = 4.0                 # an outlier
    x[7, 300:330] = np.abs(x[7, 300:330])  # a sub-block with min > 0
    x[8, :] *= 1e-20               # values below the quantizers' epsilon
    x[9, :64] = np.linspace(-1, 1, 64, dtype=np.float32)
    if fmt == lp.DType.MXFP4:   # what its scale choice, floor(log2(amax)), is sensitive to
        x[10, :32] = np.float32(8.0) * (1 - np.float32(2.0) ** -24)   # just below a power of two: its f32 log2 rounds up to 3
        x[10, 32:64] = np.nextafter(np.float32(0.25), np.float32(0))
        x[10, 64:96] = 3e-39                                            # denormals: the scale byte saturates at 0
        x[10, 96:128] = 1e30
        x[10, 128:160] = 2.0 ** -126
    want = oracle.quantize(int(fmt), x, rows, cols)
    got = quant.quantize(be, fmt, x, rows, cols)
    diff = np.flatnonzero(got != want)
    assert diff.size == 0, (name, diff[:10], got[diff[:10]], want[diff[:10]])


@pytest.mark.parametrize("fmt,name", FMTS)
def test_quantize_reference_noise_inputs(be, oracle, fmt, name):
    # the value distribution of the reference's own round-trip tests (uniform in [-2, 2))
    from tests.refgen import noise
    rows, cols = 3, 512
    x = noise(rows * cols, 11, 2.0)
    assert np.array_equal(quant.quantize(be, fmt, x, rows, cols), oracle.quantize(int(fmt), x, rows, cols))


def test_from_ggml_blocks(be, oracle):
    rows, cols = 3, 64
    x = O.normal(7, rows * cols)
    ours = oracle.quantize(O.INT8, x, rows, cols)
    l = oracle.layout(O.INT8, rows, cols)
    ng = rows * cols // 32
    blocks = np.empty((ng, 34), np.uint8)
    blocks[:, :2] = ours[l.scales_offset:l.scales_offset + 2 * ng].reshape(ng, 2)
    blocks[:, 2:] = ours[:ng * 32].reshape(ng, 32)
    assert np.array_equal(quant.from_ggml_blocks(be, quant.Format.Int8, blocks, rows, cols), ours)
    ours4 = oracle.quantize(O.INT4, x, rows, cols)          # GGUF block_q4_0: f16 d + 16 nibble bytes
    l4 = oracle.layout(O.INT4, rows, cols)
    b4 = np.empty((ng, 18), np.uint8)
    b4[:, :2] = ours4[l4.scales_offset:l4.scales_offset + 2 * ng].reshape(ng, 2)
    b4[:, 2:] = ours4[:ng * 16].reshape(ng, 16)
    assert np.array_equal(quant.from_ggml_blocks(be, quant.Format.Int4, b4, rows, cols), ours4)
    for fmt in (quant.Format.Q4K, quant.Format.Q6K):
        q = oracle.quantize(int(fmt), O.normal(8, 3 * 512, 0.02), 3, 512)
        lq = oracle.layout(int(fmt), 3, 512)
        assert np.array_equal(quant.from_ggml_blocks(be, fmt, q[:lq.qs_bytes], 3, 512), q)
        with pytest.raises(lp.LapidError) as e:
            quant.from_ggml_blocks(be, fmt, q[:lq.qs_bytes - 1], 3, 512)
        assert e.value.code == "shape_mismatch"


# ------------------------------------------------------------------ decode path
@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
def test_gemv_matches_oracle_all_row_counts(be, oracle, fmt, name, m):
    n, k = 301, 1024  # n not a multiple of any columns-per-task; k = half a stage
    w = O.normal(100 + int(fmt), n * k, 0.02)
    qb = oracle.quantize(int(fmt), w, n, k)
    a = O.normal(200 + m, m * k)
    want, path = oracle.matmul(int(fmt), a, qb, n, k, m=m)
    assert path == "int8_act"
    got = run_matmul(be, fmt, a, qb, m, n, k)
    assert max_rel(got, want) <= 1e-3
    assert max_rel(got, want) <= 2e-5


@pytest.mark.parametrize("fmt,name", FMTS)
def test_gemv_reference_test_shapes(be, oracle, fmt, name):
    # kquant_matmul_matches_dequantized_f32 (m <= 8 rows), with row padding, vs oracle and vs f64
    seed = 50
    for (m, n, k, pad) in [(1, 37, 512, 0), (3, 20, 256, 4), (6, 9, 256, 0), (1, 36, 768, 0), (3, 36, 768, 1),
                           (2, 1030, 4096, 0), (8, 77, 14336, 0), (1, 5, 2304, 0), (4, 50, 14336, 0), (3, 40, 8192, 8),
                           (2, 3, 16384, 0), (1, 300, 28672, 0)]:
        if fmt not in GROUP32 and k % 256:
            continue
        seed += 1
        w = rnd(n * k, seed) if n * k < 100000 else O.normal(seed, n * k, 0.5)
        qb = oracle.quantize(int(fmt), w, n, k)
        rs = k + pad
        a = rnd(m * rs, seed + 7) if m * rs < 100000 else O.normal(seed + 7, m * rs)
        want, _ = oracle.matmul(int(fmt), a, qb, n, k, m=m, a_view=(0, 0, rs))
        got = run_matmul(be, fmt, a, qb, m, n, k, a_row_stride=rs)
        assert max_rel(got, want) <= 1e-3, (name, m, n, k)
        deq = oracle.dequantize(int(fmt), qb, n, k).astype(np.float64)
        f64 = a.reshape(m, rs)[:, :k].astype(np.float64) @ deq.T
        assert rel_l2(got, f64) <= 2e-2  # the reference's own bound for its int8-activation path


@pytest.mark.parametrize("config", [-1, 0, 1, 2])
def test_gemv_q4k_tensor_core_decode_kernel(be, oracle, config):
    """The per-warp-ring int8 tensor-core decode kernel (what Q4_K launches of 2..8 rows take when the
    balanced-stream kernel is switched off) against the oracle and against the dp4a kernel, for every tile
    configuration, ragged n, odd super-block counts and a bias."""
    be.set_option("gemv_stream", "0")
    be.set_option("gemv_mma_config", str(config))
    try:
        seed = 900
        for (m, n, k, bias) in [(2, 130, 1024, False), (4, 77, 256, False), (5, 100, 768, True), (8, 513, 4096, False), (7, 33, 14336, True),
                                (8, 16, 512, False), (6, 1, 1280, False), (3, 40, 2048, False)]:
            seed += 1
            w = O.normal(seed, n * k, 0.05)
            qb = oracle.quantize(O.Q4_K, w, n, k)
            a = O.normal(seed + 50, m * k)
            bv = O.normal(seed + 70, n) if bias else None
            want, _ = oracle.matmul(O.Q4_K, a, qb, n, k, m=m, bias=bv)
            be.set_option("gemv_mma_rows", "2")
            got = run_matmul(be, lp.DType.Q4K, a, qb, m, n, k, bias=bv)
            be.set_option("gemv_mma_rows", "0")
            ref = run_matmul(be, lp.DType.Q4K, a, qb, m, n, k, bias=bv)
            assert max_rel(got, want) <= 2e-5, (m, n, k)
            assert max_rel(got, ref) <= 2e-5, (m, n, k)
    finally:
        be.set_option("gemv_mma_rows", "2")
        be.set_option("gemv_mma_config", "-1")
        be.set_option("gemv_stream", "1")


@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q4K, O.Q4_K), (lp.DType.Q5K, O.Q5_K)])
@pytest.mark.parametrize("config,ctas", [(-1, 0), (0, 1), (0, 2), (1, 0), (2, 0), (2, 1), (3, 0), (3, 2), (4, 0), (4, 3)])
def test_gemv_balanced_stream_kernel(be, oracle, fmt, ofmt, config, ctas):
    """The balanced-stream tensor-core decode kernel (default for Q4_K from 2 rows, Q5_K from 3) in each of its
    tile configurations and CTA counts, against the oracle and against the dp4a kernel: tiles shared by many
    spans (every k-chunk of a tile on another CTA), spans that cross tile boundaries, ragged n, a single row of
    weights, odd super-block counts (a half-empty last k-chunk), a bias, every row count."""
    be.set_option("gemv_stream", "2")
    be.set_option("gemv_stream_config", str(config))
    be.set_option("gemv_stream_ctas", str(ctas))
    try:
        seed = 1100
        for (m, n, k, bias) in [(2, 130, 1024, False), (4, 77, 256, False), (5, 100, 768, True), (8, 513, 4096, False), (7, 33, 14336, True),
                                (8, 16, 512, False), (6, 1, 1280, False), (3, 1030, 2304, False), (4, 300, 28672, False),
                                (8, 2500, 1792, True), (3, 6000, 512, False), (5, 9000, 256, False)]:
            seed += 1
            qb = oracle.quantize(ofmt, O.normal(seed, n * k, 0.05), n, k)
            a = O.normal(seed + 50, m * k)
            bv = O.normal(seed + 70, n) if bias else None
            want, _ = oracle.matmul(ofmt, a, qb, n, k, m=m, bias=bv)
            be.set_option("gemv_mma_rows", "1" if fmt == lp.DType.Q5K else "2")   # Q5_K takes the kernel from one row above the option
            got = run_matmul(be, fmt, a, qb, m, n, k, bias=bv)
            again = run_matmul(be, fmt, a, qb, m, n, k, bias=bv)
            be.set_option("gemv_mma_rows", "0")
            ref = run_matmul(be, fmt, a, qb, m, n, k, bias=bv)
            assert max_rel(got, want) <= 2e-5, (m, n, k, max_rel(got, want))
            assert max_rel(got, ref) <= 2e-5, (m, n, k)
            assert np.array_equal(got, again), (m, n, k)   # the order of the partial sums does not depend on which span finishes last
    finally:
        be.set_option("gemv_mma_rows", "2")
        be.set_option("gemv_stream_config", "-1")
        be.set_option("gemv_stream_ctas", "0")
        be.set_option("gemv_stream", "1")


@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q4K, O.Q4_K), (lp.DType.Q5K, O.Q5_K)])
@pytest.mark.parametrize("config,ctas", [(-1, 0), (1, 0), (3, 1), (4, 0)])
def test_gemv_balanced_stream_kernel_launches_that_run_ahead(be, oracle, fmt, ofmt, config, ctas):
    """Lists whose launches run ahead of their predecessors (operands quantized at the head of the list): every
    segment is staged and a second kernel adds the pieces up. Twenty launches in one list (more than there are
    staging regions, so regions are claimed again while earlier launches are in flight), shapes with many pieces per
    tile, ragged n, one weight row, odd super-block counts, a bias; a dependent launch at the end reads a staged
    result; the list runs three times (a region is claimed again by the same launch)."""
    be.set_option("gemv_stream", "2")
    be.set_option("gemv_stream_config", str(config))
    be.set_option("gemv_stream_ctas", str(ctas))
    be.set_option("gemv_mma_rows", "1" if fmt == lp.DType.Q5K else "2")
    try:
        shapes = [(8, 512, 4096, False), (7, 33, 14336, True), (3, 1030, 2304, False), (4, 300, 28672, False), (8, 2500, 1792, True),
                  (5, 9000, 256, False), (3, 130, 1024, False), (6, 1, 1280, False), (8, 4096, 4096, False), (4, 77, 256, False)]
        bufs, launches, wants = [], [], []
        for rep in range(2):
            for i, (m, n, k, bias) in enumerate(shapes):
                seed = 1400 + 10 * i
                qb = oracle.quantize(ofmt, O.normal(seed, n * k, 0.05), n, k)
                a = O.normal(seed + 1, m * k)
                bv = O.normal(seed + 2, n) if bias else None
                want, _ = oracle.matmul(ofmt, a, qb, n, k, m=m, bias=bv)
                base = len(bufs)
                bufs += [be.upload(a), be.upload(qb), be.alloc(m * n * 4)] + ([be.upload(bv)] if bias else [])
                launches.append(matmul_launch(fmt, m, n, k, inputs=(base, base + 1), output=base + 2, bias_input=base + 3 if bias else None))
                wants.append((base + 2, want))
        # a dependent launch: its activations are the [8, 512] result of the first launch
        qd = oracle.quantize(ofmt, O.normal(1390, 64 * 512, 0.05), 64, 512)
        wd, _ = oracle.matmul(ofmt, wants[0][1], qd, 64, 512, m=8)
        base = len(bufs)
        bufs += [be.upload(qd), be.alloc(8 * 64 * 4)]
        launches.append(matmul_launch(fmt, 8, 64, 512, inputs=(2, base), output=base + 1))
        be.prepare(launches)
        for _ in range(3):
            for (b, _) in wants:
                bufs[b].write(0, np.zeros(bufs[b].nbytes // 4, np.float32))
            be.take_launch_count()
            be.execute(launches, bufs)
            assert be.take_launch_count() > len(launches) + 1   # the launches that ran ahead took two kernels each
            for (b, want) in wants:
                assert max_rel(bufs[b].download().view(np.float32), want) <= 2e-5
            assert max_rel(bufs[base + 1].download().view(np.float32), wd) <= 1e-3   # (int8 rounding of a slightly different input)
    finally:
        be.set_option("gemv_mma_rows", "2")
        be.set_option("gemv_stream_config", "-1")
        be.set_option("gemv_stream_ctas", "0")
        be.set_option("gemv_stream", "1")


def test_gemv_balanced_stream_kernel_many_launches_share_the_workspace(be, oracle):
    """Launch after launch through one workspace: the slab counters return to zero after every launch, in
    lists whose members run ahead of their predecessors and in lists that run one kernel at a time."""
    m, n, k, copies = 8, 700, 4096, 12
    be.set_option("gemv_stream", "2")
    ws = [oracle.quantize(O.Q4_K, O.normal(1300 + c, n * k, 0.05), n, k) for c in range(copies)]
    x = O.normal(1350, m * k)
    wants = [oracle.matmul(O.Q4_K, x, w, n, k, m=m)[0] for w in ws]
    bufs = [be.upload(x)] + [be.upload(w) for w in ws] + [be.alloc(m * n * 4) for _ in range(copies)]
    same_out = [matmul_launch(lp.DType.Q4K, m, n, k, inputs=(0, 1 + c), output=1 + copies + (c % 2)) for c in range(copies)]
    for pdl in ("1", "0"):
        be.set_option("pdl", pdl)
        for rep in range(3):
            be.execute(same_out, bufs)   # launches that overwrite each other's output are never grouped: `copies` kernels
            assert max_rel(bufs[1 + copies + 1].download().view(np.float32), wants[-1]) <= 2e-5
            assert max_rel(bufs[1 + copies].download().view(np.float32), wants[-2]) <= 2e-5
    be.set_option("pdl", "1")
    be.set_option("gemv_stream", "1")


def test_gemv_q6k_tensor_core_decode_kernel(be, oracle):
    """The Q6_K int8 tensor-core decode kernel (2..8 rows, K a multiple of 2048) against the oracle and
    against the dp4a kernel: ragged n, every row count, bias, and the 2-byte block alignment cases
    (every block of a row starts at a different offset from a 16-byte boundary)."""
    try:
        seed = 950
        for (m, n, k, bias) in [(2, 130, 2048, False), (3, 77, 2048, True), (4, 513, 4096, False), (5, 100, 6144, False),
                                (6, 1, 2048, False), (7, 33, 14336, True), (8, 300, 4096, False), (8, 16, 14336, False)]:
            seed += 1
            w = O.normal(seed, n * k, 0.05)
            qb = oracle.quantize(O.Q6_K, w, n, k)
            a = O.normal(seed + 50, m * k)
            bv = O.normal(seed + 70, n) if bias else None
            want, _ = oracle.matmul(O.Q6_K, a, qb, n, k, m=m, bias=bv)
            be.set_option("gemv_mma_rows", "1")   # Q6_K takes the kernel from one row above the option
            got = run_matmul(be, lp.DType.Q6K, a, qb, m, n, k, bias=bv)
            be.set_option("gemv_mma_rows", "0")
            ref = run_matmul(be, lp.DType.Q6K, a, qb, m, n, k, bias=bv)
            assert max_rel(got, want) <= 2e-5, (m, n, k)
            assert max_rel(got, ref) <= 2e-5, (m, n, k)
    finally:
        be.set_option("gemv_mma_rows", "2")


def test_gemv_int8_tensor_core_decode_kernel(be, oracle):
    """The Int8 tensor-core decode kernel (2..8 rows, K a multiple of 512) against the oracle and
    against the dp4a kernel: ragged n, every row count, bias, K with several chunks per warp."""
    try:
        seed = 1000
        for (m, n, k, bias) in [(3, 77, 512, True), (4, 513, 4096, False), (5, 100, 1536, False), (6, 1, 1024, False),
                                (7, 33, 14336, True), (8, 300, 4096, False), (8, 17, 14336, False), (2, 130, 2048, False)]:
            seed += 1
            qb = oracle.quantize(O.INT8, O.normal(seed, n * k, 0.05), n, k)
            a = O.normal(seed + 50, m * k)
            bv = O.normal(seed + 70, n) if bias else None
            want, _ = oracle.matmul(O.INT8, a, qb, n, k, m=m, bias=bv)
            be.set_option("gemv_mma_rows", "2")
            got = run_matmul(be, lp.DType.Int8, a, qb, m, n, k, bias=bv)
            be.set_option("gemv_mma_rows", "0")
            ref = run_matmul(be, lp.DType.Int8, a, qb, m, n, k, bias=bv)
            assert max_rel(got, want) <= 2e-5, (m, n, k)
            assert max_rel(got, ref) <= 2e-5, (m, n, k)
    finally:
        be.set_option("gemv_mma_rows", "2")


def test_gemv_int4_tensor_core_decode_kernel(be, oracle):
    """The Int4 tensor-core decode kernel (2..8 rows, K a multiple of 512) against the oracle and against the plain
    streaming kernel: ragged n, every row count, bias, K with several chunks per warp, weights at both ends of the
    4-bit range (a row of all 0 and all 15 codes)."""
    try:
        seed = 1050
        for (m, n, k, bias) in [(3, 77, 512, True), (4, 513, 4096, False), (5, 100, 1536, False), (6, 1, 1024, False),
                                (7, 33, 14336, True), (8, 300, 4096, False), (8, 17, 14336, False), (2, 130, 2048, False)]:
            seed += 1
            w = O.normal(seed, n * k, 0.05).reshape(n, k).copy()
            w[0, :] = -1.0          # every group of the row: codes 0 (and one 8) ...
            w[0, ::32] = 0.0
            if n > 1:
                w[n - 1, :] = 0.875 * np.abs(w[n - 1, :]).max()   # ... and codes 15
                w[n - 1, ::32] = -np.abs(w[n - 1, :]).max()
            qb = oracle.quantize(O.INT4, w.reshape(-1), n, k)
            a = O.normal(seed + 50, m * k)
            bv = O.normal(seed + 70, n) if bias else None
            want, _ = oracle.matmul(O.INT4, a, qb, n, k, m=m, bias=bv)
            be.set_option("gemv_mma_rows", "2")
            be.take_launch_count()
            got = run_matmul(be, lp.DType.Int4, a, qb, m, n, k, bias=bv)
            be.set_option("gemv_mma_rows", "0")
            ref = run_matmul(be, lp.DType.Int4, a, qb, m, n, k, bias=bv)
            assert max_rel(got, want) <= 2e-5, (m, n, k, max_rel(got, want))
            assert max_rel(got, ref) <= 2e-5, (m, n, k)
    finally:
        be.set_option("gemv_mma_rows", "2")


def test_gemv_q6k_any_block_count(be, oracle):
    """Q6_K rows whose byte length is not a multiple of 16 (K not a multiple of 2048: every stage of
    the bulk-copy ring then starts at a different offset from a 16-byte boundary)."""
    seed = 980
    for (m, n, k) in [(1, 77, 256), (1, 300, 3584), (2, 65, 768), (4, 130, 7168), (8, 33, 3584), (1, 9, 9216), (3, 258, 1280)]:
        seed += 1
        qb = oracle.quantize(O.Q6_K, O.normal(seed, n * k, 0.05), n, k)
        a = O.normal(seed + 50, m * k)
        want, _ = oracle.matmul(O.Q6_K, a, qb, n, k, m=m)
        got = run_matmul(be, lp.DType.Q6K, a, qb, m, n, k)
        assert max_rel(got, want) <= 2e-5, (m, n, k)
        be.set_option("gemv", "generic")
        ref = run_matmul(be, lp.DType.Q6K, a, qb, m, n, k)
        be.set_option("gemv", "fast")
        assert max_rel(got, ref) <= 2e-5, (m, n, k)


def test_gemv_int8_k_not_multiple_of_256(be, oracle):
    for (m, n, k) in [(2, 40, 96), (1, 7, 32), (4, 33, 2080)]:
        w = O.normal(3, n * k, 0.1)
        qb = oracle.quantize(O.INT8, w, n, k)
        a = O.normal(4, m * k)
        want, _ = oracle.matmul(O.INT8, a, qb, n, k, m=m)
        got = run_matmul(be, lp.DType.Int8, a, qb, m, n, k)
        assert max_rel(got, want) <= 2e-5, (m, n, k)


@pytest.mark.parametrize("fmt,name", FMTS)
def test_config1_full_size_matvec(be, oracle, fmt, name):
    # weight [4096, 4096] N(0, 0.02) seed 0, activation [1, 4096] N(0, 1) seed 1
    n = k = 4096
    w = O.normal(0, n * k, 0.02)
    qb = quant.quantize(be, fmt, w, n, k)          # device quantizer ...
    assert np.array_equal(qb, oracle.quantize(int(fmt), w, n, k))  # ... byte-identical to the oracle
    x = O.normal(1, k)
    want, _ = oracle.matmul(int(fmt), x, qb, n, k, m=1)
    got = run_matmul(be, fmt, x, qb, 1, n, k)
    assert max_rel(got, want) <= 1e-3
    assert max_rel(got, want) <= 2e-5


def _as_half(x, kind):
    """f32 -> (bytes to upload, the f32 values those bytes widen to) for f16 / bf16 activations."""
    if kind == lp.DType.F16:
        h = x.astype(np.float16)
        return h.view(np.uint8), h.astype(np.float32)
    bits = x.astype(np.float32).view(np.uint32)
    b16 = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)   # round to nearest even
    return b16.view(np.uint8), (b16.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("kind", [lp.DType.F16, lp.DType.BF16])
@pytest.mark.parametrize("fmt,name", [(lp.DType.Q4K, "q4_k"), (lp.DType.Q5K, "q5_k"), (lp.DType.Q6K, "q6_k"), (lp.DType.Int8, "int8")])
def test_half_precision_activations(be, oracle, fmt, name, kind):
    """a_dtype F16 / BF16 (lapid-cpu's `load_contig`, crates/lapid-cpu/src/matmul/mod.rs:165-286): the rows are widened
    exactly to f32 and then take the f32 path -- the decode kernels (dp4a and tensor-core), the exact f32 GEMM (bit
    for bit) and the tensor-core GEMM, with a padded row stride and a bias."""
    n, k, pad = 200, 1024, 8
    qb = oracle.quantize(int(fmt), O.normal(1400, n * k, 0.05), n, k)
    bias = O.normal(1401, n)
    for m in (1, 4, 8, 40):
        raw, wide = _as_half(O.normal(1410 + m, m * (k + pad)), kind)
        want, path = oracle.matmul(int(fmt), wide, qb, n, k, m=m, a_view=(0, 0, k + pad), bias=bias, fma=True)
        bufs = [be.upload(raw), be.upload(qb), be.alloc(m * n * 4), be.upload(bias)]
        l = matmul_launch(fmt, m, n, k, a_row_stride=k + pad, bias_input=3, a_dtype=kind)
        if m <= 8:
            be.execute([l], bufs)
            assert max_rel(bufs[2].download().view(np.float32), want) <= 2e-5, (name, m)
        else:
            be.set_option("gemm", "f32")
            try:
                be.execute([l], bufs)
            finally:
                be.set_option("gemm", "tc")
            assert np.array_equal(bufs[2].download().view(np.uint32), want.view(np.uint32)), (name, m)
            be.execute([l], bufs)
            got = bufs[2].download().view(np.float32)
            assert rel_l2(got, want) <= 4e-3 and max_rel(got, want) <= 2e-2
    with pytest.raises(lp.LapidError) as e:   # the view is checked in elements of the operand's own type
        be.execute([matmul_launch(fmt, 8, n, k, a_dtype=kind)], [be.alloc(8 * k * 2 - 2), bufs[1], bufs[2]])
    assert e.value.code == "out_of_bounds"


def test_gemv_special_activations(be, oracle):
    n, k = 64, 512
    qb = oracle.quantize(O.Q4_K, O.normal(5, n * k, 0.02), n, k)
    a = O.normal(6, 2 * k).reshape(2, k)
    a[0, 32:64] = 0.0          # an all-zero group: d = 0, id = 0
    a[1, 100] = 1e6            # one huge value flattens its group
    a[1, 256:288] = 0.5        # ties: x*id lands on .5 boundaries
    want, _ = oracle.matmul(O.Q4_K, a, qb, n, k, m=2)
    got = run_matmul(be, lp.DType.Q4K, a, qb, 2, n, k)
    assert max_rel(got, want) <= 2e-5


def test_glue_kernels_rms_norm_and_silu_mul(be):
    """The two steps between projections against f64: rms_norm as lapid-cpu's own test does
    (crates/lapid-cpu/src/tests.rs:246-258, bound 1e-4 there; 1e-5 here), with the residual add, the
    optional weight and the in-place residual stream; silu(gate) * up."""
    rng = np.random.default_rng(7)
    for rows, cols in [(1, 4096), (3, 8192), (8, 16384), (2, 260), (5, 4)]:
        x = rng.standard_normal((rows, cols), dtype=np.float32) * 3
        r = rng.standard_normal((rows, cols), dtype=np.float32)
        w = rng.standard_normal(cols, dtype=np.float32)
        bx, br, bw, bo, bs = be.upload(x), be.upload(r), be.upload(w), be.alloc(rows * cols * 4), be.alloc(rows * cols * 4)
        for res, wt, so in [(None, None, None), (br, None, bs), (br, bw, br), (None, bw, None)]:
            br.write(0, r)
            be.rms_norm(bx, bo, rows, cols, 1e-6, residual=res, weight=wt, sum_out=so)
            be.synchronize()
            h = x.astype(np.float64) + (r if res is not None else 0)
            want = h / np.sqrt((h ** 2).mean(axis=1, keepdims=True) + 1e-6) * (w if wt is not None else 1)
            got = bo.download().view(np.float32).reshape(rows, cols)
            assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
            if so is not None:
                assert np.array_equal(so.download().view(np.float32).reshape(rows, cols), (x + r).astype(np.float32))
    g = rng.standard_normal(4096 * 3, dtype=np.float32) * 4
    u = rng.standard_normal(4096 * 3, dtype=np.float32)
    g[:4] = [0.0, -100.0, 100.0, -1e-20]
    bg, bu = be.upload(g), be.upload(u)
    be.silu_mul(bg, bu, bg, g.size)   # in place over gate
    be.synchronize()
    want = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u
    got = bg.download().view(np.float32)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    with pytest.raises(lp.LapidError) as e:
        be.rms_norm(bg, bu, 1, 4098)
    assert e.value.code == "invalid_launch"


# ------------------------------------------------------------------ exact-f32 GEMM path
@pytest.mark.parametrize("fmt,name", FMTS)
def test_gemm_f32_bit_exact_vs_oracle(be, oracle, fmt, name):
    be.set_option("gemm", "f32")
    try:
        _gemm_f32_cases(be, oracle, fmt, name)
    finally:
        be.set_option("gemm", "tc")


def _gemm_f32_cases(be, oracle, fmt, name):
    seed = 70
    for (batch, m, n, k, pad, epi) in [(1, 9, 45, 256, 0, False), (2, 35, 70, 512, 5, True), (1, 130, 200, 256, 3, True),
                                       (1, 20, 45, 256, 3, False), (1, 33, 300, 1024, 0, False)]:
        seed += 1
        w = rnd(n * k, seed)
        qb = oracle.quantize(int(fmt), w, n, k)
        rs = k + pad
        a = rnd(batch * m * rs, seed + 7)
        bias = rnd(n, seed + 9) if epi else None
        want, path = oracle.matmul(int(fmt), a, qb, n, k, batch=batch, m=m, a_view=(0, m * rs, rs), bias=bias, fma=True)
        assert path == "f32_act"
        got = run_matmul(be, fmt, a, qb, m, n, k, batch=batch, a_row_stride=rs, bias=bias)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (name, batch, m, n, k)


# ------------------------------------------------------------------ tensor-core GEMM path (Q4_K)
def bf16_round(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


@pytest.mark.parametrize("tall", ["-1", "1"])
@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q4K, O.Q4_K), (lp.DType.Q5K, O.Q5_K), (lp.DType.Q6K, O.Q6_K)])
def test_gemm_tensor_core(be, oracle, fmt, ofmt, tall):
    be.set_option("gemm_tall", tall)   # "1": 512 activation rows per CTA wherever a launch has more than 256 rows
    try:
        _gemm_tensor_core_cases(be, oracle, fmt, ofmt, tall == "1")
    finally:
        be.set_option("gemm_tall", "-1")


def _gemm_tensor_core_cases(be, oracle, fmt, ofmt, tall_only):
    """bf16 tensor-core prefill (Q4_K; Q6_K when K is a multiple of 2048): stated bounds vs lapid-cpu's
    f32 path are rel_l2 <= 4e-3 and max_rel <= 2e-2 (both operands rounded to bf16, 2^-9 each; the
    reference allows 2e-3 for its f16 tensor-core kernel, crates/lapid-cuda/src/kquant_tests.rs:191-192).
    Against the same product computed from bf16-rounded operands the result must agree to
    summation-order noise."""
    seed = 90
    q4 = [(1, 64, 256, 512, 0, False), (1, 20, 45, 256, 3, False), (1, 130, 70, 512, 0, True),
          (1, 33, 300, 1024, 0, False), (2, 137, 300, 2048, 8, True), (1, 9, 128, 256, 0, False),
          (1, 512, 1024, 4096, 0, False), (1, 300, 130, 14336, 0, False), (1, 700, 200, 512, 0, True)]
    q6 = [(1, 64, 256, 2048, 0, False), (1, 20, 45, 2048, 3, False), (1, 130, 70, 4096, 0, True),
          (2, 137, 300, 2048, 8, True), (1, 9, 128, 2048, 0, False), (1, 512, 1024, 4096, 0, False),
          (1, 300, 130, 14336, 0, False), (1, 257, 129, 6144, 0, False),
          # K not a multiple of 2048: rows are not 16-byte multiples, the kernel copies them one by one
          (1, 64, 256, 512, 0, False), (1, 33, 300, 1024, 0, True), (1, 140, 131, 3584, 0, False), (1, 9, 5, 256, 0, False)]
    for (batch, m, n, k, pad, epi) in (q4 if fmt == lp.DType.Q4K else q6):
        seed += 1
        if tall_only and batch * m <= 256:
            continue
        big = n * k > 200000
        w = O.normal(seed, n * k, 0.02) if big else rnd(n * k, seed)
        qb = oracle.quantize(ofmt, w, n, k)
        rs = k + pad
        a = O.normal(seed + 7, batch * m * rs) if big else rnd(batch * m * rs, seed + 7)
        bias = rnd(n, seed + 9) if epi else None
        be.take_launch_count()
        got = run_matmul(be, fmt, a, qb, m, n, k, batch=batch, a_row_stride=rs, bias=bias).reshape(batch * m, n)
        assert be.take_launch_count() in (2, 3)   # bf16 copy of the activations + the tensor-core kernel (+ the split-K sum)
        deq = oracle.dequantize(ofmt, qb, n, k)
        av = a.reshape(batch * m, rs)[:, :k]
        b64 = bias.astype(np.float64) if epi else 0.0
        exact = av.astype(np.float64) @ deq.astype(np.float64).T + b64
        assert rel_l2(got, exact) <= 4e-3, (m, n, k, rel_l2(got, exact))
        assert max_rel(got, exact) <= 2e-2, (m, n, k, max_rel(got, exact))
        rounded = bf16_round(av).astype(np.float64) @ bf16_round(deq).astype(np.float64).T + b64
        assert rel_l2(got, rounded) <= 2e-5, (m, n, k, rel_l2(got, rounded))
    if True:  # the exact path still answers for the same launch when asked
        be.set_option("gemm", "f32")
        got = run_matmul(be, fmt, a, qb, m, n, k, batch=batch, a_row_stride=rs)
        be.set_option("gemm", "tc")
        want, _ = oracle.matmul(ofmt, a, qb, n, k, batch=batch, m=m, a_view=(0, m * rs, rs), fma=True)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_gemm_tensor_core_cta_pairs(be, oracle):
    """Q4_K prefill with two CTAs per tensor-core unit (`cta_group::2`): the same bounds as the
    single-CTA kernel and, since the products and the f32 accumulation order per output are the same,
    the same bits."""
    seed = 400
    for (m, n, k, epi) in [(512, 1024, 4096, False), (300, 1000, 1024, True), (260, 700, 512, False), (1000, 512, 2048, False)]:
        seed += 1
        qb = oracle.quantize(O.Q4_K, O.normal(seed, n * k, 0.02), n, k)
        a = O.normal(seed + 7, m * k)
        bias = rnd(n, seed + 9) if epi else None
        be.set_option("gemm_splitk", "0")   # same k order in both runs
        be.set_option("gemm_pair", "1")
        try:
            got = run_matmul(be, lp.DType.Q4K, a, qb, m, n, k, bias=bias).reshape(m, n)
            be.set_option("gemm_pair", "0")
            ref = run_matmul(be, lp.DType.Q4K, a, qb, m, n, k, bias=bias).reshape(m, n)
        finally:
            be.set_option("gemm_pair", "0")
            be.set_option("gemm_splitk", "-1")
        deq = oracle.dequantize(O.Q4_K, qb, n, k)
        rounded = bf16_round(a.reshape(m, k)).astype(np.float64) @ bf16_round(deq).astype(np.float64).T + (bias.astype(np.float64) if epi else 0.0)
        assert rel_l2(got, rounded) <= 2e-5, (m, n, k, rel_l2(got, rounded))
        assert np.array_equal(got, ref), (m, n, k)


def test_gemm_tensor_core_split_k(be, oracle):
    """Few output tiles (small n): K is split over several CTAs per tile and the partial tiles are
    summed in a fixed order by a second kernel. Same bounds; forced split counts including ones that
    do not divide the number of super-blocks; strided output and bias go through the sum kernel."""
    seed = 500
    for fmt, ofmt in ((lp.DType.Q4K, O.Q4_K), (lp.DType.Q5K, O.Q5_K), (lp.DType.Q6K, O.Q6_K)):
        for (m, n, k, ways, epi) in [(64, 256, 4096, -1, False), (300, 130, 14336, -1, True), (40, 100, 1792, 3, False),
                                     (512, 1024, 4096, 5, True), (20, 45, 1024, 16, False)]:
            seed += 1
            qb = oracle.quantize(ofmt, O.normal(seed, n * k, 0.02), n, k)
            a = O.normal(seed + 7, m * k)
            bias = rnd(n, seed + 9) if epi else None
            be.set_option("gemm_splitk", str(ways))
            try:
                be.take_launch_count()
                got = run_matmul(be, fmt, a, qb, m, n, k, bias=bias).reshape(m, n)
                launched = be.take_launch_count()
            finally:
                be.set_option("gemm_splitk", "-1")
            assert launched == 3, (m, n, k, ways)
            deq = oracle.dequantize(ofmt, qb, n, k)
            rounded = bf16_round(a.reshape(m, k)).astype(np.float64) @ bf16_round(deq).astype(np.float64).T + (bias.astype(np.float64) if epi else 0.0)
            assert rel_l2(got, rounded) <= 2e-5, (m, n, k, ways, rel_l2(got, rounded))


def test_gemm_tensor_core_strided_output(be, oracle):
    k, n, off, batch, m = 256, 40, 7, 3, 30
    a = rnd(batch * m * k, 100)
    qb = oracle.quantize(O.Q4_K, rnd(n * k, 101), n, k)
    total = off + m * batch * n + 5
    got = run_matmul(be, lp.DType.Q4K, a, qb, m, n, k, batch=batch, out=np.full(total, -1.0, np.float32),
                     out_view=MatView(off, n, batch * n))
    want = np.full(total, -1.0, np.float32)
    oracle.matmul(O.Q4_K, a, qb, n, k, batch=batch, m=m, out=want, out_view=(off, n, batch * n))
    touched = want != -1.0
    assert (got[~touched] == -1.0).all()
    assert rel_l2(got[touched], want[touched]) <= 4e-3


# ------------------------------------------------------------------ views, epilogue, validation
def test_strided_output_view_and_bias(be, oracle):
    k, n, off, batch = 64, 40, 7, 3
    for m in (2, 30):
        a = rnd(batch * m * k, 100 + m)
        qb = oracle.quantize(O.INT8, rnd(n * k, 101 + m), n, k)
        total = off + m * batch * n + 5
        want = np.full(total, -1.0, np.float32)
        oracle.matmul(O.INT8, a, qb, n, k, batch=batch, m=m, out=want, out_view=(off, n, batch * n))
        got = run_matmul(be, lp.DType.Int8, a, qb, m, n, k, batch=batch, out=np.full(total, -1.0, np.float32),
                         out_view=MatView(off, n, batch * n))
        touched = want != -1.0
        assert (got[~touched] == -1.0).all()  # nothing outside the view is written
        assert max_rel(got[touched], want[touched]) <= (2e-5 if batch * m <= 8 else 0.0)
    # bias epilogue on the decode path
    m, n, k = 4, 50, 512
    qb = oracle.quantize(O.Q6_K, O.normal(9, n * k, 0.02), n, k)
    a, bias = O.normal(10, m * k), O.normal(11, n)
    want, _ = oracle.matmul(O.Q6_K, a, qb, n, k, m=m, bias=bias)
    assert max_rel(run_matmul(be, lp.DType.Q6K, a, qb, m, n, k, bias=bias), want) <= 2e-5


@pytest.mark.parametrize("fmt,name", FMTS + [(lp.DType.F32, "f32")])
def test_gather_rows_from_a_quantized_table(be, oracle, fmt, name):
    """Kernel::Gather (the embedding lookup): out[i, :] = dequant(table[ids[i], :]), bit-identical to the
    oracle's dequantization of the same rows (the reference's own check: crates/lapid-cpu/src/tests.rs,
    gather against dequantized rows); repeated and unordered indices; an index outside the table fails
    with index_out_of_range and leaves the device usable."""
    from lapid_b200.backend import gather_launch
    rows, cols, count = 300, 1024, 37
    w = O.normal(31, rows * cols, 0.05)
    if fmt == lp.DType.F32:
        table, deq = w.view(np.uint8), w.reshape(rows, cols)
    else:
        table = oracle.quantize(int(fmt), w, rows, cols)
        deq = oracle.dequantize(int(fmt), table, rows, cols).reshape(rows, cols)
    ids = np.array([0, 299, 5, 5, 17] + list(np.random.default_rng(3).integers(0, rows, count - 5)), np.int32)
    bufs = [be.upload(table), be.upload(ids.view(np.uint8)), be.alloc(count * cols * 4)]
    l = gather_launch(fmt, rows, cols, count)
    be.prepare([l])
    be.execute([l], bufs)
    got = bufs[2].download().view(np.float32).reshape(count, cols)
    assert np.array_equal(got.view(np.uint32), deq[ids].astype(np.float32).view(np.uint32))
    # a gathered row feeds a projection in the same launch list (embedding -> first matmul)
    if fmt != lp.DType.F32:
        n = 64
        qb = oracle.quantize(O.Q4_K, O.normal(32, n * cols, 0.05), n, cols)
        bufs2 = bufs + [be.upload(qb), be.alloc(2 * n * 4)]
        l2 = matmul_launch(lp.DType.Q4K, 2, n, cols, inputs=(2, 3), output=4)
        be.execute([gather_launch(fmt, rows, cols, 2), l2], bufs2)
        want, _ = oracle.matmul(O.Q4_K, deq[ids[:2]].reshape(-1), qb, n, cols, m=2)
        assert max_rel(bufs2[4].download().view(np.float32), want) <= 2e-5
    bad = ids.copy()
    bad[7] = rows
    bufs[1].write(0, bad.view(np.uint8))
    with pytest.raises(lp.LapidError) as e:
        be.execute([l], bufs)
    assert e.value.code == "index_out_of_range"
    bad[7] = -1
    bufs[1].write(0, bad.view(np.uint8))
    with pytest.raises(lp.LapidError) as e:
        be.execute([l], bufs)
    assert e.value.code == "index_out_of_range"
    bufs[1].write(0, ids.view(np.uint8))
    be.execute([l], bufs)   # still usable
    assert np.array_equal(bufs[2].download().view(np.float32).reshape(count, cols), got)


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_glue_kernels_quantize_for_the_next_projection(be, oracle, fmt, name, m):
    """rms_norm / silu_mul with a quantized copy of their result: a launch that reads that copy (a_dtype
    ACT_Q8, no pre-pass kernel) gives bit for bit what the same launch gives from the f32 result, in each
    of the three operand layouts; the f32 result itself is unchanged."""
    n, k = 96, 2048
    be.set_option("early_acts", "0")   # keep the plain launch on the kernel act_layout describes (bit-equality below)
    qb = oracle.quantize(int(fmt), O.normal(5, n * k, 0.05), n, k)
    x = O.normal(6, m * k, 1.0)
    x[3] = 0.0
    res = O.normal(7, m * k, 0.5)
    wgt = (1.0 + 0.1 * O.normal(8, k, 1.0)).astype(np.float32)
    plain = matmul_launch(fmt, m, n, k, inputs=(0, 1), output=2)
    fused = matmul_launch(fmt, m, n, k, inputs=(3, 1), output=2, a_quantized=True)
    layout, nbytes = be.act_layout(plain)
    assert be.act_layout(fused) == (layout, nbytes)
    bx, bres, bw = be.upload(x), be.upload(res), be.upload(wgt)
    for producer in ("rms_norm", "silu_mul"):
        normed, normed2, qact = be.alloc(m * k * 4), be.alloc(m * k * 4), be.alloc(nbytes)
        if producer == "rms_norm":
            be.rms_norm(bx, normed, m, k, residual=bres, weight=bw)
            be.rms_norm(bx, normed2, m, k, residual=bres, weight=bw, qact=qact, layout=layout)
        else:
            be.silu_mul(bx, bres, normed, m * k, rows=m)
            be.silu_mul(bx, bres, normed2, m * k, rows=m, qact=qact, layout=layout)
        a = normed.download()
        assert np.array_equal(a, normed2.download())
        out = be.alloc(m * n * 4)
        be.take_launch_count()
        be.execute([plain], [normed, be.upload(qb), out])
        want = out.download().copy()
        assert be.take_launch_count() == 2
        out.write(0, np.zeros(m * n * 4, np.uint8))
        be.execute([fused], [normed, be.upload(qb), out, qact])
        assert be.take_launch_count() == 1          # no pre-pass
        assert np.array_equal(out.download(), want)
    with pytest.raises(lp.LapidError):              # a prefill-sized launch takes no quantized operand
        be.prepare([matmul_launch(fmt, 16, n, k, a_quantized=True)])
    with pytest.raises(lp.LapidError) as e:
        be.execute([fused], [normed, be.upload(qb), out, be.alloc(64)])
    assert e.value.code == "out_of_bounds"
    be.set_option("early_acts", "1")


@pytest.mark.parametrize("fmt,name", [(lp.DType.Q4K, "q4_k"), (lp.DType.Q6K, "q6_k"), (lp.DType.Int8, "int8")])
@pytest.mark.parametrize("m", [1, 2, 8])
def test_launches_that_run_ahead_of_their_predecessor(be, oracle, fmt, name, m):
    """A list of decode launches that share activations quantized at its head: from the second launch on the
    kernels read and compute before the kernel in front of them has finished and park their results
    (GemvArgs::early). Same values as with the mode switched off, whatever the launches write to: distinct
    buffers, the same buffer again and again, or a buffer a later launch of the list reads."""
    n, k, copies = 520, 2048, 9
    ws = [oracle.quantize(int(fmt), O.normal(400 + c, n * k, 0.05), n, k) for c in range(copies)]
    x = O.normal(77, m * k, 1.0)
    wants = [oracle.matmul(int(fmt), x, w, n, k, m=m)[0] for w in ws]
    bufs = [be.upload(x)] + [be.upload(w) for w in ws] + [be.alloc(m * n * 4) for _ in range(copies)]
    distinct = [matmul_launch(fmt, m, n, k, inputs=(0, 1 + c), output=1 + copies + c) for c in range(copies)]
    same = [matmul_launch(fmt, m, n, k, inputs=(0, 1 + c), output=1 + copies) for c in range(copies)]
    for early in ("1", "0"):
        be.set_option("early_acts", early)
        be.execute(distinct, bufs)                                      # (independent launches also go out in groups)
        for c in range(copies):
            assert max_rel(bufs[1 + copies + c].download().view(np.float32), wants[c]) <= 2e-5
        be.take_launch_count()
        be.execute(same, bufs)                                          # write-after-write in stream order
        assert be.take_launch_count() == 1 + copies                     # one pre-pass at the head, then one kernel each
        assert max_rel(bufs[1 + copies].download().view(np.float32), wants[-1]) <= 2e-5
    be.set_option("early_acts", "1")
    # the fused `acc + bias[n]` epilogue is applied when the parked results are stored
    bias = O.normal(78, n, 1.0)
    bb = bufs + [be.upload(bias)]
    biased = [matmul_launch(fmt, m, n, k, inputs=(0, 1 + c), output=1 + copies + c, bias_input=len(bb) - 1) for c in range(copies)]
    be.execute(biased, bb)
    for c in range(copies):
        got = bb[1 + copies + c].download().view(np.float32).reshape(m, n)
        assert max_rel(got, wants[c].reshape(m, n) + bias[None, :]) <= 2e-5
    if m == 1:   # a launch that reads what an early launch wrote (k == n here would be needed: use a square pair)
        n2 = k
        w2 = oracle.quantize(int(fmt), O.normal(450, n2 * k, 0.05), n2, k)
        w3 = oracle.quantize(int(fmt), O.normal(451, n * n2, 0.05), n, n2)
        y2 = oracle.matmul(int(fmt), x, w2, n2, k, m=1)[0]
        y3 = oracle.matmul(int(fmt), y2, w3, n, n2, m=1)[0]
        b2 = [be.upload(x), be.upload(ws[0]), be.alloc(n * 4), be.upload(w2), be.alloc(n2 * 4), be.upload(w3), be.alloc(n * 4)]
        chain = [matmul_launch(fmt, 1, n, k, inputs=(0, 1), output=2), matmul_launch(fmt, 1, n2, k, inputs=(0, 3), output=4),
                 matmul_launch(fmt, 1, n, n2, inputs=(4, 5), output=6)]
        for _ in range(3):
            be.execute(chain, b2)
            assert max_rel(b2[6].download().view(np.float32), y3) <= 1e-4


def _expert_stack(oracle, fmt, e, n, k, seed):
    one = oracle.layout(int(fmt), n, k).total
    stack = np.zeros(e * one, np.uint8)
    for x in range(e):
        q = oracle.quantize(int(fmt), O.normal(seed + x, n * k, 0.05), n, k)
        stack[x * one:x * one + q.size] = q
    return stack


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("t,r,e,n,k", [(1, 2, 5, 24, 512), (1, 4, 8, 200, 1024), (3, 2, 4, 64, 256), (8, 8, 16, 96, 2048),
                                       (2, 3, 6, 40, 4096 + 512)])
def test_matmul_id_decode(be, oracle, fmt, name, t, r, e, n, k):
    """Kernel::MatMulId at decode sizes (t <= 8): every (token, slot) pair is the int8-activation GEMV of the
    token's row against the matrix of its expert -- what lapid-cpu computes per used expert
    (crates/lapid-cpu/src/moe.rs:80-118; its test crates/lapid-cpu/src/tests.rs:350-383 uses the same id pattern)."""
    from lapid_b200.backend import matmul_id_launch
    stack = _expert_stack(oracle, fmt, e, n, k, 50)
    x = O.normal(70, t * k, 1.0)
    ids = np.array([(i * 7 + i // r) % e for i in range(t * r)], np.int32)
    want = oracle.matmul_id(int(fmt), x, stack, ids, t, r, e, n, k)
    bufs = [be.upload(x), be.upload(stack), be.upload(ids.view(np.uint8)), be.alloc(t * r * n * 4)]
    l = matmul_id_launch(fmt, t, r, e, n, k)
    be.prepare([l])
    be.execute([l], bufs)
    got = bufs[3].download().view(np.float32).reshape(t, r, n)
    assert max_rel(got, want) <= 2e-5
    for gemv in ("generic", "fast"):   # the any-shape kernel gives the same
        be.set_option("gemv", gemv)
        be.execute([l], bufs)
        assert max_rel(bufs[3].download().view(np.float32).reshape(t, r, n), want) <= 2e-5
    bad = ids.copy()
    bad[-1] = e
    bufs[2].write(0, bad.view(np.uint8))
    with pytest.raises(lp.LapidError) as err:
        be.execute([l], bufs)
    assert err.value.code == "index_out_of_range"
    bufs[2].write(0, ids.view(np.uint8))
    be.execute([l], bufs)
    assert max_rel(bufs[3].download().view(np.float32).reshape(t, r, n), want) <= 2e-5


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("t,r,e,n,k", [(40, 3, 5, 24, 512), (70, 2, 4, 200, 256), (300, 4, 8, 136, 1024), (9, 1, 3, 64, 256)])
def test_matmul_id_prefill_exact(be, oracle, fmt, name, t, r, e, n, k):
    """t > 8: float activations for every expert (moe.rs:107-109). With gemm=f32 the grouped exact kernel
    is bit-identical to the oracle's per-expert f32 matmul, whatever tile a pair lands in."""
    from lapid_b200.backend import matmul_id_launch
    stack = _expert_stack(oracle, fmt, e, n, k, 90)
    x = O.normal(71, t * k, 1.0)
    ids = np.array([(i * 7 + i // r) % e for i in range(t * r)], np.int32)
    if e > 4:
        ids[ids == 1] = 2        # an expert nobody uses
    want = oracle.matmul_id(int(fmt), x, stack, ids, t, r, e, n, k)
    bufs = [be.upload(x), be.upload(stack), be.upload(ids.view(np.uint8)), be.alloc(t * r * n * 4)]
    l = matmul_id_launch(fmt, t, r, e, n, k)
    be.set_option("gemm", "f32")
    try:
        for _ in range(2):
            be.execute([l], bufs)
            got = bufs[3].download().view(np.float32).reshape(t, r, n)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        bad = ids.copy()
        bad[3] = -2
        bufs[2].write(0, bad.view(np.uint8))
        with pytest.raises(lp.LapidError) as err:
            be.execute([l], bufs)
        assert err.value.code == "index_out_of_range"
    finally:
        be.set_option("gemm", "tc")


@pytest.mark.parametrize("fmt,name", [(lp.DType.Q4K, "q4_k"), (lp.DType.Q5K, "q5_k"), (lp.DType.Q6K, "q6_k")])
@pytest.mark.parametrize("t,r,e,n,k", [(64, 2, 4, 256, 2048), (200, 4, 8, 384, 4096), (1024, 2, 4, 128, 2048)])
def test_matmul_id_prefill_tensor_core(be, oracle, fmt, name, t, r, e, n, k):
    """The same launch on the tensor cores (bf16 operands): the bounds of the dense prefill kernel
    against the exact result."""
    from lapid_b200.backend import matmul_id_launch
    stack = _expert_stack(oracle, fmt, e, n, k, 110)
    x = O.normal(72, t * k, 1.0)
    rng = np.random.default_rng(5)
    ids = np.stack([rng.permutation(e)[:r] for _ in range(t)]).astype(np.int32).reshape(-1)
    want = oracle.matmul_id(int(fmt), x, stack, ids, t, r, e, n, k)
    bufs = [be.upload(x), be.upload(stack), be.upload(ids.view(np.uint8)), be.alloc(t * r * n * 4)]
    l = matmul_id_launch(fmt, t, r, e, n, k)
    be.take_launch_count()
    be.execute([l], bufs)
    assert be.take_launch_count() == 3        # route, gather to bf16, grouped tensor-core GEMM
    got = bufs[3].download().view(np.float32).reshape(t, r, n)
    assert rel_l2(got, want) <= 4e-3 and max_rel(got, want) <= 2e-2


def test_zero_sized_launches(be, oracle):
    qb = oracle.quantize(O.Q4_K, O.normal(1, 4 * 256, 0.02), 4, 256)
    out = run_matmul(be, lp.DType.Q4K, np.zeros(1, np.float32), qb[:256], 2, 4, 0, out=np.full(8, 9.0, np.float32))
    assert not out.any()  # k == 0 writes zeros
    out = run_matmul(be, lp.DType.Q4K, np.zeros(1, np.float32), qb, 0, 4, 256, out=np.full(8, 9.0, np.float32))
    assert (out == 9.0).all()  # m == 0 is a no-op


def test_launch_validation_codes(be, oracle):
    n, k, m = 4, 256, 2
    qb = oracle.quantize(O.Q4_K, rnd(n * k, 1), n, k)
    a = rnd(m * k, 2)
    bufs = [be.upload(a), be.upload(qb), be.alloc(m * n * 4)]

    def code(l, bs=bufs):
        with pytest.raises(lp.LapidError) as e:
            be.execute([l], bs)
        return e.value.code

    ok = matmul_launch(lp.DType.Q4K, m, n, k)
    be.execute([ok], bufs)
    import dataclasses as dc
    assert code(dc.replace(ok, dims=dc.replace(ok.dims, n=5))) == "out_of_bounds"       # weights too small for [5, k]
    assert code(dc.replace(ok, dims=dc.replace(ok.dims, b=MatView(0, 0, 512)))) == "shape_mismatch"
    assert code(dc.replace(ok, dims=dc.replace(ok.dims, b=MatView(1, 0, k)))) == "invalid_launch"
    assert code(dc.replace(ok, spec=dc.replace(ok.spec, b_transposed=False))) == "invalid_launch"
    assert code(dc.replace(ok, dims=dc.replace(ok.dims, k=128, b=MatView(0, 0, 128)))) == "invalid_launch"  # k % 256
    assert code(dc.replace(ok, dims=dc.replace(ok.dims, m=3, out=MatView.contiguous(3, n)))) == "out_of_bounds"
    assert code(dc.replace(ok, dims=dc.replace(ok.dims, a=MatView(1, m * k, k)))) == "out_of_bounds"
    assert code(dc.replace(ok, spec=dc.replace(ok.spec, b_dtype=lp.DType.F16))) == "unsupported_dtype"
    assert code(dc.replace(ok, inputs=(0, 1, 1))) == "invalid_launch"       # 3 inputs without an epilogue
    assert code(dc.replace(ok, inputs=(0, 7))) == "invalid_launch"          # BufId out of range
    assert code(dc.replace(ok, inputs=(2, 1))) == "buffer_aliasing"         # input is the output
    assert code(dc.replace(ok, kind=9)) == "unsupported"
    # the device stays usable after every rejected launch
    be.execute([ok], bufs)
    want, _ = oracle.matmul(O.Q4_K, a, qb, n, k, m=m)
    assert max_rel(bufs[2].download().view(np.float32), want) <= 2e-5


def test_launch_sequences_see_earlier_writes(be, oracle):
    # launch 2 consumes launch 1's output (o_proj after q_proj in a layer): [1,512] -> [1,256] -> [1,64]
    w1 = oracle.quantize(O.Q4_K, O.normal(1, 256 * 512, 0.05), 256, 512)
    w2 = oracle.quantize(O.Q6_K, O.normal(2, 64 * 256, 0.05), 64, 256)
    x = O.normal(3, 512)
    bufs = [be.upload(x), be.upload(w1), be.alloc(256 * 4), be.upload(w2), be.alloc(64 * 4)]
    l1 = matmul_launch(lp.DType.Q4K, 1, 256, 512, inputs=(0, 1), output=2)
    l2 = matmul_launch(lp.DType.Q6K, 1, 64, 256, inputs=(2, 3), output=4)
    for _ in range(3):
        be.execute([l1, l2], bufs)
    h, _ = oracle.matmul(O.Q4_K, x, w1, 256, 512, m=1)
    want, _ = oracle.matmul(O.Q6_K, bufs[2].download().view(np.float32), w2, 64, 256, m=1)
    assert max_rel(bufs[2].download().view(np.float32), h) <= 2e-5
    assert max_rel(bufs[4].download().view(np.float32), want) <= 2e-5


def test_write_then_execute_ordering_and_wrap(be, oracle):
    import torch
    n, k = 128, 512
    qb = oracle.quantize(O.Q4_K, O.normal(1, n * k, 0.02), n, k)
    wt = torch.from_numpy(qb).cuda()
    at = torch.zeros(k, device="cuda")
    ot = torch.zeros(n, device="cuda")
    torch.cuda.synchronize()
    bufs = [be.wrap_tensor(at), be.wrap_tensor(wt), be.wrap_tensor(ot)]
    l = matmul_launch(lp.DType.Q4K, 1, n, k)
    for seed in (5, 6):
        x = O.normal(seed, k)
        bufs[0].write(0, x)
        be.execute([l], bufs)
        want, _ = oracle.matmul(O.Q4_K, x, qb, n, k, m=1)
        assert max_rel(ot.cpu().numpy(), want) <= 2e-5


def test_activation_sharing_and_hoisting(be, oracle):
    """Launches that read the same input share one activation pre-pass, pre-passes of inputs that
    the list does not write are hoisted to its head, and a write to the input in between is seen."""
    k = 256
    ws = [oracle.quantize(O.Q4_K, O.normal(30 + i, k * k, 0.08), k, k) for i in range(4)]
    x = O.normal(40, k)
    # buffers: 0 x, 1..4 weights, 5..7 outputs of q/k/v, 8 out of launch 5
    bufs = [be.upload(x)] + [be.upload(w) for w in ws] + [be.alloc(k * 4) for _ in range(4)]
    ls = [matmul_launch(lp.DType.Q4K, 1, k, k, inputs=(0, 1), output=5),
          matmul_launch(lp.DType.Q4K, 1, k, k, inputs=(0, 2), output=6),
          matmul_launch(lp.DType.Q4K, 1, k, k, inputs=(0, 3), output=7),
          matmul_launch(lp.DType.Q4K, 1, k, k, inputs=(5, 4), output=0),   # overwrites x with W4 . out_q
          matmul_launch(lp.DType.Q4K, 1, k, k, inputs=(0, 1), output=8)]   # must see the new x
    be.prepare(ls)
    be.set_option("gemv_group", "0")
    for opt in ("1", "0"):
        be.set_option("act_reuse", opt)
        bufs[0].write(0, x)
        be.take_launch_count()
        be.execute(ls, bufs)
        launched = be.take_launch_count()
        q1, _ = oracle.matmul(O.Q4_K, x, ws[0], k, k, m=1)
        q2, _ = oracle.matmul(O.Q4_K, x, ws[1], k, k, m=1)
        q3, _ = oracle.matmul(O.Q4_K, x, ws[2], k, k, m=1)
        got1 = bufs[5].download().view(np.float32)
        x2, _ = oracle.matmul(O.Q4_K, got1, ws[3], k, k, m=1)
        got_x2 = bufs[0].download().view(np.float32)
        q5, _ = oracle.matmul(O.Q4_K, got_x2, ws[0], k, k, m=1)
        for got, want in ((got1, q1), (bufs[6].download().view(np.float32), q2), (bufs[7].download().view(np.float32), q3),
                          (got_x2, x2), (bufs[8].download().view(np.float32), q5)):
            assert max_rel(got, want) <= 2e-5
        # 5 GEMVs; pre-passes: one shared by q/k/v (hoisted), one for out_q, one for the rewritten x
        assert launched == (8 if opt == "1" else 10)
    be.set_option("act_reuse", "1")
    be.set_option("gemv_group", "1")


@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q4K, O.Q4_K), (lp.DType.Q6K, O.Q6_K)])
@pytest.mark.parametrize("m", [1, 3, 8])
def test_grouped_decode_launches(be, oracle, fmt, ofmt, m):
    """Consecutive independent decode launches with the same format, rows and k go out as one
    kernel; the results are those of the launches run one by one, bit for bit, and a launch that
    reads or overwrites what a pending one writes is never merged with it."""
    k = 2048
    ns = [512, 136, 77, 1024, 256]
    ws = [oracle.quantize(ofmt, O.normal(50 + i, n * k, 0.05), n, k) for i, n in enumerate(ns)]
    wd = oracle.quantize(ofmt, O.normal(60, k * k, 0.05), k, k)   # consumes a [m, k] output
    x = O.normal(70, m * k)
    y = O.normal(71, m * k)
    bias = O.normal(72, ns[1])
    # 0 x, 1 y, 2..6 weights, 7 wd, 8 bias, 9 packed outputs, 10 out of the dependent launch, 11 [m,k] scratch
    total = sum(m * n for n in ns)
    bufs = [be.upload(x), be.upload(y)] + [be.upload(w) for w in ws] + [be.upload(wd), be.upload(bias),
            be.alloc(total * 4), be.alloc(m * k * 4), be.alloc(m * k * 4)]
    offs = np.cumsum([0] + [m * n for n in ns])
    ls = []
    for i, n in enumerate(ns):
        ls.append(matmul_launch(fmt, m, n, k, inputs=(0 if i != 3 else 1, 2 + i), output=9, out=MatView(int(offs[i]), m * n, n),
                                bias_input=8 if i == 1 else None))
    ls.append(matmul_launch(fmt, m, k, k, inputs=(0, 7), output=11))    # independent: same group or next
    ls.append(matmul_launch(fmt, m, k, k, inputs=(11, 7), output=10))   # reads the launch before it: new group
    ls.append(matmul_launch(fmt, m, k, k, inputs=(10, 7), output=11))   # overwrites its own producer's input
    be.prepare(ls)
    res = {}
    for opt in ("0", "1"):
        be.set_option("gemv_group", opt)
        for b in (9, 10, 11):
            bufs[b].write(0, np.zeros(bufs[b].nbytes // 4, np.float32))
        be.take_launch_count()
        be.execute(ls, bufs)
        res[opt] = (be.take_launch_count(), [bufs[b].download().view(np.float32).copy() for b in (9, 10, 11)])
    be.set_option("gemv_group", "1")
    for a, b in zip(res["0"][1], res["1"][1]):
        if fmt == lp.DType.Q5K and m >= 3:
            # the balanced-stream kernel cuts the k-chunks of a row tile where the launch's equal shares end, so
            # the order of its f32 partial sums depends on what shares the launch
            assert max_rel(a, b) <= 2e-6
        else:
            assert np.array_equal(a, b)
    # the tensor-core kernels share a launch; dp4a launches that may run ahead of their predecessor (one row, operands
    # quantized at the head of the list) overlap on their own and are left as they are
    assert res["1"][0] < res["0"][0] if m >= 3 else res["1"][0] <= res["0"][0]
    # and against the oracle
    got = res["1"][1][0]
    for i, n in enumerate(ns):
        want, _ = oracle.matmul(ofmt, x if i != 3 else y, ws[i], n, k, m=m, bias=bias if i == 1 else None)
        assert max_rel(got[offs[i]:offs[i + 1]], want) <= 2e-5
    h1, _ = oracle.matmul(ofmt, x, wd, k, k, m=m)
    h2, _ = oracle.matmul(ofmt, h1, wd, k, k, m=m)
    h3, _ = oracle.matmul(ofmt, res["1"][1][1], wd, k, k, m=m)
    assert max_rel(res["1"][1][1], h2) <= 1e-3   # second hop: int8 rounding of a slightly different input
    assert max_rel(res["1"][1][2], h3) <= 2e-5


def test_a_device_side_wait_that_runs_out_is_reported(be, oracle):
    """Failure detection without a GPU fault: a tensor-parallel all-reduce whose second "rank" never writes (its
    buffer is a local one nobody touches) polls with a short limit (option tp_spin_limit), gives up, returns, and
    records that in the host-visible status word. The next waiting call fails with "backend" and clears the word;
    the device, the comm buffers and later launches work as before."""
    import ctypes as C
    from lapid_b200 import _lib
    lib = _lib.lib()
    world, max_elems, count = 2, 1024, 256
    nbytes = int(lib.lapid_b200_tp_comm_bytes(world, max_elems))
    mine, silent = be.upload(np.zeros(nbytes, np.uint8)), be.upload(np.zeros(nbytes, np.uint8))
    ptrs = (C.c_void_p * world)(mine.device_ptr, silent.device_ptr)
    comm = C.c_void_p()
    _lib.check(lib.lapid_b200_tp_comm_create(be._h, 0, world, ptrs, max_elems, C.byref(comm)))
    data = be.upload(np.ones(count, np.float32))
    be.set_option("tp_spin_limit", "2000")
    try:
        _lib.check(lib.lapid_b200_tp_all_reduce(comm, data._h, 0, count))     # queued; the kernel gives up after 2000 polls
        with pytest.raises(lp.LapidError) as e:
            be.synchronize()
        assert e.value.code == "backend" and "gave up" in e.value.message
        be.synchronize()                                                        # the word was cleared: the device is usable
        # the same through execute: the all-reduce in front of a launch list poisons that list's wait
        _lib.check(lib.lapid_b200_tp_all_reduce(comm, data._h, 0, count))
        n, k = 64, 512
        qb = oracle.quantize(O.Q4_K, O.normal(1500, n * k, 0.05), n, k)
        x = O.normal(1501, k)
        bufs = [be.upload(x), be.upload(qb), be.alloc(n * 4)]
        with pytest.raises(lp.LapidError) as e:
            be.execute([matmul_launch(lp.DType.Q4K, 1, n, k)], bufs)
        assert e.value.code == "backend"
        be.execute([matmul_launch(lp.DType.Q4K, 1, n, k)], bufs)               # and the next one works
        want, _ = oracle.matmul(O.Q4_K, x, qb, n, k, m=1)
        assert max_rel(bufs[2].download().view(np.float32), want) <= 2e-5
    finally:
        be.set_option("tp_spin_limit", "0")
        lib.lapid_b200_tp_comm_free(comm)


def test_a_staging_region_that_is_never_freed_is_reported(be, oracle):
    """Failure detection without a GPU fault, balanced-stream kernel: the staging region of a launch that runs ahead
    looks owned by a launch that never frees it (a test hook writes a foreign owner word), so the claim of every CTA
    runs out after a short limit (option gemv_stream_spin_limit); the kernels return, the list's wait fails with
    "backend", the workspace is cleared and the same list then runs and is right."""
    m, n, k = 8, 2048, 4096
    qbs = [oracle.quantize(O.Q4_K, O.normal(1700 + i, n * k, 0.05), n, k) for i in range(3)]
    x = O.normal(1710, m * k)
    want = oracle.matmul(O.Q4_K, x, qbs[-1], n, k, m=m)[0]
    bufs = [be.upload(x)] + [be.upload(q) for q in qbs] + [be.alloc(m * n * 4)]
    # (launches that overwrite each other's output are never grouped: three kernels, the last two run ahead)
    ls = [matmul_launch(lp.DType.Q4K, m, n, k, inputs=(0, 1 + i), output=4) for i in range(3)]
    be.set_option("gemv_stream", "2")
    be.set_option("gemv_stream_spin_limit", "3000")
    be.set_option("gemv_stream_debug", "8")
    try:
        with pytest.raises(lp.LapidError) as e:
            be.execute(ls, bufs)
        assert e.value.code == "backend" and "gave up" in e.value.message
    finally:
        be.set_option("gemv_stream_debug", "0")
        be.set_option("gemv_stream_spin_limit", "0")
    try:
        be.execute(ls, bufs)
        assert max_rel(bufs[4].download().view(np.float32), want) <= 2e-5
    finally:
        be.set_option("gemv_stream", "1")


# ------------------------------------------------------------------ epilogue expressions
def _expr_cases():
    from lapid_b200.backend import Expr
    acc, ext = Expr.load(0), Expr.load(1)
    return [("silu", Expr.silu(acc), False), ("mul", acc * ext, True), ("silu_mul", Expr.silu(acc) * ext, True),
            ("gelu_tanh", Expr.gelu_tanh(acc), False), ("relu", Expr.where(acc.lt(0.0), 0.0, acc), False),
            ("mix", ((acc * acc + 1.0).sqrt() - ext.abs().max(0.25)).min(acc * 0.5 + 1.0), True)]


@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q4K, O.Q4_K), (lp.DType.Q5K, O.Q5_K), (lp.DType.Q6K, O.Q6_K), (lp.DType.Int8, O.INT8),
                                      (lp.DType.Int4, O.INT4), (lp.DType.MXFP4, O.MXFP4)])
def test_epilogue_expressions(be, oracle, fmt, ofmt):
    """`MatMulSpec.epilogue` as an expression (crates/lapid-compiler/src/ir.rs:94-111, applied by
    `Epilogue::apply`, crates/lapid-cpu/src/matmul/mod.rs:133-161): the gate / up epilogues of a gated MLP
    (crates/lapid-nn/src/mlp.rs:84) and other f32 trees, through every decode kernel (one row, few rows, shapes that
    take the fast, the tensor-core, the balanced-stream and the generic kernels, a list whose launches run ahead) and
    through the prefill kernels, against the oracle's result with the expression applied by numpy. Bars: decode
    and the exact prefill kernel max_rel 2e-5 (transcendental nodes: CUDA's f32 functions against numpy's); prefill on
    tensor cores (bf16 operands) rel_l2 4e-3 and max_rel 5e-2 (the expression scales the operands' rounding)."""
    shapes = [(1, 96, 2048), (2, 130, 2048), (4, 77, 4096), (8, 2500, 4096), (3, 33, 256), (8, 4096, 4096), (40, 200, 2048), (128, 256, 4096)]
    for (name, e, has) in _expr_cases():
        launches, bufs, wants = [], [], []
        for i, (m, n, k) in enumerate(shapes):
            seed = 1500 + 7 * i
            qb = oracle.quantize(ofmt, O.normal(seed, n * k, 0.05), n, k)
            a = O.normal(seed + 1, m * k)
            x = (O.normal(seed + 2, m * n) * 0.5 + 0.7).astype(np.float32)
            acc, path = oracle.matmul(ofmt, a, qb, n, k, m=m)
            want = O.epilogue(e.words, acc.reshape(m, n), x.reshape(m, n) if has else None).reshape(-1)
            base = len(bufs)
            bufs += [be.upload(a), be.upload(qb), be.alloc(m * n * 4)] + ([be.upload(x)] if has else [])
            launches.append(matmul_launch(fmt, m, n, k, inputs=(base, base + 1), output=base + 2, expr=e, extra_input=base + 3 if has else None))
            wants.append((base + 2, want, m, path))
        be.prepare(launches)
        be.execute(launches, bufs)      # one list: the decode launches behind the first run ahead of their predecessors
        for (b, want, m, path) in wants:
            got = bufs[b].download().view(np.float32)
            tc = path == "f32_act" and fmt in (lp.DType.Q4K, lp.DType.Q5K, lp.DType.Q6K)
            assert max_rel(got, want) <= (5e-2 if tc else 2e-5), (name, m, max_rel(got, want))
            assert rel_l2(got, want) <= (4e-3 if tc else 1e-5), (name, m, rel_l2(got, want))
        for l, (b, want, m, path) in zip(launches, wants):   # and each launch alone (a dependent launch)
            bufs[b].write(0, np.zeros(want.size, np.float32))
            be.execute([l], bufs)
            got = bufs[b].download().view(np.float32)
            tc = path == "f32_act" and fmt in (lp.DType.Q4K, lp.DType.Q5K, lp.DType.Q6K)
            assert max_rel(got, want) <= (5e-2 if tc else 2e-5), (name, m, "alone", max_rel(got, want))


def test_epilogue_expression_is_validated(be, oracle):
    from lapid_b200.backend import Expr
    n, k = 64, 256
    qb = oracle.quantize(O.Q4_K, O.normal(1600, n * k, 0.05), n, k)
    bufs = [be.upload(O.normal(1601, k)), be.upload(qb), be.alloc(n * 4), be.upload(O.normal(1602, n))]

    def run(words, extra=False):
        l = matmul_launch(lp.DType.Q4K, 1, n, k, expr=Expr(words), extra_input=3 if extra else None)
        with pytest.raises(lp.LapidError) as err:
            be.execute([l], bufs)
        return err.value.code

    assert run([16]) == "invalid_launch"                     # a unary node on an empty stack
    assert run([1, 1]) == "invalid_launch"                   # two values left
    assert run([1, 2]) == "invalid_launch"                   # ends inside a constant
    assert run([1, 99]) == "unsupported"                     # an unknown node
    assert run([1 | 2 << 8]) == "unsupported"                # Load(2): one extra is supported
    assert run([1, 1, 1, 1, 1, 32, 32, 32, 32]) == "unsupported"   # five values on the stack
    l = matmul_launch(lp.DType.Q4K, 1, n, k, expr=Expr.load(0) * Expr.load(1), extra_input=3)
    import dataclasses as dc
    with pytest.raises(lp.LapidError) as err:                # the program loads the extra but the launch has two inputs
        be.execute([dc.replace(l, inputs=(0, 1))], bufs)
    assert err.value.code == "invalid_launch"
    be.execute([l], bufs)                                    # and the device still works
    acc, _ = oracle.matmul(O.Q4_K, bufs[0].download().view(np.float32), qb, n, k, m=1)
    assert max_rel(bufs[2].download().view(np.float32), acc * bufs[3].download().view(np.float32)) <= 2e-5


def test_take_profile(be, oracle):
    """`Backend::take_profile` (crates/lapid-compiler/src/backend.rs:59-62): with the option on, the GPU time of every
    launch is added to its kernel kind; the call returns (kind, launches, ms) by time and clears the totals; results are
    those of an ordinary run."""
    n, k = 512, 2048
    qb = oracle.quantize(O.Q4_K, O.normal(1800, n * k, 0.05), n, k)
    a1, a64 = O.normal(1801, k), O.normal(1802, 64 * k)
    table = oracle.quantize(O.Q6_K, O.normal(1803, 32 * 256, 0.05), 32, 256)
    ids = np.array([3, 31, 0], np.int32)
    bufs = [be.upload(a1), be.upload(qb), be.alloc(n * 4), be.upload(a64), be.alloc(64 * n * 4), be.upload(table), be.upload(ids), be.alloc(3 * 256 * 4)]
    ls = [matmul_launch(lp.DType.Q4K, 1, n, k, inputs=(0, 1), output=2), matmul_launch(lp.DType.Q4K, 1, n, k, inputs=(0, 1), output=2),
          matmul_launch(lp.DType.Q4K, 64, n, k, inputs=(3, 1), output=4), lp.backend.gather_launch(lp.DType.Q6K, 32, 256, 3, inputs=(5, 6), output=7)]
    assert be.take_profile() == []
    be.execute(ls, bufs)
    assert be.take_profile() == []              # off by default
    be.set_option("profile", "1")
    try:
        be.execute(ls, bufs)
        be.execute(ls[:1], bufs)
        prof = be.take_profile()
        assert sorted((kind, cnt) for kind, cnt, _ in prof) == [("gather", 1), ("matmul_decode", 3), ("matmul_prefill", 1)]
        assert all(0.0 < ms < 50.0 for _, _, ms in prof) and [ms for _, _, ms in prof] == sorted((ms for _, _, ms in prof), reverse=True)
        assert be.take_profile() == []          # drained
    finally:
        be.set_option("profile", "0")
    want, _ = oracle.matmul(O.Q4_K, a1, qb, n, k, m=1)
    assert max_rel(bufs[2].download().view(np.float32), want) <= 2e-5


def test_execute_io_pipelines_a_step_with_host_buffers(be, oracle):
    """`lapid_b200_execute_io`: Backend::write, execute and read of a step (crates/lapid-compiler/src/backend.rs:36-58)
    as one call whose uploads, launches and downloads overlap by chunks. Same results as the three calls one after
    the other, for every chunk size; launches of a later chunk read what an earlier chunk wrote; misdeclared
    transfers are refused."""
    import torch
    from lapid_b200.backend import matmul_launch
    k = 2048
    shapes = [(1, 96), (2, 130), (4, 77), (8, 2500), (3, 33), (8, 512), (40, 200), (1, 64)]
    a_off = np.cumsum([0] + [m * k for m, _ in shapes])
    o_off = np.cumsum([0] + [m * n for m, n in shapes])
    h_in = torch.randn(int(a_off[-1])).pin_memory()
    h_out = torch.zeros(int(o_off[-1]) + 8 * 64).pin_memory()
    weights = [oracle.quantize(O.Q4_K, O.normal(1700 + i, n * k, 0.05), n, k) for i, (m, n) in enumerate(shapes)]
    w_chain = oracle.quantize(O.Q4_K, O.normal(1750, 64 * shapes[5][1], 0.05), 64, shapes[5][1])   # reads launch 5's output (8 x 512)
    bufs = [be.alloc(int(a_off[-1]) * 4), be.alloc(int(o_off[-1]) * 4)] + [be.upload(w) for w in weights] + [be.upload(w_chain), be.alloc(8 * 64 * 4)]
    launches = [matmul_launch(lp.DType.Q4K, m, n, k, inputs=(0, 2 + i), output=1, a=MatView(int(a_off[i]), m * k, k), out=MatView(int(o_off[i]), m * n, n))
                for i, (m, n) in enumerate(shapes)]
    chain = len(launches)
    launches.append(matmul_launch(lp.DType.Q4K, 8, 64, shapes[5][1], inputs=(1, 2 + len(shapes)), output=3 + len(shapes),
                                  a=MatView(int(o_off[5]), 8 * 512, 512)))
    writes = [(0, int(a_off[i]) * 4, h_in.data_ptr() + int(a_off[i]) * 4, shapes[i][0] * k * 4, i) for i in range(len(shapes))]
    reads = [(1, int(o_off[i]) * 4, h_out.data_ptr() + int(o_off[i]) * 4, shapes[i][0] * shapes[i][1] * 4, i) for i in range(len(shapes))]
    reads.append((3 + len(shapes), 0, h_out.data_ptr() + int(o_off[-1]) * 4, 8 * 64 * 4, chain))
    # the three calls one after the other
    be.write_ptr(bufs[0], 0, h_in.data_ptr(), int(a_off[-1]) * 4)
    be.execute(launches, bufs)
    want = np.concatenate([bufs[1].download().view(np.float32), bufs[3 + len(shapes)].download().view(np.float32)[:8 * 64]])
    for i, (m, n) in enumerate(shapes):   # (and those against the oracle)
        ref, _ = oracle.matmul(O.Q4_K, h_in.numpy()[a_off[i]:a_off[i + 1]], weights[i], n, k, m=m)
        tc = m > 8
        assert max_rel(want[o_off[i]:o_off[i + 1]], ref) <= (2e-2 if tc else 2e-5)
    for chunk in (0, 1, 2, 3, 4, len(launches), 100):
        bufs[0].write(0, np.zeros(int(a_off[-1]), np.float32))
        bufs[1].write(0, np.zeros(int(o_off[-1]), np.float32))
        h_out.zero_()
        be.execute_io(launches, bufs, writes, reads, chunk)
        # (which decode launches share a kernel depends on the chunk: the order of some f32 partial sums with it)
        assert max_rel(h_out.numpy()[:want.size], want) <= 2e-6, chunk
    # a write tied to launch 6 whose memory launch 1 (an earlier chunk) reads; a read tied to launch 0 of memory that launch 7 writes
    bad_w = writes[:1] + [(0, int(a_off[1]) * 4, h_in.data_ptr(), 64, 6)]
    with pytest.raises(lp.LapidError) as err:
        be.execute_io(launches, bufs, bad_w, reads, 2)
    assert err.value.code == "invalid_launch"
    bad_r = [(1, int(o_off[7]) * 4, h_out.data_ptr(), 64, 0)]
    with pytest.raises(lp.LapidError) as err:
        be.execute_io(launches, bufs, writes, bad_r, 2)
    assert err.value.code == "invalid_launch"
    with pytest.raises(lp.LapidError) as err:
        be.execute_io(launches, bufs, [(0, bufs[0].nbytes - 8, h_in.data_ptr(), 64, 0)], reads, 2)
    assert err.value.code == "out_of_bounds"
    with pytest.raises(lp.LapidError) as err:
        be.execute_io(launches, bufs, [(0, 0, h_in.data_ptr(), 64, len(launches))], reads, 2)
    assert err.value.code == "invalid_launch"
    be.execute_io([], bufs, writes[:1], [(0, 0, h_out.data_ptr(), 64, 0)], 0)       # no launches: the writes, then the reads
    assert np.array_equal(h_out.numpy()[:16], h_in.numpy()[:16])
    h_out.zero_()
    be.execute_io(launches, bufs, writes, reads, 0)                                  # and the device still works
    assert max_rel(h_out.numpy()[:want.size], want) <= 2e-6


@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q5K, O.Q5_K), (lp.DType.Q6K, O.Q6_K)])
def test_small_matrices_at_three_and_four_rows_take_the_dp4a_kernel(oracle, fmt, ofmt):
    """Default routing: a Q5_K / Q6_K launch over at most 6 M weights with three or four rows runs on the dp4a kernel
    (its result is bit-identical to the run with the tensor-core kernels switched off), five rows and larger matrices
    on the tensor-core kernels; all of them agree with the oracle."""
    be = lp.Backend(0)
    for (m, n, k, dp4a) in [(3, 1024, 4096, True), (4, 1024, 4096, True), (5, 1024, 4096, False), (4, 1536, 4096, True), (4, 4096, 4096, False)]:
        qb = oracle.quantize(ofmt, O.normal(1800 + m, n * k, 0.05), n, k)
        a = O.normal(1810 + m, m * k)
        want, _ = oracle.matmul(ofmt, a, qb, n, k, m=m)
        got = run_matmul(be, fmt, a, qb, m, n, k)
        assert max_rel(got, want) <= 2e-5, (m, n, k)
        be.set_option("gemv_mma_rows", "0")
        plain = run_matmul(be, fmt, a, qb, m, n, k)
        be.set_option("gemv_mma_rows", "2")
        assert np.array_equal(got, plain) == dp4a, (m, n, k)


def test_mxfp4_decode_staged_and_direct_forms(be, oracle):
    """The MXFP4 decode kernel streams rows through shared memory when K is a multiple of 512 and reads them directly
    otherwise: same arithmetic in the same order, so the two forms agree bit for bit on shapes both can run; both
    against the oracle; the expert-indexed launch included."""
    from lapid_b200.backend import matmul_id_launch
    rng = np.random.default_rng(21)
    for (m, n, k) in [(1, 4096, 4096), (2, 130, 512), (2, 77, 1024), (8, 1030, 14336), (1, 9, 2560), (1, 33, 28672), (2, 700, 7680), (4, 50, 96)]:
        raw = rng.integers(0, 256, n * k // 32 * 17, dtype=np.uint8)
        raw.reshape(-1, 17)[:, 0] = rng.integers(118, 132, n * k // 32, dtype=np.uint8)   # scales around 2^-8
        qb = np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])
        a = O.normal(1900 + m, m * k)
        want, _ = oracle.matmul(O.MXFP4, a, qb, n, k, m=m)
        got = {}
        be.set_option("gemv_mxfp4_mma_rows", "0")       # (the dp4a kernel at every row count)
        be.set_option("gemv_mxfp4_k_split", "1")
        for staged in ("1", "0"):
            be.set_option("gemv_mxfp4_staged", staged)
            got[staged] = run_matmul(be, lp.DType.MXFP4, a, qb, m, n, k)
            assert max_rel(got[staged], want) <= 2e-5, (m, n, k, staged)
        assert np.array_equal(got["0"], got["1"]), (m, n, k)
        for split in ("2", "4", "0"):                   # two and four warps per row, then the launch's own choice
            be.set_option("gemv_mxfp4_k_split", split)
            assert max_rel(run_matmul(be, lp.DType.MXFP4, a, qb, m, n, k), want) <= 2e-5, (m, n, k, split)
        be.set_option("gemv_mxfp4_staged", "1")
        be.set_option("gemv_mxfp4_mma_rows", "3")
    t, r, e, n, k = 3, 2, 4, 200, 1024   # (an expert-indexed launch is one-row work per pair: staged)
    one = oracle.layout(O.MXFP4, n, k).total
    stack = np.zeros(e * one, np.uint8)
    for x in range(e):
        raw = rng.integers(0, 256, n * k // 32 * 17, dtype=np.uint8)
        raw.reshape(-1, 17)[:, 0] = rng.integers(118, 132, n * k // 32, dtype=np.uint8)
        stack[x * one:x * one + raw.size] = raw
    xs = O.normal(1950, t * k)
    ids = np.array([(i * 3 + 1) % e for i in range(t * r)], np.int32)
    want = oracle.matmul_id(O.MXFP4, xs, stack, ids, t, r, e, n, k)
    bufs = [be.upload(xs), be.upload(stack), be.upload(ids.view(np.uint8)), be.alloc(t * r * n * 4)]
    res = {}
    for staged in ("1", "0"):
        be.set_option("gemv_mxfp4_staged", staged)
        be.execute([matmul_id_launch(lp.DType.MXFP4, t, r, e, n, k)], bufs)
        res[staged] = bufs[3].download().view(np.float32).copy()
        assert max_rel(res[staged], want) <= 2e-5
    be.set_option("gemv_mxfp4_staged", "1")
    assert np.array_equal(res["0"], res["1"])


def test_gemv_mxfp4_tensor_core_decode_kernel(be, oracle):
    """The MXFP4 tensor-core decode kernel (1..8 rows, K a multiple of 512) against the oracle and against the dp4a
    kernel: random blocks (every code, "-0" included, scale bytes from denormal to large), ragged n, every row
    count, a bias, K with several chunks per warp, a row of all-negative and a row of all-zero codes."""
    rng = np.random.default_rng(23)
    try:
        for (m, n, k, bias) in [(1, 200, 512, False), (2, 130, 2048, False), (3, 77, 512, True), (4, 513, 4096, False), (5, 100, 1536, False),
                                (6, 1, 1024, False), (7, 33, 14336, True), (8, 300, 4096, False), (8, 17, 14336, False), (1, 4096, 4096, False)]:
            raw = rng.integers(0, 256, n * k // 32 * 17, dtype=np.uint8)
            b2 = raw.reshape(-1, 17)
            b2[:, 0] = rng.integers(110, 140, b2.shape[0], dtype=np.uint8)
            b2[:4, 0] = [0, 1, 2, 150]                     # denormal, smallest normal and a large scale
            b2[5, 1:] = 0xFF                               # all codes 15 (-12)
            b2[6, 1:] = 0x88                               # all "-0"
            b2[7, 1:] = 0x00
            qb = np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])
            a = O.normal(2000 + m, m * k)
            bv = O.normal(2050 + m, n) if bias else None
            want, _ = oracle.matmul(O.MXFP4, a, qb, n, k, m=m, bias=bv)
            be.set_option("gemv_mxfp4_mma_rows", "1")
            got = run_matmul(be, lp.DType.MXFP4, a, qb, m, n, k, bias=bv)
            be.set_option("gemv_mxfp4_mma_rows", "0")
            ref = run_matmul(be, lp.DType.MXFP4, a, qb, m, n, k, bias=bv)
            assert max_rel(got, want) <= 2e-5, (m, n, k, max_rel(got, want))
            assert max_rel(got, ref) <= 2e-5, (m, n, k)
    finally:
        be.set_option("gemv_mxfp4_mma_rows", "3")


def test_gemv_int4_bulk_copy_kernel(be, oracle):
    """The bulk-copy decode kernel over Int4 nibble planes (K a multiple of 512; one row by default, every row count
    with the tensor-core kernels switched off) against the oracle and against the plain streaming kernel: a K whose last
    1024-weight step is half empty, several stages per row, ragged n, a bias, launches that run ahead of their
    predecessor (a list of one-row launches), both ends of the 4-bit range."""
    be.set_option("gemv_mma_rows", "0")
    try:
        seed = 2100
        for (m, n, k, bias) in [(1, 77, 512, True), (1, 4096, 4096, False), (2, 513, 1536, False), (3, 100, 5632, True), (5, 33, 14336, False),
                                (8, 300, 4096, False), (1, 9, 28672, False)]:
            seed += 1
            w = O.normal(seed, n * k, 0.05).reshape(n, k).copy()
            w[0, :] = -1.0
            w[0, ::32] = 0.0
            qb = oracle.quantize(O.INT4, w.reshape(-1), n, k)
            a = O.normal(seed + 50, m * k)
            bv = O.normal(seed + 70, n) if bias else None
            want, _ = oracle.matmul(O.INT4, a, qb, n, k, m=m, bias=bv)
            got = run_matmul(be, lp.DType.Int4, a, qb, m, n, k, bias=bv)
            be.set_option("gemv", "generic")
            ref = run_matmul(be, lp.DType.Int4, a, qb, m, n, k, bias=bv)
            be.set_option("gemv", "fast")
            assert max_rel(got, want) <= 2e-5, (m, n, k, max_rel(got, want))
            assert max_rel(ref, want) <= 2e-5, (m, n, k)
        # a list of one-row launches: all but the first run ahead of their predecessor (early mode)
        n, k = 1024, 4096
        qbs = [oracle.quantize(O.INT4, O.normal(2150 + i, n * k, 0.05), n, k) for i in range(4)]
        x = O.normal(2160, k)
        bufs = [be.upload(x)] + [be.upload(q) for q in qbs] + [be.alloc(n * 4) for _ in range(4)]
        ls = [matmul_launch(lp.DType.Int4, 1, n, k, inputs=(0, 1 + i), output=5 + i) for i in range(4)]
        be.execute(ls, bufs)
        for i in range(4):
            want, _ = oracle.matmul(O.INT4, x, qbs[i], n, k, m=1)
            assert max_rel(bufs[5 + i].download().view(np.float32), want) <= 2e-5, i
    finally:
        be.set_option("gemv_mma_rows", "2")
        be.set_option("gemv", "fast")
