"""Pins the CPU oracle: every known-answer / property test the reference holds for the
quantized-matmul path, restated against ``oracle/lapid_oracle.c``, plus independent cross-checks
(numpy float16 conversion, the third-party ``gguf`` package's dequantizers and Q8_0 quantizer).

Reference tests ported here (file:line within the reference tree):
  crates/lapid-quant/src/imp.rs:275-389   layout_sizes, i8_test_vector, zero_groups,
                                          round_trip_error_bounds, k_formats, ggml_blocks_round_trip
  crates/lapid-quant/src/kquant.rs:419-452 nearest_int_rounds_half_even, round_trip_relative_error,
                                          zeros_and_constants
  crates/lapid-cpu/src/kquant.rs:360-386   dequant_matches_ggml, tiles_match_dequant_reference
  crates/lapid-cpu/src/matmul/qkernels.rs:217-255 simd_tiles_match_scalar (scalar tile vs dequant)
  crates/lapid-cpu/src/matmul/quant.rs:191-215    quantize_row_roundtrip
  crates/lapid-cpu/src/matmul/matmul_tests.rs:30-139 quantized_large_m_matches_dequantized_f32,
                                          kquant_matmul_matches_dequantized_f32
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.refgen import make_blocks, noise, rnd

INT8, INT4, Q4_K, Q5_K, Q6_K = O.INT8, O.INT4, O.Q4_K, O.Q5_K, O.Q6_K


def rel_err(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    return float(np.sqrt(((got - want) ** 2).sum() / max((want ** 2).sum(), 1e-30)))


# ------------------------------------------------------------------ half conversions
def test_f16_to_f32_matches_numpy_for_every_half(oracle):
    allh = np.arange(1 << 16, dtype=np.uint16)
    want = allh.view(np.float16).astype(np.float32).view(np.uint32)
    got = np.array([np.float32(oracle.f16_bits_to_f32(int(h))) for h in allh], dtype=np.float32).view(np.uint32)
    finite = (allh & 0x7C00) != 0x7C00
    assert np.array_equal(got[finite], want[finite])
    inf = (allh & 0x7FFF) == 0x7C00
    assert np.array_equal(got[inf], want[inf])


def test_f32_to_f16_round_to_nearest_even(oracle):
    rng = np.random.default_rng(5)
    # exact halves, their midpoints and neighbours, subnormals, overflow edge, random values
    halves = np.arange(1 << 16, dtype=np.uint16).view(np.float16).astype(np.float32)
    halves = halves[np.isfinite(halves)]
    mids = (halves[:-1].astype(np.float64) + halves[1:].astype(np.float64)) / 2
    mids = mids[np.isfinite(mids)].astype(np.float32)
    cand = np.concatenate([
        halves[::17], mids[::13], np.nextafter(mids[::29], np.float32(np.inf)), np.nextafter(mids[::31], np.float32(-np.inf)),
        rng.standard_normal(20000).astype(np.float32) * np.float32(0.02),
        rng.standard_normal(5000).astype(np.float32) * np.float32(1e-6),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 5.96e-8,
                  16.0 / 127.0, np.inf, -np.inf], dtype=np.float32),
    ])
    with np.errstate(over="ignore"):
        want = cand.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16_bits(float(v)) for v in cand], dtype=np.uint16)
    assert np.array_equal(got, want)
    assert oracle.f32_to_f16_bits(float("nan")) & 0x7C00 == 0x7C00 and oracle.f32_to_f16_bits(float("nan")) & 0x3FF


def test_nearest_int_rounds_half_even(oracle):
    assert [oracle.nearest_int(v) for v in (0.5, 1.5, -0.5, -1.5, 2.4)] == [0, 2, 0, -2, 2]


# ------------------------------------------------------------------ lapid-quant: layout and Int8
def test_layout_sizes(oracle):
    l = oracle.layout(INT8, 1, 32)
    assert (l.qs_bytes, l.scales_offset, l.scales_bytes, l.total) == (32, 256, 2, 512)
    l = oracle.layout(INT8, 768, 768)
    assert l.scales_offset == 768 * 768 and l.total % 256 == 0
    for fmt, bb in ((Q4_K, 144), (Q5_K, 176), (Q6_K, 210)):
        l = oracle.layout(fmt, 3, 512)
        assert (l.qs_offset, l.qs_bytes, l.scales_offset, l.scales_bytes) == (0, 3 * 2 * bb, 3 * 2 * bb, 0)
        assert l.total == (3 * 2 * bb + 255) // 256 * 256
    # sizes quoted for the benchmark shapes
    assert oracle.layout(Q4_K, 4096, 4096).total == 9_437_184
    assert oracle.layout(Q6_K, 4096, 4096).total == 13_762_560
    assert oracle.layout(INT8, 4096, 4096).total == 17_825_792
    assert oracle.layout(Q4_K, 14336, 4096).total == 33_030_144
    with pytest.raises(O.OracleError):
        oracle.layout(Q4_K, 2, 128)
    with pytest.raises(O.OracleError):
        oracle.layout(INT8, 2, 48)


def test_i8_test_vector(oracle):
    ramp = np.arange(32, dtype=np.float32) - 16.0
    q = oracle.quantize(INT8, ramp, 1, 32)
    expect = [-127, -119, -111, -103, -95, -87, -79, -71, -64, -56, -48, -40, -32, -24, -16, -8, 0, 8, 16, 24, 32, 40,
              48, 56, 64, 71, 79, 87, 95, 103, 111, 119]
    assert q[:32].view(np.int8).tolist() == expect
    assert q[256:258].tolist() == [0x08, 0x30]  # f16 bits 0x3008, little endian
    assert not q[32:256].any() and not q[258:].any()
    assert q.size == 512


def test_i4_test_vector(oracle):
    """`i4_test_vector` and `i4_positive_max_maps_to_minus_eight` (crates/lapid-quant/src/imp.rs:283-304)."""
    ramp = np.arange(32, dtype=np.float32) - 16.0
    q = oracle.quantize(INT4, ramp, 1, 32)
    assert q[:16].tolist() == [0x80, 0x91, 0x91, 0xa2, 0xa2, 0xb3, 0xb3, 0xc4, 0xc4, 0xd5, 0xd5, 0xe6, 0xe6, 0xf7, 0xf7, 0xf8]
    assert q[256:258].tolist() == [0x00, 0x40]  # d = -16 / -8 = 2.0 = f16 0x4000
    x = oracle.dequantize(INT4, q, 1, 32).reshape(-1)
    assert (x[0], x[16], x[31]) == (-16.0, 0.0, 14.0)
    l = oracle.layout(INT4, 1, 32)
    assert (l.qs_bytes, l.scales_offset, l.scales_bytes, l.total) == (16, 256, 2, 512)
    v = np.full(32, 0.5, np.float32)
    v[3] = 4.0
    assert oracle.dequantize(INT4, oracle.quantize(INT4, v, 1, 32), 1, 32).reshape(-1)[3] == 4.0


def test_zero_groups(oracle):
    for fmt in (INT8, INT4):
        q = oracle.quantize(fmt, np.zeros(64, dtype=np.float32), 2, 32)
        l = oracle.layout(fmt, 2, 32)
        assert not q[l.scales_offset:l.scales_offset + l.scales_bytes].any()
        assert not oracle.dequantize(fmt, q, 2, 32).any()


def test_round_trip_error_bounds_int8(oracle):
    rows, cols = 7, 96
    x = noise(rows * cols, 42, 3.0)
    q = oracle.quantize(INT8, x, rows, cols)
    assert q.size == oracle.layout(INT8, rows, cols).total
    y = oracle.dequantize(INT8, q, rows, cols).reshape(-1)
    g = x.reshape(rows, cols // 32, 32)
    amax = np.abs(g).max(axis=2, keepdims=True)
    tol = amax / 127.0 * 0.5 + amax * 1e-3 + 1e-6
    assert (np.abs(g - y.reshape(g.shape)) <= tol).all()
    # Int4: up to one step (the side opposite to the extreme saturates at +7), imp.rs:325-330
    q4 = oracle.quantize(INT4, x, rows, cols)
    assert q4.size == oracle.layout(INT4, rows, cols).total
    y4 = oracle.dequantize(INT4, q4, rows, cols).reshape(g.shape)
    assert (np.abs(g - y4) <= amax / 8.0 + amax * 1e-3 + 1e-6).all()


def test_k_formats(oracle):
    rows, cols = 3, 512
    x = noise(rows * cols, 11, 2.0)
    for fmt, tol, bb in ((Q4_K, 0.25, 144), (Q5_K, 0.12, 176), (Q6_K, 0.06, 210)):
        q = oracle.quantize(fmt, x, rows, cols)
        l = oracle.layout(fmt, rows, cols)
        assert q.size == l.total and l.qs_bytes == rows * 2 * bb
        y = oracle.dequantize(fmt, q, rows, cols)
        assert (np.abs(x - y.reshape(-1)) < tol).all()
        assert np.array_equal(oracle.from_ggml_blocks(fmt, q[:l.qs_bytes], rows, cols), q)
        with pytest.raises(O.OracleError):
            oracle.from_ggml_blocks(fmt, q[:l.qs_bytes - 1], rows, cols)


def test_ggml_blocks_round_trip_int8(oracle):
    rows, cols = 3, 64
    x = noise(rows * cols, 7, 1.0)
    ours = oracle.quantize(INT8, x, rows, cols)
    l = oracle.layout(INT8, rows, cols)
    ng = rows * cols // 32
    blocks = np.empty((ng, 34), dtype=np.uint8)
    blocks[:, :2] = ours[l.scales_offset:l.scales_offset + 2 * ng].reshape(ng, 2)
    blocks[:, 2:] = ours[:ng * 32].reshape(ng, 32)
    assert np.array_equal(oracle.from_ggml_blocks(INT8, blocks.reshape(-1), rows, cols), ours)


# ------------------------------------------------------------------ lapid-quant: K formats
def test_round_trip_relative_error(oracle):
    x = noise(256, 3)
    x[17] = 4.0
    rms = np.sqrt((x.astype(np.float64) ** 2).mean())
    for fmt, tol in ((Q4_K, 0.08), (Q5_K, 0.04), (Q6_K, 0.02)):
        y = oracle.dequantize_block(fmt, oracle.quantize_block(fmt, x))
        err = np.sqrt(((x - y).astype(np.float64) ** 2).mean())
        assert err / rms < tol


def test_zeros_and_constants(oracle):
    for fmt in (Q4_K, Q5_K, Q6_K):
        for c in (0.0, 1.0, -2.5):
            b = oracle.quantize_block(fmt, np.full(256, c, dtype=np.float32))
            y = oracle.dequantize_block(fmt, b)
            assert (np.abs(y - c) <= abs(c) * 0.01 + 1e-6).all(), (fmt, c)
            if c == 0.0:
                assert not b.any()  # kquant.rs:304-307 for Q6_K; scale 0 everywhere for Q4_K


def _gguf():
    """The third-party package of the independent cross-checks; only the tests that use it skip without it."""
    return pytest.importorskip("gguf")


def _gguf_deq(fmt, blocks):
    gguf = _gguf()
    from gguf import quants
    t = {Q4_K: gguf.GGMLQuantizationType.Q4_K, Q5_K: gguf.GGMLQuantizationType.Q5_K, Q6_K: gguf.GGMLQuantizationType.Q6_K,
         INT8: gguf.GGMLQuantizationType.Q8_0}[fmt]
    return quants.dequantize(blocks, t)


@pytest.mark.parametrize("fmt,bb,d_off,dm_off", [(Q4_K, 144, 0, 2), (Q5_K, 176, 0, 2), (Q6_K, 210, 208, None)])
def test_dequant_bit_exact_vs_independent_dequantizer(oracle, fmt, bb, d_off, dm_off):
    """`dequant_matches_ggml`: random valid blocks decode to the same f32 bits as an independent
    implementation of GGUF's K-quant dequantizers."""
    blocks = make_blocks(bb, 64, 7, d_off, dm_off)
    # vary d / dmin across blocks (finite halves of several magnitudes, a negative one, a subnormal)
    b2 = blocks.reshape(64, bb)
    ds = np.array([0.01, 0.25, 3e-5, -0.02, 6e-8, 1.5, 0.003, 7.0], dtype=np.float16).view(np.uint8).reshape(8, 2)
    for i in range(64):
        b2[i, d_off:d_off + 2] = ds[i % 8]
        if dm_off is not None:
            b2[i, dm_off:dm_off + 2] = ds[(i * 3 + 1) % 8]
    want = _gguf_deq(fmt, b2.copy()).reshape(64, 256).astype(np.float32)
    got = np.stack([oracle.dequantize_block(fmt, b2[i]) for i in range(64)])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # and whole-matrix dequantize == per-block
    full = oracle.dequantize(fmt, np.concatenate([blocks, np.zeros((-blocks.size) % 256, np.uint8)]), 8, 2048)
    assert np.array_equal(full.reshape(64, 256).view(np.uint32), want.view(np.uint32))


def test_quantized_bytes_decode_identically_elsewhere(oracle):
    """Bytes produced by the oracle's quantizers are valid GGUF blocks: the independent dequantizer
    reads them to the same values the oracle does (cross-checks packing order and scale packing)."""
    x = O.normal(3, 16 * 1024, 0.02)
    for fmt, bb in ((Q4_K, 144), (Q5_K, 176), (Q6_K, 210)):
        q = oracle.quantize(fmt, x, 16, 1024)
        mine = oracle.dequantize(fmt, q, 16, 1024)
        other = _gguf_deq(fmt, q[:16 * 4 * bb].reshape(64, bb)).reshape(16, 1024).astype(np.float32)
        assert np.array_equal(mine.view(np.uint32), other.view(np.uint32))
        assert rel_err(mine, x) < {Q4_K: 0.08, Q5_K: 0.04, Q6_K: 0.02}[fmt]


def test_int4_planes_decode_like_q4_0_blocks(oracle):
    """GGUF block_q4_0 (f16 d + 16 nibble bytes) -> lapid Int4 planes (`from_ggml_blocks`, imp.rs:180-199):
    the oracle's dequantization of the planes equals the independent Q4_0 dequantizer on the blocks, bit for bit,
    and AoS -> SoA of the oracle's own bytes is the identity."""
    gguf = _gguf()
    from gguf import quants
    rows, cols = 5, 256
    x = O.normal(19, rows * cols, 0.7)
    ours = oracle.quantize(INT4, x, rows, cols)
    l = oracle.layout(INT4, rows, cols)
    ng = rows * cols // 32
    blocks = np.empty((ng, 18), dtype=np.uint8)
    blocks[:, :2] = ours[l.scales_offset:l.scales_offset + 2 * ng].reshape(ng, 2)
    blocks[:, 2:] = ours[:ng * 16].reshape(ng, 16)
    assert np.array_equal(oracle.from_ggml_blocks(INT4, blocks.reshape(-1), rows, cols), ours)
    want = quants.dequantize(blocks, gguf.GGMLQuantizationType.Q4_0).reshape(rows, cols).astype(np.float32)
    got = oracle.dequantize(INT4, ours, rows, cols).reshape(rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_int8_bytes_match_independent_q8_0_quantizer(oracle):
    gguf = _gguf()
    from gguf import quants
    rows, cols = 5, 256
    x = O.normal(9, rows * cols, 0.7).reshape(rows, cols)
    x[2, 40:72] = 0.0
    want = quants.quantize(x, gguf.GGMLQuantizationType.Q8_0).reshape(-1)  # AoS 34-byte blocks
    ours = oracle.quantize(INT8, x, rows, cols)
    assert np.array_equal(oracle.from_ggml_blocks(INT8, want, rows, cols), ours)
    deq = quants.dequantize(want.reshape(rows, -1), gguf.GGMLQuantizationType.Q8_0).astype(np.float32)
    assert np.array_equal(oracle.dequantize(INT8, ours, rows, cols).view(np.uint32), deq.reshape(rows, cols).view(np.uint32))


# ------------------------------------------------------------------ lapid-cpu: activations, tiles
def test_mxfp4_reference_tests_and_independent_codec(oracle):
    """MXFP4 (crates/lapid-quant/src/mxfp4.rs): the reference's own tests `round_trip_exact_grid` and
    `e2m1_pairs_match_blocks` (:90-113), and -- where the third-party package has the format -- its independent
    quantizer AND dequantizer on the same data, byte for byte and bit for bit."""
    MX = O.MXFP4
    x = np.array([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0][i % 8] * (-0.25 if i % 3 == 0 else 0.25) for i in range(32)], np.float32)
    assert np.array_equal(oracle.dequantize_block(MX, oracle.quantize_block(MX, x)), x)
    codes = np.array([i % 16 for i in range(32)], np.uint8)
    packed = (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8)
    y = oracle.dequantize_block(MX, oracle.mxfp4_from_e2m1_pairs(packed, np.array([127], np.uint8), 1, 32))
    e2m1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert all(y[i] == e2m1[c & 7] * (-1.0 if c & 8 else 1.0) for i, c in enumerate(codes))
    l = oracle.layout(MX, 3, 96)
    assert (l.qs_bytes, l.scales_bytes, l.total) == (3 * 3 * 17, 0, 256)
    assert not oracle.quantize(MX, np.zeros(64, np.float32), 2, 32)[:34].any()          # an all-zero block: e = 0, codes 0
    # a block of denormals: floor(log2(amax)) - 2 + 127 is negative and Rust's `as u8` saturates to 0 (mxfp4.rs:43);
    # a C cast of a negative float to uint8_t is undefined (other implementations wrap to 253 here)
    assert oracle.quantize_block(MX, np.full(32, 3e-39, np.float32))[0] == 0
    gguf = _gguf()
    from gguf import quants
    if not hasattr(gguf.GGMLQuantizationType, "MXFP4"):
        pytest.skip("this gguf package has no MXFP4")
    rows, cols = 16, 512
    w = O.normal(77, rows * cols, 0.7).reshape(rows, cols)
    w[0, :32] = np.float32(8.0) * (1 - np.float32(2.0) ** -24)   # log2 rounds up to 3.0 in f32
    w[2, :32] = 1e30
    q = oracle.quantize(MX, w, rows, cols)
    blocks = q[:rows * cols // 32 * 17].reshape(rows, -1)
    assert np.array_equal(quants.quantize(w, gguf.GGMLQuantizationType.MXFP4).reshape(-1), blocks.reshape(-1))
    deq = quants.dequantize(blocks, gguf.GGMLQuantizationType.MXFP4).astype(np.float32)
    assert np.array_equal(deq.view(np.uint32), oracle.dequantize(MX, q, rows, cols).reshape(rows, cols).view(np.uint32))
    # the decode tile against the dequantized product (crates/lapid-cpu/src/matmul/matmul_tests.rs:96-139, shapes with k % 256 != 0)
    for (m, n, k) in [(1, 11, 96), (5, 7, 224), (3, 20, 256), (40, 13, 160)]:
        wq = oracle.quantize(MX, O.normal(80 + m, n * k, 0.5), n, k)
        a = O.normal(90 + m, m * k)
        got, path = oracle.matmul(MX, a, wq, n, k, m=m)
        ref = a.reshape(m, k).astype(np.float64) @ oracle.dequantize(MX, wq, n, k).reshape(n, k).astype(np.float64).T
        err = np.sqrt(((got.reshape(m, n) - ref) ** 2).sum() / (ref ** 2).sum())
        assert path == ("int8_act" if m <= 8 else "f32_act") and err <= (2e-2 if m <= 8 else 1e-5)


def test_quantize_row_roundtrip(oracle):
    x = np.array([((i * 37) % 29) * 0.37 - 5.0 for i in range(64)], dtype=np.float32)
    q, s, _ = oracle.quantize_row_sums(x)
    v = q.astype(np.float32).reshape(2, 32) * s[:, None]
    assert (np.abs(v - x.reshape(2, 32)) <= s[:, None] * 0.5 + 1e-6).all()
    x = np.array([((i * 53) % 61) * 0.21 - 6.0 + (0.5 if i % 32 == 5 else 0.0) for i in range(96)], dtype=np.float32)
    q, s, bs = oracle.quantize_row_sums(x)
    # numpy restatement: d = amax/127, id = 1/d, round half even, bs = d * sum(q)
    g = x.reshape(3, 32)
    d = (np.abs(g).max(axis=1) / np.float32(127.0)).astype(np.float32)
    idv = (np.float32(1.0) / d).astype(np.float32)
    qq = np.clip(np.rint((g * idv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert np.array_equal(q.reshape(3, 32), qq) and np.array_equal(s, d)
    assert np.array_equal(bs, d * qq.astype(np.int32).sum(axis=1).astype(np.float32))
    q, s, bs = oracle.quantize_row_sums(np.zeros(32, dtype=np.float32))
    assert not q.any() and s[0] == 0.0 and bs[0] == 0.0


def test_tiles_match_dequant_reference(oracle):
    rows, n, k = 5, 6, 512
    x = np.array([((i * 37 % 101) - 50.0) * 0.013 for i in range(rows * k)], dtype=np.float32).reshape(rows, k)
    for fmt, bb, d_off, dm_off in ((Q4_K, 144, 0, 2), (Q5_K, 176, 0, 2), (Q6_K, 210, 208, None)):
        raw = make_blocks(bb, n * k // 256, 11, d_off, dm_off)
        w = np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])
        deq = oracle.dequantize(fmt, w, n, k)
        got, path = oracle.matmul(fmt, x, w, n, k, m=rows)
        assert path == "int8_act"
        got = got.reshape(rows, n)
        for r in range(rows):
            q, s, _ = oracle.quantize_row_sums(x[r])
            xa = q.astype(np.float32) * np.repeat(s, 32)
            want = (xa.astype(np.float64)[None, :] * deq.astype(np.float64)).sum(axis=1)
            assert (np.abs(want - got[r]) <= 1e-3 * np.maximum(np.abs(want), 1.0)).all(), fmt


def test_int8_tile_matches_dequant_reference(oracle):
    rows, n, k = 5, 7, 96
    l = oracle.layout(INT8, n, k)
    w = np.zeros(l.total, dtype=np.uint8)
    for i in range(l.qs_bytes):
        b = (i * 73 + 11) % 251
        w[i] = 0x81 if b == 0x80 else b
    sc = np.array([0.01 + (g % 7) * 0.003 for g in range(n * k // 32)], dtype=np.float32).astype(np.float16)
    w[l.scales_offset:l.scales_offset + l.scales_bytes] = sc.view(np.uint8)
    x = O.normal(4, rows * k, 1.0).reshape(rows, k)
    got, path = oracle.matmul(INT8, x, w, n, k, m=rows)
    assert path == "int8_act"
    deq = oracle.dequantize(INT8, w, n, k)
    for r in range(rows):
        q, s, _ = oracle.quantize_row_sums(x[r], want_bs=False)
        xa = q.astype(np.float64) * np.repeat(s, 32)
        want = (xa[None, :] * deq.astype(np.float64)).sum(axis=1)
        assert (np.abs(want - got.reshape(rows, n)[r]) <= 1e-3 * np.maximum(np.abs(want), 1.0)).all()


# ------------------------------------------------------------------ lapid-cpu: whole launches
def test_kquant_matmul_matches_dequantized_f32(oracle):
    seed = 50
    for fmt in (Q4_K, Q5_K, Q6_K):
        for (m, n, k, pad) in [(1, 37, 512, 0), (3, 20, 256, 4), (6, 9, 256, 0), (20, 45, 256, 3), (130, 70, 512, 0),
                               (33, 300, 1024, 0)]:
            seed += 1
            w = rnd(n * k, seed)
            qb = oracle.quantize(fmt, w, n, k)
            deq = oracle.dequantize(fmt, qb, n, k).astype(np.float64)
            rs = k + pad
            a = rnd(m * rs, seed + 7)
            want = a.reshape(m, rs)[:, :k].astype(np.float64) @ deq.T
            for fma in (True, False):
                got, path = oracle.matmul(fmt, a, qb, n, k, m=m, a_view=(0, 0, rs), fma=fma)
                assert path == ("int8_act" if m <= 8 else "f32_act")
                tol = 2e-2 if m <= 8 else 2e-5
                assert rel_err(got, want) <= tol, (fmt, m, n, k)


@pytest.mark.parametrize("fmt", [INT8, INT4])
def test_quantized_large_m_matches_dequantized_f32_int8(oracle, fmt):
    seed = 1 if fmt == INT8 else 5
    for (batch, m, n, k, pad, epi) in [(1, 9, 45, 96, 0, False), (2, 35, 70, 128, 5, True), (1, 130, 200, 256, 3, True)]:
        seed += 1
        w = rnd(n * k, seed)
        qb = oracle.quantize(fmt, w, n, k)
        deq = oracle.dequantize(fmt, qb, n, k).astype(np.float64)
        rs = k + pad
        a = rnd(batch * m * rs, seed + 7)
        bias = rnd(n, seed + 9)
        want = a.reshape(batch * m, rs)[:, :k].astype(np.float64) @ deq.T + (bias.astype(np.float64) if epi else 0.0)
        got, path = oracle.matmul(fmt, a, qb, n, k, batch=batch, m=m, a_view=(0, m * rs, rs), bias=bias if epi else None)
        assert path == "f32_act"
        assert rel_err(got, want) <= 2e-5
    # decode-sized launches: int8 activations against the re-centred nibbles (simd_tiles_match_scalar's reference)
    n, k = 7, 96
    qb = oracle.quantize(fmt, rnd(n * k, 40), n, k)
    deq = oracle.dequantize(fmt, qb, n, k).astype(np.float64)
    x = O.normal(41, 5 * k, 1.0).reshape(5, k)
    got, path = oracle.matmul(fmt, x, qb, n, k, m=5)
    assert path == "int8_act"
    for r in range(5):
        qa, sa, _ = oracle.quantize_row_sums(x[r], want_bs=False)
        want = ((qa.astype(np.float64) * np.repeat(sa, 32))[None, :] * deq).sum(axis=1)
        assert (np.abs(want - got.reshape(5, n)[r]) <= 1e-3 * np.maximum(np.abs(want), 1.0)).all()


def test_strided_output_view_and_validation(oracle):
    """matmul_strided_output_view (matmul_tests.rs:141-218) for the quantized rows, plus the
    launch checks of matmul::run (mod.rs:186-247)."""
    k, n, off, batch = 64, 40, 7, 3
    for m in (2, 30):
        a = rnd(batch * m * k, 100 + m)
        w = rnd(n * k, 101 + m)
        qb = oracle.quantize(INT8, w, n, k)
        deq = oracle.dequantize(INT8, qb, n, k).astype(np.float64)
        total = off + m * batch * n + 5
        out = np.full(total, -1.0, dtype=np.float32)
        oracle.matmul(INT8, a, qb, n, k, batch=batch, m=m, out=out, out_view=(off, n, batch * n))
        want = np.full(total, -1.0)
        prod = a.reshape(batch, m, k).astype(np.float64) @ deq.T
        for bt in range(batch):
            for i in range(m):
                o = off + bt * n + i * batch * n
                want[o:o + n] = prod[bt, i]
        assert rel_err(out[want != -1.0], want[want != -1.0]) <= (2e-2 if batch * m <= 8 else 5e-3)
        assert (out[want == -1.0] == -1.0).all()
    qb = oracle.quantize(Q4_K, rnd(4 * 256, 1), 4, 256)
    a = rnd(2 * 256, 2)
    with pytest.raises(O.OracleError) as e:
        oracle.matmul(Q4_K, a, qb, 5, 256, m=2, w_shape=(4, 256))
    assert e.value.code == "shape_mismatch"
    with pytest.raises(O.OracleError) as e:
        oracle.matmul(Q4_K, a, qb, 4, 256, m=2, out=np.zeros(7, np.float32))
    assert e.value.code == "out_of_bounds"
    with pytest.raises(O.OracleError) as e:
        oracle.matmul(Q4_K, a, qb[:500], 4, 256, m=2)
    assert e.value.code == "out_of_bounds"
    out, _ = oracle.matmul(Q4_K, np.zeros(0, np.float32), qb, 4, 0, m=2, w_shape=(4, 0))
    assert out.size == 8 and not out.any()


@pytest.mark.parametrize("fmt,k", [(INT8, 96), (INT4, 96), (Q4_K, 256), (Q5_K, 256), (Q6_K, 512)])
def test_matmul_id_matches_dequantized_f64(oracle, fmt, k):
    """`matmul_id_quant` (crates/lapid-cpu/src/tests.rs:350-383) for the three formats of this path:
    5 experts of [24, k], decode-sized (int8 activations, 2e-2) and prefill-sized (exact, 1e-5) launches
    against the f64 product with the dequantized matrices, same id pattern; bad ids are refused."""
    e, n = 5, 24
    one = oracle.layout(fmt, n, k).total
    stack = np.zeros(e * one, np.uint8)
    wf = []
    for x in range(e):
        q = oracle.quantize(fmt, O.normal(9 + x, n * k, 0.1), n, k)
        stack[x * one:x * one + q.size] = q
        wf.append(oracle.dequantize(fmt, q, n, k).reshape(n, k).astype(np.float64))
    for t, r in [(1, 2), (40, 3)]:
        x = O.normal(33, t * k, 1.0).reshape(t, k)
        ids = np.array([(i * 7 + i // r) % e for i in range(t * r)], np.int32)
        want = np.stack([wf[ids[i]] @ x[i // r].astype(np.float64) for i in range(t * r)]).astype(np.float32)
        got = oracle.matmul_id(fmt, x, stack, ids, t, r, e, n, k).reshape(t * r, n)
        err = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want)
        assert err < (2e-2 if t * r <= 8 else 1e-5), (fmt, t, r, err)
    with pytest.raises(O.OracleError) as ex:
        oracle.matmul_id(fmt, x, stack, np.full(t * r, e, np.int32), t, r, e, n, k)
    assert ex.value.code == "index_out_of_range"
    assert oracle.matmul_id(fmt, x, stack, ids, 0, r, e, n, k).size == 0


def test_seeded_generator_is_counter_based():
    a = O.normal(3, 1000, 0.02)
    b = O.normal(3, 400, 0.02, start=600)
    assert np.array_equal(a[600:], b)
    assert abs(float(a.std()) - 0.02) < 0.002 and abs(float(a.mean())) < 0.003
    assert not np.array_equal(O.normal(4, 1000, 0.02), a)


# ------------------------------------------------------------------ i-quants
IQ_CASES = [("iq2_xxs", O.IQ2_XXS), ("iq2_xs", O.IQ2_XS), ("iq2_s", O.IQ2_S), ("iq3_xxs", O.IQ3_XXS)]


@pytest.mark.parametrize("name,fmt", IQ_CASES)
def test_iquant_dequantizers_match_the_reference_golden_bytes(oracle, name, fmt):
    """The reference's `iq*_matches_ggml` (crates/lapid-quant/tests/iquant_golden.rs:64-86): the blocks ggml produced
    for the fixture input dequantize to ggml's f32 bits. (Its quantizer half is not restated: no i-quant quantizer.)"""
    from tests.refgen import iq_fixture
    secs = iq_fixture(name)
    assert len(secs) == (2 if name in ("iq2_s", "iq3_xxs") else 1)
    for blocks, values in secs:
        bb = O.BLOCK_BYTES[fmt]
        for i in range(16):
            y = oracle.dequantize_block(fmt, blocks[i * bb:(i + 1) * bb])
            assert np.array_equal(y.view(np.uint32), values[i * 256:(i + 1) * 256].view(np.uint32))
        qb = np.concatenate([blocks, np.zeros((-blocks.size) % 256, np.uint8)])
        assert np.array_equal(oracle.dequantize(fmt, qb, 8, 512).reshape(-1).view(np.uint32), values.view(np.uint32))


def test_iquant_codebooks(oracle):
    """`grids_match_ggml` (iquant_golden.rs:53-62) fixes the order of the codebook file; its sign table follows the
    parity rule of crates/lapid-quant/src/iqgrid.rs:19-30, the 2-bit grids hold the levels 8, 25, 43 and the 3-bit grid
    4, 12 .. 52, 62 (iqgrid.rs:33-71). The copy the CUDA library embeds is the same file."""
    import os
    g = np.fromfile(O.IQ_GRIDS, dtype=np.uint8)
    assert g.size == 2048 + 8192 + 1024 + 128 + 4096
    assert np.array_equal(g[11264:11392], np.array([i | ((bin(i).count("1") & 1) << 7) for i in range(128)], np.uint8))
    for a, b in ((0, 2048), (2048, 10240), (11392, 15488)):
        assert set(np.unique(g[a:b])) == {8, 25, 43}
    assert set(np.unique(g[10240:11264])) == {4, 12, 20, 28, 36, 44, 52, 62}
    for a, b, w in ((0, 2048, 8), (2048, 10240, 8), (10240, 11264, 4), (11392, 15488, 8)):   # no entry twice
        assert np.unique(g[a:b].reshape(-1, w), axis=0).shape[0] == (b - a) // w
    shipped = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lapid_b200", "csrc", "iq_grids.bin")
    assert np.array_equal(np.fromfile(shipped, dtype=np.uint8), g)


@pytest.mark.parametrize("name,fmt", IQ_CASES)
def test_iquant_random_blocks_against_the_gguf_package_and_the_decode_tile(oracle, name, fmt):
    """Every byte pattern is a valid block: random blocks dequantize like the `gguf` package's independent
    dequantizer, bit for bit; the int8-activation decode tile (crates/lapid-cpu/src/iquant.rs:108-128) agrees with the
    dequantized weights times the dequantized activations (the reference's `tiles_match_dequant_reference`, :319-352);
    layout and block sizes as `layout_and_generic_quantize` (iquant_golden.rs:88-99) states them."""
    from tests.refgen import iq_matrix
    n, k = 24, 1024
    l = oracle.layout(fmt, n, k)
    assert l.qs_bytes == n * k // 256 * {"iq2_xxs": 66, "iq2_xs": 74, "iq2_s": 82, "iq3_xxs": 98}[name] and l.scales_bytes == 0
    qb = iq_matrix(fmt, n, k, 17)
    deq = oracle.dequantize(fmt, qb, n, k).reshape(n, k)
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    t = getattr(gguf.GGMLQuantizationType, name.upper())
    theirs = quants.dequantize(qb[:l.qs_bytes].reshape(n, -1), t).astype(np.float32)
    assert np.array_equal(theirs.view(np.uint32), deq.view(np.uint32))
    for m in (1, 3, 8):
        a = O.normal(18 + m, m * k).reshape(m, k)
        got, path = oracle.matmul(fmt, a, qb, n, k, m=m)
        assert path == "int8_act"
        qa = [oracle.quantize_row_sums(a[i], want_bs=False) for i in range(m)]
        adq = np.stack([q[0].astype(np.float64).reshape(-1, 32) * q[1].astype(np.float64)[:, None] for q in qa]).reshape(m, k)
        ref = adq @ deq.astype(np.float64).T
        assert np.abs(got.reshape(m, n) - ref).max() <= 1e-5 * np.abs(ref).max()
    with pytest.raises(O.OracleError):
        oracle.quantize(fmt, np.zeros(256, np.float32), 1, 256)
