"""The activation quantizer of the decode path, read back from the device and compared bit for bit.

Reference: ``quantize_row_sums`` / ``quantize_row_scalar`` (crates/lapid-cpu/src/matmul/quant.rs:30-89) and its
test ``quantize_row_roundtrip`` (:191-215). Bar: the int8 quants byte for byte, the f32 group scales ``d`` and the
sums ``d * sum(q)`` bit for bit (u32 compare), in each of the three layouts the device kernels read (planes,
336-byte records, tensor-core tiles), for 1..8 rows, against the oracle and against the frozen vectors
``qa3 / sa3 / bs3`` of tests/golden/golden.npz.
"""
import os

import numpy as np
import pytest

import lapid_b200 as lp
from lapid_b200 import quant
from lapid_b200.backend import matmul_launch
from oracle import oracle as O

pytestmark = pytest.mark.gpu

LAYOUTS = [(quant.ACT_PLANES, "planes"), (quant.ACT_RECORDS, "records"), (quant.ACT_TILES, "tiles")]


@pytest.fixture(scope="module")
def be():
    return lp.Backend(0)


def oracle_rows(oracle, x):
    qs = [oracle.quantize_row_sums(row) for row in x]
    return np.stack([q[0] for q in qs]), np.stack([q[1] for q in qs]), np.stack([q[2] for q in qs])


def same_bits(a, b):
    return np.array_equal(np.ascontiguousarray(a, np.float32).view(np.uint32), np.ascontiguousarray(b, np.float32).view(np.uint32))


def special_rows(m, k):
    """Rows with the cases the reference's arithmetic is sensitive to."""
    x = O.normal(300 + m, m * k).reshape(m, k).copy()
    x[0, 32:64] = 0.0                                   # an all-zero group: d = 0, id = 0, every q = 0
    x[0, 64:96] = 0.0
    x[0, 64] = -0.0                                     # ... with a negative zero in it
    x[m - 1, 96:128] = np.arange(32, dtype=np.float32) + 0.5   # d = 31.5/127: products near .5 boundaries
    x[m - 1, 128:160] = 0.0
    x[m - 1, 128] = 127.0                               # d = 1, id = 1: the values below are exact ties
    x[m - 1, 129:137] = [0.5, 1.5, 2.5, 3.5, -0.5, -1.5, -2.5, 126.5]   # round half to even: 0 2 2 4 -0 -2 -2 126
    x[m // 2, 160] = 1e6                                # one huge value flattens its group
    x[m // 2, 200] = 1e-30                              # a tiny one beside ordinary values
    x[0, 224:256] = 3e-39                               # a whole group of denormals
    return x


@pytest.mark.parametrize("layout,lname", LAYOUTS)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
def test_activation_quantizer_bit_exact(be, oracle, layout, lname, m):
    for k in (256, 4096):
        x = special_rows(m, k)
        q, d, bs = oracle_rows(oracle, x)
        raw = quant.quantize_activations(be, x, m, k, layout)
        gq, gd, gbs = quant.unpack_activations(layout, raw, m, k)
        assert np.array_equal(gq, q), (lname, m, k)
        assert same_bits(gd, d), (lname, m, k)
        assert same_bits(gbs, bs), (lname, m, k)
    # the ties, spelled out (crates/lapid-cpu/src/math.rs:134-136 rounds half to even)
    assert list(gq[m - 1, 129:137]) == [0, 2, 2, 4, 0, -2, -2, 126]
    assert not gq[0, 32:96].any() and not gd[0, 1:3].any()


@pytest.mark.parametrize("layout,lname", LAYOUTS)
def test_activation_quantizer_golden_vectors(be, layout, lname):
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
    k = 512
    x3 = O.normal(20, 3 * k).reshape(3, k)
    raw = quant.quantize_activations(be, x3, 3, k, layout)
    q, d, bs = quant.unpack_activations(layout, raw, 3, k)
    assert np.array_equal(q, g["qa3"])
    assert same_bits(d, g["sa3"]) and same_bits(bs, g["bs3"])


def test_activation_quantizer_reference_roundtrip(be, oracle):
    """`quantize_row_roundtrip` (quant.rs:191-215): |x - q*d| <= d/2 + ulp for every element, the all-zero group
    has scale 0, and q stays in [-127, 127]."""
    k = 1024
    x = (O.normal(9, k) * 3.0).astype(np.float32)
    x[64:96] = 0.0
    raw = quant.quantize_activations(be, x.reshape(1, k), 1, k, quant.ACT_PLANES)
    q, d, _ = quant.unpack_activations(quant.ACT_PLANES, raw, 1, k)
    rec = q[0].astype(np.float32).reshape(-1, 32) * d[0][:, None]
    assert np.all(np.abs(rec - x.reshape(-1, 32)) <= d[0][:, None] * 0.5 + 1e-6)
    assert d[0, 2] == 0.0 and np.abs(q).max() <= 127


@pytest.mark.parametrize("layout,lname", LAYOUTS)
def test_k_not_multiple_of_256_only_as_planes(be, layout, lname):
    x = O.normal(5, 2 * 96).reshape(2, 96)
    if layout == quant.ACT_PLANES:
        raw = quant.quantize_activations(be, x, 2, 96, layout)
        assert raw.size == quant.act_bytes(layout, 2, 96)
    else:
        src, dst = be.upload(x), be.alloc(4096)
        with pytest.raises(lp.LapidError) as e:
            be.quantize_activations(src, 2, 96, layout, dst)
        assert e.value.code == "invalid_launch"


@pytest.mark.parametrize("fmt", [lp.DType.Q4K, lp.DType.Q5K, lp.DType.Q6K, lp.DType.Int8])
@pytest.mark.parametrize("m", [1, 4, 8])
def test_producers_write_what_the_prepass_writes(be, oracle, fmt, m):
    """rms_norm / silu_mul with a quantized copy: the operand bytes equal those the pre-pass makes from their
    f32 result (same layout the consuming launch asks for), and a launch fed with the pre-pass's own operand
    (a_dtype ACT_Q8) gives the oracle's result."""
    n, k = 64, 2048
    launch = matmul_launch(fmt, m, n, k)
    layout, nbytes = be.act_layout(launch)
    x, res = O.normal(61, m * k), O.normal(62, m * k, 0.5)
    bx, bres = be.upload(x), be.upload(res)
    for producer in ("rms_norm", "silu_mul"):
        out, qact = be.alloc(m * k * 4), be.upload(np.zeros(nbytes, np.uint8))
        if producer == "rms_norm":
            be.rms_norm(bx, out, m, k, residual=bres, qact=qact, layout=layout)
        else:
            be.silu_mul(bx, bres, out, m * k, rows=m, qact=qact, layout=layout)
        f32 = out.download().view(np.float32).reshape(m, k)
        mine = quant.unpack_activations(layout, qact.download(), m, k)
        pre = quant.unpack_activations(layout, quant.quantize_activations(be, f32, m, k, layout), m, k)
        want = oracle_rows(oracle, f32)
        for a, b_, c in zip(mine, pre, want):
            assert np.array_equal(a.view(np.uint8), b_.view(np.uint8)) and np.array_equal(a.view(np.uint8), c.view(np.uint8)), producer
    qb = oracle.quantize(int(fmt), O.normal(63, n * k, 0.05), n, k)
    pre_op = be.upload(np.zeros(nbytes, np.uint8))   # the size act_layout asks for (padded; the operand itself is act_bytes long)
    be.quantize_activations(be.upload(x), m, k, layout, pre_op)
    outb = be.alloc(m * n * 4)
    be.execute([matmul_launch(fmt, m, n, k, inputs=(0, 1), output=2, a_quantized=True)], [pre_op, be.upload(qb), outb])
    want, _ = oracle.matmul(int(fmt), x, qb, n, k, m=m)
    got = outb.download().view(np.float32)
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    assert float((np.abs(got - want) / np.maximum(np.abs(want), rms)).max()) <= 2e-5
