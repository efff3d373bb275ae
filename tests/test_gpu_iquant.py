"""The grid-based i-quants (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS) on the GPU against the reference's golden bytes and the
CPU oracle, through the C ABI.

Bars: dequantized values, gathered rows and the exact prefill kernel bit for bit; decode (batch*m <= 8, lapid-cpu's
int8-activation arithmetic, crates/lapid-cpu/src/iquant.rs:108-128) max_rel <= 2e-5 (exact integer sums and the
reference's products; the order of the f32 additions differs).
"""
import numpy as np
import pytest

import lapid_b200 as lp
from lapid_b200 import quant
from lapid_b200.backend import gather_launch, matmul_id_launch, matmul_launch
from oracle import oracle as O
from tests.refgen import iq_fixture, iq_matrix
from tests.test_gpu_parity import max_rel, run_matmul

pytestmark = pytest.mark.gpu

IQ = [(lp.DType.Iq2Xxs, "iq2_xxs"), (lp.DType.Iq2Xs, "iq2_xs"), (lp.DType.Iq2S, "iq2_s"), (lp.DType.Iq3Xxs, "iq3_xxs")]


@pytest.fixture(scope="module")
def be():
    return lp.Backend(0)


@pytest.mark.parametrize("fmt,name", IQ)
def test_dequantize_reference_golden_bytes(be, fmt, name):
    """The blocks ggml quantized for the reference's fixture dequantize, on the device, to the very f32 bits ggml
    produced (the reference's `iq*_matches_ggml`, crates/lapid-quant/tests/iquant_golden.rs:64-86)."""
    for blocks, values in iq_fixture(name):
        qb = np.concatenate([blocks, np.zeros((-blocks.size) % 256, np.uint8)])
        got = quant.dequantize(be, fmt, qb, 8, 512).reshape(-1)
        assert np.array_equal(got.view(np.uint32), values.view(np.uint32))
        dst = quant.from_ggml_blocks(be, fmt, blocks, 8, 512)     # blocks are kept as they are
        assert np.array_equal(dst[:blocks.size], blocks) and not dst[blocks.size:].any()


@pytest.mark.parametrize("fmt,name", IQ)
def test_dequantize_and_gather_random_blocks(be, oracle, fmt, name):
    rows, cols, count = 48, 2048, 21
    qb = iq_matrix(fmt, rows, cols, 5)
    want = oracle.dequantize(int(fmt), qb, rows, cols).reshape(-1)
    got = quant.dequantize(be, fmt, qb, rows, cols).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ids = np.array([0, rows - 1, 5, 5] + list(np.random.default_rng(3).integers(0, rows, count - 4)), np.int32)
    bufs = [be.upload(qb), be.upload(ids.view(np.uint8)), be.alloc(count * cols * 4)]
    l = gather_launch(fmt, rows, cols, count)
    be.execute([l], bufs)
    got = bufs[2].download().view(np.float32).reshape(count, cols)
    assert np.array_equal(got.view(np.uint32), want.reshape(rows, cols)[ids].view(np.uint32))
    ids[3] = rows
    bufs[1].write(0, ids.view(np.uint8))
    with pytest.raises(lp.LapidError) as e:
        be.execute([l], bufs)
    assert e.value.code == "index_out_of_range"


@pytest.mark.parametrize("fmt,name", IQ)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
def test_decode_matches_oracle_all_row_counts(be, oracle, fmt, name, m):
    for (n, k, seed) in ((520, 2048, 11), (33, 768, 12), (7, 256, 13)):     # ragged rows, an odd number of blocks, one block
        qb = iq_matrix(fmt, n, k, seed)
        a = O.normal(seed + 100, m * k)
        want, path = oracle.matmul(int(fmt), a, qb, n, k, m=m)
        assert path == "int8_act"
        for rows, split in (("1", "1"), ("2", "0"), ("1", "2"), ("1", "4"), ("0", "0")):   # rows per warp, warps per row; last: the launch's own choice
            be.set_option("gemv_iq_rows", rows)
            be.set_option("gemv_iq_k_split", split)
            assert max_rel(run_matmul(be, fmt, a, qb, m, n, k), want) <= 2e-5, (n, k, rows, split)


@pytest.mark.parametrize("fmt,name", IQ)
def test_decode_fixture_blocks_bias_views_and_expression(be, oracle, fmt, name):
    """The reference's fixture blocks as an 8 x 512 weight matrix; then a bias, a strided output view and an epilogue
    expression on a benchmark-sized matrix."""
    from lapid_b200.backend import Expr, MatView
    blocks, _ = iq_fixture(name)[0]
    qb = np.concatenate([blocks, np.zeros((-blocks.size) % 256, np.uint8)])
    a = O.normal(31, 4 * 512)
    want, _ = oracle.matmul(int(fmt), a, qb, 8, 512, m=4)
    assert max_rel(run_matmul(be, fmt, a, qb, 4, 8, 512), want) <= 2e-5
    m, n, k = 3, 4096, 4096
    qb = iq_matrix(fmt, n, k, 41)
    a, bias = O.normal(42, m * k), O.normal(43, n)
    want, _ = oracle.matmul(int(fmt), a, qb, n, k, m=m, bias=bias)
    assert max_rel(run_matmul(be, fmt, a, qb, m, n, k, bias=bias), want) <= 2e-5
    out = np.full(5 + m * (n + 9), 7.0, np.float32)
    got = run_matmul(be, fmt, a, qb, m, n, k, out=out, out_view=MatView(5, 0, n + 9))
    ref = out.copy()
    acc, _ = oracle.matmul(int(fmt), a, qb, n, k, m=m)
    for i in range(m):
        ref[5 + i * (n + 9):5 + i * (n + 9) + n] = acc.reshape(m, n)[i]
    assert max_rel(got, ref) <= 2e-5 and np.array_equal(got[ref == 7.0], ref[ref == 7.0])
    x = (O.normal(44, m * n) * 0.5 + 0.7).astype(np.float32)
    e = Expr.silu(Expr.load(0)) * Expr.load(1)
    bufs = [be.upload(a), be.upload(qb), be.alloc(m * n * 4), be.upload(x)]
    be.execute([matmul_launch(fmt, m, n, k, expr=e, extra_input=3)], bufs)
    want = O.epilogue(e.words, acc.reshape(m, n), x.reshape(m, n)).reshape(-1)
    assert max_rel(bufs[2].download().view(np.float32), want) <= 2e-5


@pytest.mark.parametrize("fmt,name", IQ)
def test_prefill_exact_kernel_bit_exact(be, oracle, fmt, name):
    """batch*m > 8: f32 activations times dequantized weights, accumulated in k order with fused multiply-adds
    (crates/lapid-cpu/src/matmul/qdeq.rs): bit-identical to the oracle."""
    for (m, n, k, seed) in ((12, 24, 512, 51), (70, 130, 1024, 52), (9, 64, 256, 53)):
        qb = iq_matrix(fmt, n, k, seed)
        a = O.normal(seed + 100, m * k)
        want, path = oracle.matmul(int(fmt), a, qb, n, k, m=m)
        assert path == "f32_act"
        got = run_matmul(be, fmt, a, qb, m, n, k)
        assert np.array_equal(got.view(np.uint32), want.reshape(-1).view(np.uint32))


def _expert_stack(oracle, fmt, e, n, k, seed):
    one = oracle.layout(int(fmt), n, k).total
    stack = np.zeros(e * one, np.uint8)
    for x in range(e):
        q = iq_matrix(fmt, n, k, seed + x)
        stack[x * one:x * one + q.size] = q
    return stack


@pytest.mark.parametrize("fmt,name", IQ)
@pytest.mark.parametrize("t,r,e,n,k", [(1, 2, 5, 24, 512), (3, 2, 4, 64, 256), (8, 8, 16, 96, 2048), (40, 3, 5, 24, 512), (70, 2, 4, 200, 256)])
def test_matmul_id(be, oracle, fmt, name, t, r, e, n, k):
    """Kernel::MatMulId (crates/lapid-cpu/src/moe.rs:80-118): int8-activation GEMVs per (token, slot) pair for
    t <= 8, float activations above (bit-identical to the oracle's per-expert f32 matmul)."""
    stack = _expert_stack(oracle, fmt, e, n, k, 60)
    x = O.normal(70, t * k, 1.0)
    ids = np.array([(i * 7 + i // r) % e for i in range(t * r)], np.int32)
    want = oracle.matmul_id(int(fmt), x, stack, ids, t, r, e, n, k)
    bufs = [be.upload(x), be.upload(stack), be.upload(ids.view(np.uint8)), be.alloc(t * r * n * 4)]
    l = matmul_id_launch(fmt, t, r, e, n, k)
    be.execute([l], bufs)
    got = bufs[3].download().view(np.float32).reshape(t, r, n)
    if t <= 8:
        assert max_rel(got, want) <= 2e-5
    else:
        assert np.array_equal(got.reshape(-1).view(np.uint32), want.reshape(-1).view(np.uint32))
    bad = ids.copy()
    bad[-1] = e
    bufs[2].write(0, bad.view(np.uint8))
    with pytest.raises(lp.LapidError) as err:
        be.execute([l], bufs)
    assert err.value.code == "index_out_of_range"


def test_quantize_is_refused_and_gguf_tensors_load(be, oracle, tmp_path):
    """No i-quant quantizer is built (`unsupported`); tensors of a GGUF file written by the `gguf` package load with
    their blocks kept and multiply like the same bytes handed over directly."""
    with pytest.raises(lp.LapidError) as err:
        quant.quantize(be, quant.Format.Iq2Xxs, O.normal(1, 512), 2, 256)
    assert err.value.code == "unsupported"
    gguf = pytest.importorskip("gguf")
    from lapid_b200.gguf import GgufFile
    path = str(tmp_path / "iq.gguf")
    w = gguf.GGUFWriter(path, "llama")
    mats = {}
    for fmt, name in IQ:
        n, k = 40, 1024
        raw = iq_matrix(fmt, n, k, 80 + int(fmt), pad=False)
        mats[name] = (fmt, n, k, raw)
        w.add_tensor(name, raw.reshape(n, -1), raw_dtype=getattr(gguf.GGMLQuantizationType, name.upper()))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    f = GgufFile(path)
    for name, (fmt, n, k, raw) in mats.items():
        buf, dtype, shape = f.load(be, name)
        assert dtype == fmt and tuple(shape) == (n, k)
        assert np.array_equal(buf.download()[:raw.size], raw)
        a = O.normal(90, 2 * k)
        out = be.alloc(2 * n * 4)
        be.execute([matmul_launch(fmt, 2, n, k)], [be.upload(a), buf, out])
        qb = np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])
        want, _ = oracle.matmul(int(fmt), a, qb, n, k, m=2)
        assert max_rel(out.download().view(np.float32), want) <= 2e-5
