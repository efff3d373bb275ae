"""The benchmark's configurations at their full sizes against the CPU oracle, through the C ABI, on a B200.

  config 2  decode sweep: the four Llama-3-8B-shaped projections, M in {1, 2, 4, 8}, every format; once more as
            launch lists whose later members run ahead of their predecessors (activations quantized at the head)
  config 3  prefill: Q4_K / Q6_K 14336 x 4096 and 4096 x 14336 at M in {64, 512, 2048} on the tensor cores against
            the ORACLE's f32 path on weight-row slices (128 weight rows are a contiguous byte range of the
            quantized matrix, so the oracle runs the same launch on the slice alone)
  config 4  one 8B-shaped layer in the Q4_K_M-style mix plus the 128256 x 4096 Q6_K output head, M = 1 and 8,
            every launch of the chain against the oracle on the input that launch actually read

Bars: decode max_rel <= 2e-5 (stated bound 1e-3); prefill rel_l2 <= 4e-3 and max_rel <= 2e-2 (bf16 operands).
Weights are quantized on the device; that its bytes are the oracle's is checked here on slices and in
test_gpu_parity.py (test_quantize_byte_exact, test_config1_full_size_matvec) on whole matrices.
"""
import numpy as np
import pytest

import lapid_b200 as lp
from lapid_b200 import quant, tp
from lapid_b200.backend import matmul_launch
from oracle import oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]
FMTS = [(lp.DType.Int8, "int8"), (lp.DType.Int4, "int4"), (lp.DType.Q4K, "q4_k"), (lp.DType.Q5K, "q5_k"), (lp.DType.Q6K, "q6_k"),
        (lp.DType.MXFP4, "mxfp4")]
BLOCK_BYTES = {lp.DType.Q4K: 144, lp.DType.Q5K: 176, lp.DType.Q6K: 210}


@pytest.fixture(scope="module")
def be():
    return lp.Backend(0)


@pytest.fixture(scope="module")
def fast():
    """The oracle's -O3 OpenMP build: same arithmetic for the integer decode path; the f32 path differs from
    the strict build only in summation details far below the bounds used here."""
    return O.load(fast=True)


def max_rel(got, ref):
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = np.sqrt((ref ** 2).mean())
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), max(rms, 1e-30))).max())


def rel_l2(got, ref):
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.sqrt(((got - ref) ** 2).sum() / max((ref ** 2).sum(), 1e-30)))


_weights, _quantized = {}, {}


def source_weights(si):
    """N(0, 0.02) weights of shape SHAPES[si] from seed 100 + si (generated once per session: the generator is slow)."""
    if si not in _weights:
        n, k = SHAPES[si]
        _weights[si] = O.normal(100 + si, n * k, 0.02)
    return _weights[si]


def quantized_weights(be, fmt, si):
    if (int(fmt), si) not in _quantized:
        n, k = SHAPES[si]
        _quantized[(int(fmt), si)] = quant.quantize(be, fmt, source_weights(si), n, k)
    return _quantized[(int(fmt), si)]


def device_quantized(be, fmt, n, k, seed):
    """Random N(0, 0.02) weights made and quantized on the device; returns (device buffer, host bytes)."""
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    w = torch.randn(n * k, device="cuda", generator=g) * 0.02
    out = torch.empty(quant.layout(fmt, n, k).total, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    be.quantize_into(fmt, be.wrap_tensor(w), n, k, be.wrap_tensor(out))
    return be.wrap_tensor(out), out.cpu().numpy(), w


def row_slice(fmt, qb, k, j0, rows):
    """The quantized bytes of weight rows [j0, j0 + rows) of a K-format matrix, padded like a matrix of its own."""
    rb = k // 256 * BLOCK_BYTES[fmt]
    part = qb[j0 * rb:(j0 + rows) * rb]
    return np.concatenate([part, np.zeros((-part.size) % 256, np.uint8)])


# ------------------------------------------------------------------------------------------ config 2
@pytest.mark.parametrize("fmt,name", FMTS)
def test_config2_every_batch_size(be, oracle, fast, fmt, name):
    for si, (n, k) in enumerate(SHAPES):
        qb = quantized_weights(be, fmt, si)
        wbuf = be.upload(qb)
        for m in (1, 2, 4, 8):
            x = O.normal(200 + m, m * k)
            want, path = fast.matmul(int(fmt), x, qb, n, k, m=m)
            assert path == "int8_act"
            if m == 2 and si == 0:  # the fast build against the strict one, once per format
                strict, _ = oracle.matmul(int(fmt), x, qb, n, k, m=m)
                assert max_rel(want, strict) <= 2e-6
            out = be.alloc(m * n * 4)
            be.execute([matmul_launch(fmt, m, n, k)], [be.upload(x), wbuf, out])
            got = out.download().view(np.float32)
            assert max_rel(got, want) <= 1e-3, (name, n, k, m)
            assert max_rel(got, want) <= 2e-5, (name, n, k, m, max_rel(got, want))


@pytest.mark.parametrize("fmt,name", [(lp.DType.Q4K, "q4_k"), (lp.DType.Q5K, "q5_k"), (lp.DType.Q6K, "q6_k"), (lp.DType.Int8, "int8")])
def test_config2_lists_that_run_ahead(be, fast, fmt, name):
    """Four launches per list on the same activations (quantized once, at the head of the list) into four
    output buffers: from the second launch on the kernels compute before the kernel in front has finished."""
    for si, (n, k) in enumerate(SHAPES):
        qb = quantized_weights(be, fmt, si)
        wbuf = be.upload(qb)
        for m in (1, 2, 4, 8):
            x = O.normal(200 + m, m * k)
            want, _ = fast.matmul(int(fmt), x, qb, n, k, m=m)
            bufs = [be.upload(x), wbuf] + [be.alloc(m * n * 4) for _ in range(4)]
            be.take_launch_count()
            be.execute([matmul_launch(fmt, m, n, k, inputs=(0, 1), output=2 + c) for c in range(4)], bufs)
            assert be.take_launch_count() <= 5   # one pre-pass, then at most one kernel per launch
            for c in range(4):
                got = bufs[2 + c].download().view(np.float32)
                assert max_rel(got, want) <= 2e-5, (name, n, k, m, c, max_rel(got, want))


# ------------------------------------------------------------------------------------------ config 3
@pytest.mark.parametrize("fmt,ofmt", [(lp.DType.Q4K, O.Q4_K), (lp.DType.Q6K, O.Q6_K)])
def test_config3_prefill_against_the_oracle_on_row_slices(be, oracle, fast, fmt, ofmt):
    for si in (2, 3):
        n, k = SHAPES[si]
        wsrc = source_weights(si)
        qb = quantized_weights(be, fmt, si)
        # first tile, a middle tile off the tile grid, and a ragged tail (the last 100 rows)
        slices = [(0, 128), (n // 2 + 64, 128), (n - 100, 100)]
        for (j0, rows) in slices[:1]:  # the device quantizer's bytes are the oracle's on the slice
            rb = k // 256 * BLOCK_BYTES[fmt]
            assert np.array_equal(qb[j0 * rb:(j0 + rows) * rb], oracle.quantize(ofmt, wsrc[j0 * k:(j0 + rows) * k], rows, k)[:rows * rb])
        wbuf = be.upload(qb)
        for m in (64, 512, 2048):
            a = O.normal(300 + m, m * k)
            out = be.alloc(m * n * 4)
            be.execute([matmul_launch(fmt, m, n, k)], [be.upload(a), wbuf, out])
            got = out.download().view(np.float32).reshape(m, n)
            for (j0, rows) in (slices if m < 2048 else slices[1:]):
                want, path = fast.matmul(ofmt, a, row_slice(fmt, qb, k, j0, rows), rows, k, m=m)
                assert path == "f32_act"
                g = got[:, j0:j0 + rows]
                assert rel_l2(g, want) <= 4e-3, (n, k, m, j0, rel_l2(g, want))
                assert max_rel(g, want) <= 2e-2, (n, k, m, j0, max_rel(g, want))


def test_config3_exact_kernel_against_the_oracle_on_a_slice(be, oracle):
    """The exact-f32 kernel at a full prefill size: bit-identical to the strict oracle on a row slice."""
    n, k, m = 14336, 4096, 64
    qb = quantized_weights(be, lp.DType.Q4K, 2)
    a = O.normal(364, m * k)
    out = be.alloc(m * n * 4)
    be.set_option("gemm", "f32")
    try:
        be.execute([matmul_launch(lp.DType.Q4K, m, n, k)], [be.upload(a), be.upload(qb), out])
    finally:
        be.set_option("gemm", "tc")
    got = out.download().view(np.float32).reshape(m, n)
    j0, rows = n - 72, 72
    want, _ = oracle.matmul(O.Q4_K, a, row_slice(lp.DType.Q4K, qb, k, j0, rows), rows, k, m=m, fma=True)
    assert np.array_equal(np.ascontiguousarray(got[:, j0:]).view(np.uint32), want.reshape(m, rows).view(np.uint32))


# ------------------------------------------------------------------------------------------ config 4
@pytest.mark.parametrize("m", [1, 8])
def test_config4_layer_and_output_head(be, fast, m):
    shape, n_layers, vocab = tp.LLAMA3_8B, 32, 128256
    d = shape.d_model
    for layer in (0, 5):   # a `use_more_bits` layer (Q6_K ffn_down) and one without
        dims = {name: (n, k) for name, n, k, _ in shape.projections()}
        fmts = {name: tp.q4km_format(name, layer, n_layers) for name in dims}
        assert fmts["v"] == tp.Q6_K and fmts["q"] == tp.Q4_K and (fmts["down"] == tp.Q6_K) == (layer == 0)
        bufs, host = [], {}

        def add(b):
            bufs.append(b)
            return len(bufs) - 1

        x = add(be.upload(O.normal(500 + m, m * d)))
        wid, oid = {}, {}
        for j, name in enumerate(dims):
            wb, wh, _ = device_quantized(be, fmts[name], *dims[name], seed=4000 + 8 * layer + j)
            wid[name], host[name] = add(wb), wh
            oid[name] = add(be.alloc(m * dims[name][0] * 4))
        src = {"q": x, "k": x, "v": x, "o": oid["q"], "gate": oid["o"], "up": oid["o"], "down": oid["gate"]}
        order = ("q", "k", "v", "o", "gate", "up", "down")
        launches = [matmul_launch(fmts[nm], m, *dims[nm], inputs=(src[nm], wid[nm]), output=oid[nm]) for nm in order]
        be.prepare(launches)
        be.execute(launches, bufs)
        for nm in order:
            n, k = dims[nm]
            a_in = bufs[src[nm]].download().view(np.float32)[:m * k]   # what this launch read
            want, path = fast.matmul(fmts[nm], a_in, host[nm], n, k, m=m)
            got = bufs[oid[nm]].download().view(np.float32)
            assert path == "int8_act" and max_rel(got, want) <= 2e-5, (layer, nm, m, max_rel(got, want))
    # the output head: 128256 x 4096, Q6_K
    wb, wh, _ = device_quantized(be, tp.Q6_K, vocab, d, seed=4999)
    xh = O.normal(600 + m, m * d)
    out = be.alloc(m * vocab * 4)
    be.execute([matmul_launch(tp.Q6_K, m, vocab, d)], [be.upload(xh), wb, out])
    want, _ = fast.matmul(tp.Q6_K, xh, wh, vocab, d, m=m)
    got = out.download().view(np.float32)
    assert max_rel(got, want) <= 2e-5, ("head", m, max_rel(got, want))
