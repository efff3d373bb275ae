"""Tensor-parallel host logic on CPU: shard/repack of lapid-quant matrices, "sum of shards = unsharded
result", and a two-rank layer over the gloo backend with the oracle as the per-rank matmul."""
import os
import socket

import numpy as np
import pytest

from lapid_b200 import tp
from oracle import oracle as O

FMTS = [O.INT8, O.Q4_K, O.Q6_K]
MORE = [O.INT4, O.Q5_K, O.MXFP4, O.IQ2_XXS, O.IQ2_XS, O.IQ2_S, O.IQ3_XXS]   # the formats beyond the benchmark's three


@pytest.mark.parametrize("fmt", MORE)
@pytest.mark.parametrize("world", [2, 4])
def test_shards_of_the_other_formats(oracle, fmt, world):
    """Every quantized format shards the same way: a column-parallel shard dequantizes to the rows, a row-parallel
    shard to the columns of the unsharded matrix, bit for bit, and has the size the layout gives; the partial results of
    the row-parallel shards add up to the unsharded result."""
    from tests.refgen import iq_matrix
    n, k = 24, 2048
    q = iq_matrix(fmt, n, k, 40 + fmt) if fmt in O.IQUANTS else oracle.quantize(fmt, O.normal(5 + fmt, n * k, 0.02), n, k)
    full = oracle.dequantize(fmt, q, n, k).reshape(n, k)
    a = O.normal(60 + fmt, 3 * k).reshape(3, k)
    want, _ = oracle.matmul(fmt, a, q, n, k, m=3)
    total = np.zeros(3 * n, np.float32)
    for rank in range(world):
        qs, nl = tp.shard_rows(fmt, q, n, k, rank, world)
        assert nl == n // world and qs.size == oracle.layout(fmt, nl, k).total == tp.layout_total(fmt, nl, k)
        assert np.array_equal(oracle.dequantize(fmt, qs, nl, k).reshape(nl, k).view(np.uint32), full[rank * nl:(rank + 1) * nl].view(np.uint32))
        qc, kl = tp.shard_cols(fmt, q, n, k, rank, world)
        assert kl == k // world and qc.size == oracle.layout(fmt, n, kl).total
        assert np.array_equal(oracle.dequantize(fmt, qc, n, kl).reshape(n, kl).view(np.uint32),
                              np.ascontiguousarray(full[:, rank * kl:(rank + 1) * kl]).view(np.uint32))
        total += oracle.matmul(fmt, np.ascontiguousarray(a[:, rank * kl:(rank + 1) * kl]), qc, n, kl, m=3)[0]
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    assert (np.abs(total - want) / np.maximum(np.abs(want), rms)).max() <= 1e-5
    with pytest.raises(ValueError):
        tp.shard_cols(fmt, q, n, k, 0, 128)
    with pytest.raises(ValueError):
        tp.layout_total(3, n, k)      # not a quantized format


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("world", [2, 4])
def test_shards_are_bit_identical_block_subsets(oracle, fmt, world):
    n, k = 24, 2048
    q = oracle.quantize(fmt, O.normal(5 + fmt, n * k, 0.02), n, k)
    full = oracle.dequantize(fmt, q, n, k)
    for rank in range(world):
        qs, nl = tp.shard_rows(fmt, q, n, k, rank, world)
        assert nl == n // world and qs.size == oracle.layout(fmt, nl, k).total == tp.layout_total(fmt, nl, k)
        assert np.array_equal(oracle.dequantize(fmt, qs, nl, k).view(np.uint32), full[rank * nl:(rank + 1) * nl].view(np.uint32))
        qc, kl = tp.shard_cols(fmt, q, n, k, rank, world)
        assert kl == k // world and qc.size == oracle.layout(fmt, n, kl).total
        assert np.array_equal(oracle.dequantize(fmt, qc, n, kl).view(np.uint32),
                              np.ascontiguousarray(full[:, rank * kl:(rank + 1) * kl]).view(np.uint32))
        # what the repack must equal: quantizing the slice directly gives the same bytes for block-local formats
        direct = oracle.quantize(fmt, np.ascontiguousarray(full[:, rank * kl:(rank + 1) * kl]) * 0 +
                                 np.ascontiguousarray(O.normal(5 + fmt, n * k, 0.02).reshape(n, k)[:, rank * kl:(rank + 1) * kl]), n, kl)
        assert np.array_equal(direct, qc)
    with pytest.raises(ValueError):
        tp.shard_cols(fmt, q, n, k, 0, 16 if fmt != O.INT8 else 128)
    with pytest.raises(ValueError):
        tp.shard_rows(fmt, q, n, k, 0, 5)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m", [1, 4, 12])
def test_sum_of_row_parallel_partials_is_the_unsharded_result(oracle, fmt, m):
    n, k, world = 40, 1024, 4
    q = oracle.quantize(fmt, O.normal(9, n * k, 0.02), n, k)
    a = O.normal(10 + m, m * k).reshape(m, k)
    want, _ = oracle.matmul(fmt, a, q, n, k, m=m)
    total = np.zeros(m * n, np.float32)
    for rank in range(world):
        qc, kl = tp.shard_cols(fmt, q, n, k, rank, world)
        part, _ = oracle.matmul(fmt, np.ascontiguousarray(a[:, rank * kl:(rank + 1) * kl]), qc, n, kl, m=m)
        total += part
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    assert (np.abs(total - want) / np.maximum(np.abs(want), rms)).max() <= 1e-5
    # column-parallel: concatenating the shards' outputs is exact
    cols = []
    for rank in range(world):
        qs, nl = tp.shard_rows(fmt, q, n, k, rank, world)
        cols.append(oracle.matmul(fmt, a, qs, nl, k, m=m)[0].reshape(m, nl))
    assert np.array_equal(np.concatenate(cols, axis=1).reshape(-1), want)


def test_q4km_mix_rule():
    picks = [i for i in range(32) if tp.use_more_bits(i, 32)]
    assert len(picks) == 16 and picks[:5] == [0, 1, 2, 3, 6] and picks[-4:] == [28, 29, 30, 31]
    assert sum(tp.use_more_bits(i, 80) for i in range(80)) == 40
    assert tp.q4km_format("v", 7, 32) == tp.Q6_K and tp.q4km_format("q", 0, 32) == tp.Q4_K
    assert tp.q4km_format("down", 0, 32) == tp.Q6_K and tp.q4km_format("down", 4, 32) == tp.Q4_K
    # byte counts quoted for the 8B and 70B stacks (projections only, no output head)
    def stack_bytes(shape, layers):
        return sum(tp.layout_total(tp.q4km_format(nm, i, layers), n, k) for i in range(layers) for nm, n, k, _ in shape.projections())
    assert stack_bytes(tp.LLAMA3_8B, 32) + tp.layout_total(tp.Q6_K, 128256, 4096) == 4_633_632_768
    assert stack_bytes(tp.LLAMA_70B, 80) == 41_098_936_320


SHAPE = tp.LayerShape(512, 4, 2, 128, 1024)


def _layer_weights(o, rank, world):
    w, f = {}, {}
    for i, (name, n, k, kind) in enumerate(SHAPE.projections()):
        fmt = tp.q4km_format(name, 0, 8) if name != "k" else O.INT8  # all three formats in one layer
        full = o.quantize(fmt, O.normal(60 + i, n * k, 0.05), n, k)
        w[name] = (tp.shard_rows if kind == "column" else tp.shard_cols)(fmt, full, n, k, rank, world)[0]
        f[name] = fmt
    return w, f


def _run_layer(o, rank, world, all_reduce, m):
    w, f = _layer_weights(o, rank, world)

    def mm(fmt, x, wq, n, k):
        return o.matmul(fmt, np.ascontiguousarray(x, np.float32), wq, n, k, m=m)[0].reshape(m, n)

    layer = tp.TpLayer(SHAPE, w, f, world, mm, all_reduce, tp.NumpyOps)
    h = O.normal(77, m * SHAPE.d_model).reshape(m, SHAPE.d_model)
    return layer.forward(h)


def _worker(rank, world, port, m, out_path):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = O.load()
        o.set_num_threads(1)

        def all_reduce(t):
            tt = torch.from_numpy(t)
            dist.all_reduce(tt)

        # q's sharded output is o's k shard only if both use the same column range: true by construction
        out = _run_layer(o, rank, world, all_reduce, m)
        if rank == 0:
            np.save(out_path, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [1, 12])
def test_two_rank_layer_over_gloo_matches_single_rank(tmp_path, oracle, m):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "out.npy")
    mp.spawn(_worker, args=(2, port, m, out_path), nprocs=2, join=True)
    got = np.load(out_path)
    want = _run_layer(oracle, 0, 1, lambda t: None, m)
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    err = float((np.abs(got - want) / np.maximum(np.abs(want), rms)).max())
    # M = 1: int8 activations are quantized per 32-group on both sides, only the f32 sum order differs;
    # the sharded silu(gate)*up input of `down` is elementwise identical to the unsharded one
    assert err <= 1e-5, err
