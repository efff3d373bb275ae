"""Two GPU ranks over NCCL: the sharded layer stack must give the unsharded stack's result
(stated bar: max_rel <= 1e-5 at batch 1, where only f32 summation order differs)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPE_ARGS = (1024, 8, 2, 128, 2048)


def _build(be, tp, O, quant, torch, rank, world, dev, n_sets):
    shape = tp.LayerShape(*SHAPE_ARGS)
    weights, formats = [], []
    for s in range(n_sets):
        w, f = {}, {}
        for i, (name, n, k, kind) in enumerate(shape.projections()):
            fmt = tp.q4km_format(name, s, 2) if name != "k" else tp.INT8
            full = torch.from_numpy(quant.quantize(be, fmt, O.normal(300 + 10 * s + i, n * k, 0.04), n, k)).to(dev)
            w[name] = (tp.shard_rows if kind == "column" else tp.shard_cols)(fmt, full, n, k, rank, world)[0]
            f[name] = fmt
        weights.append(w)
        formats.append(f)
    return shape, weights, formats


def _worker(rank, world, port, m, out_path, peer):
    import torch
    import torch.distributed as dist
    import lapid_b200 as lp
    from lapid_b200 import quant, tp
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        be = lp.Backend(rank)
        stream = torch.cuda.Stream(device=dev)
        be.set_stream(stream.cuda_stream)
        results = []
        reducer = tp.PeerAllReduce(be, rank, world, dev) if peer else None
        if peer:
            # the fused hand-off (GEMV epilogue pushes, rms_norm sums) adds the same numbers in the same
            # order as the stand-alone all-reduce kernel: the residual stream must match bit for bit
            shape, weights, formats = _build(be, tp, O, quant, torch, rank, world, dev, 2)
            outs = []
            for fused, fuse_act in ((False, False), (True, False), (True, True), (False, True)):
                layers = tp.GpuTpLayers(be, shape, world, rank, m, weights, formats, peer_all_reduce=reducer, fused=fused,
                                        fuse_act=fuse_act)
                assert layers.fused == fused
                layers.h.copy_(torch.from_numpy(O.normal(99, m * shape.d_model).reshape(m, -1)).to(dev))
                torch.cuda.synchronize(dev)
                with torch.cuda.stream(stream):
                    out = layers.token(4).clone()
                stream.synchronize()
                outs.append(out)
                be.synchronize()
            assert all(torch.equal(outs[0], o_) for o_ in outs[1:])
        for w_ in ((world, rank), (1, 0)):
            shape, weights, formats = _build(be, tp, O, quant, torch, w_[1], w_[0], dev, 2)
            layers = tp.GpuTpLayers(be, shape, w_[0], w_[1], m, weights, formats, peer_all_reduce=reducer)
            layers.h.copy_(torch.from_numpy(O.normal(99, m * shape.d_model).reshape(m, -1)).to(dev))
            torch.cuda.synchronize(dev)
            with torch.cuda.stream(stream):
                out = layers.token(1)
            stream.synchronize()
            first_o = layers.outs["o"].cpu().numpy().copy()  # first all-reduced row-parallel output
            with torch.cuda.stream(stream):
                layers.h.copy_(out)
                out = layers.token(3)
            stream.synchronize()
            results.append(np.concatenate([first_o.reshape(-1), out.cpu().numpy().reshape(-1)]))
        if peer:  # the one-shot all-reduce gives every rank the same bits
            mine = torch.from_numpy(results[0]).to(dev)
            other = mine.clone()
            dist.broadcast(other, src=0)
            assert torch.equal(mine, other)
        if rank == 0:
            np.save(out_path, np.stack(results))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [1, 2, 4])
def test_layer_stack_with_activations_quantized_by_their_producers(m):
    """One GPU: the layer stack whose rms_norm / silu_mul kernels also write the quantized operand of the
    projections that follow gives the same residual stream, bit for bit, as the stack with a pre-pass
    kernel in front of every projection group, with fewer kernels."""
    import torch
    import lapid_b200 as lp
    from lapid_b200 import quant, tp
    from oracle import oracle as O
    dev = torch.device("cuda", 0)
    be = lp.Backend(0)
    be.set_option("early_acts", "0")   # both stacks on the same decode kernels (two-row Q4_K launches would differ otherwise)
    stream = torch.cuda.Stream(device=dev)
    be.set_stream(stream.cuda_stream)
    shape, weights, formats = _build(be, tp, O, quant, torch, 0, 1, dev, 2)
    outs, kernels = [], []
    for fuse_act in (False, True):
        layers = tp.GpuTpLayers(be, shape, 1, 0, m, weights, formats, fuse_act=fuse_act)
        layers.h.copy_(torch.from_numpy(O.normal(99, m * shape.d_model).reshape(m, -1)).to(dev))
        torch.cuda.synchronize(dev)
        be.take_launch_count()
        with torch.cuda.stream(stream):
            out = layers.token(4).clone()
        stream.synchronize()
        be.synchronize()
        kernels.append(be.take_launch_count())
        outs.append(out)
        assert any(l is not None for ls in layers.act_layouts for l in ls) == fuse_act
    assert torch.isfinite(outs[0]).all() and torch.equal(outs[0], outs[1])
    assert kernels[1] <= kernels[0] - 4 * 2      # at least the gate/up and down pre-passes of every layer are gone


@pytest.mark.parametrize("peer", [False, True])
@pytest.mark.parametrize("m", [1, 4])
def test_two_gpu_layer_stack_matches_one_gpu(tmp_path, m, peer):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "out.npy")
    mp.spawn(_worker, args=(2, port, m, out_path, peer), nprocs=2, join=True)
    sharded, single = np.load(out_path)
    n_o = m * SHAPE_ARGS[0]

    def max_rel(a, b):
        rms = float(np.sqrt((b.astype(np.float64) ** 2).mean()))
        return float((np.abs(a - b) / np.maximum(np.abs(b), rms)).max())

    # the first row-parallel result has identical inputs on both sides: only the f32 sum order differs
    assert max_rel(sharded[:n_o], single[:n_o]) <= 1e-5
    # after several layers the ~1e-7 differences pass through the int8 activation quantizer of later
    # projections, where a value sitting on a rounding boundary may land on the other side. One such
    # step (amax/127 of one element) moves every output of that projection by about
    # (3/127)/sqrt(k) of its rms: 1e-3 at this test's k = 512 (6e-5 at k = 8192), and a handful of
    # them add up over four layers. A wrong shard or a lost partial would be an O(1) error.
    diff = (sharded[n_o:] - single[n_o:]).astype(np.float64)
    assert np.sqrt((diff ** 2).sum() / (single[n_o:].astype(np.float64) ** 2).sum()) <= 1e-2
    assert max_rel(sharded[n_o:], single[n_o:]) <= 3e-2


def test_two_devices_in_one_process():
    """Per-device kernel settings (the dynamic shared-memory opt-in) are made on every device a
    process uses: the same launches on GPU 0 and then GPU 1 of one process give the same bits."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import lapid_b200 as lp
    from lapid_b200.backend import matmul_launch
    from oracle import oracle as O
    o = O.load()
    outs = []
    for ordinal in (0, 1):
        be = lp.Backend(ordinal)
        res = []
        for fmt, ofmt in ((lp.DType.Q4K, O.Q4_K), (lp.DType.Q6K, O.Q6_K), (lp.DType.Int8, O.INT8)):
            n, k = 300, 2048
            qb = o.quantize(ofmt, O.normal(int(fmt), n * k, 0.05), n, k)
            for m in (1, 4, 40):
                a = O.normal(60 + m, m * k)
                bufs = [be.upload(a), be.upload(qb), be.alloc(m * n * 4)]
                be.execute([matmul_launch(fmt, m, n, k)], bufs)
                res.append(bufs[2].download().view(np.float32).copy())
        outs.append(res)
        be.close()
    for a, b in zip(*outs):
        assert np.array_equal(a, b)
