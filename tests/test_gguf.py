"""GGUF tensor-table reader (lapid_b200/gguf.py) on files written with the third-party ``gguf`` package.

CPU part: container parsing (metadata of every value type, tensor table, alignment, row-major shapes, raw bytes)
and its error cases. GPU part (-m gpu): tensors go from the file into lapid-quant layout on the device --
K-quant blocks kept, Q8_0 / Q4_0 repacked -- and dequantize to exactly what the oracle gives for the same blocks
(crates/lapid-convert/src/gguf.rs:177-215, crates/lapid-quant/src/imp.rs:171-200); a decode launch on a loaded
tensor matches the oracle; a 3-D tensor loads as an expert stack that a MatMulId launch reads.
"""
import os
import struct

import numpy as np
import pytest

from oracle import oracle as O

BLOCK = {O.Q4_K: 144, O.Q5_K: 176, O.Q6_K: 210}


def _write(path, oracle, with_experts=False):
    gguf = pytest.importorskip("gguf")
    from gguf import GGMLQuantizationType as T
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.block_count", 2)
    w.add_float32("llama.rope.freq_base", 10000.0)
    w.add_string("general.name", "tiny test model")
    w.add_bool("general.flag", True)
    w.add_array("tokenizer.scores", [0.5, -1.25, 2.0])
    w.add_array("tokenizer.tokens", ["a", "bc", "def"])
    tensors = {}
    rows, cols = 24, 512
    for i, (name, fmt, t) in enumerate([("blk.0.attn_q.weight", O.Q4_K, T.Q4_K), ("blk.0.attn_v.weight", O.Q6_K, T.Q6_K),
                                        ("blk.0.ffn_up.weight", O.Q5_K, T.Q5_K)]):
        src = O.normal(600 + i, rows * cols, 0.05)
        q = oracle.quantize(fmt, src, rows, cols)
        blocks = q[:rows * (cols // 256) * BLOCK[fmt]]
        w.add_tensor(name, blocks.reshape(rows, -1), raw_dtype=t)
        tensors[name] = (fmt, rows, cols, q)
    # Q8_0 / Q4_0: GGUF's array-of-structs blocks, built from the oracle's plane layout
    for name, fmt, t, payload, blk in (("blk.1.attn_k.weight", O.INT8, T.Q8_0, 32, 34), ("blk.1.attn_o.weight", O.INT4, T.Q4_0, 16, 18)):
        src = O.normal(610 + fmt, rows * cols, 0.7)
        q = oracle.quantize(fmt, src, rows, cols)
        l = oracle.layout(fmt, rows, cols)
        ng = rows * cols // 32
        aos = np.empty((ng, blk), np.uint8)
        aos[:, :2] = q[l.scales_offset:l.scales_offset + 2 * ng].reshape(ng, 2)
        aos[:, 2:] = q[:ng * payload].reshape(ng, payload)
        w.add_tensor(name, aos.reshape(rows, -1), raw_dtype=t)
        tensors[name] = (fmt, rows, cols, q)
    norm = O.normal(620, cols)
    w.add_tensor("blk.0.attn_norm.weight", norm)
    tensors["blk.0.attn_norm.weight"] = (None, 1, cols, norm)
    if with_experts:
        e, n, k = 3, 16, 256
        stack, per = [], []
        for x in range(e):
            q = oracle.quantize(O.Q4_K, O.normal(630 + x, n * k, 0.05), n, k)
            stack.append(q)
            per.append(q[:n * (k // 256) * 144].reshape(n, -1))
        w.add_tensor("blk.0.ffn_gate_exps.weight", np.stack(per), raw_dtype=T.Q4_K)
        tensors["blk.0.ffn_gate_exps.weight"] = (O.Q4_K, (e, n, k), None, np.concatenate(stack))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return tensors


def test_tensor_table_and_metadata(tmp_path, oracle):
    from lapid_b200 import gguf as G
    path = str(tmp_path / "tiny.gguf")
    tensors = _write(path, oracle, with_experts=True)
    with G.GgufFile(path) as f:
        assert f.version == 3 and f.architecture() == "llama"
        assert f.metadata["llama.block_count"] == 2 and f.metadata["general.name"] == "tiny test model"
        assert f.metadata["general.flag"] is True and abs(f.metadata["llama.rope.freq_base"] - 10000.0) < 1e-6
        assert f.metadata["tokenizer.scores"] == [0.5, -1.25, 2.0] and f.metadata["tokenizer.tokens"] == ["a", "bc", "def"]
        assert {t.name for t in f.tensors} == set(tensors)
        assert f.data_offset % f.alignment == 0
        t = f.tensor("blk.0.attn_q.weight")
        assert t.shape == (24, 512) and t.type_name == "Q4_K" and t.nbytes == 24 * 2 * 144 and t.offset % 32 == 0
        q = tensors["blk.0.attn_q.weight"][3]
        assert np.array_equal(f.tensor_data(t), q[:t.nbytes])          # K-quant blocks are kept byte for byte
        t = f.tensor("blk.0.ffn_gate_exps.weight")
        assert t.shape == (3, 16, 256) and t.nbytes == 3 * 16 * 144
        t = f.tensor("blk.0.attn_norm.weight")
        assert t.type_name == "F32" and t.shape == (512,)
        assert np.array_equal(f.tensor_data(t).view(np.float32), tensors["blk.0.attn_norm.weight"][3])
        assert f.tensor("nope") is None


def test_malformed_files(tmp_path, oracle):
    from lapid_b200 import gguf as G
    path = str(tmp_path / "tiny.gguf")
    _write(path, oracle)
    raw = open(path, "rb").read()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + raw[4:])
    with pytest.raises(G.GgufError) as e:
        G.GgufFile(str(bad))
    assert e.value.code == "invalid_gguf"
    bad.write_bytes(raw[:4] + struct.pack("<I", 7) + raw[8:])
    with pytest.raises(G.GgufError) as e:
        G.GgufFile(str(bad))
    assert e.value.code == "unsupported_gguf_version"
    bad.write_bytes(raw[:len(raw) - 1000])                              # tensor data cut off
    with pytest.raises(G.GgufError) as e:
        G.GgufFile(str(bad))
    assert e.value.code == "invalid_gguf"
    bad.write_bytes(raw[:40])                                           # header cut off
    with pytest.raises(G.GgufError):
        G.GgufFile(str(bad))


@pytest.mark.gpu
def test_tensors_load_into_lapid_layout_on_the_device(tmp_path, oracle):
    import lapid_b200 as lp
    from lapid_b200 import gguf as G, quant
    from lapid_b200.backend import matmul_id_launch, matmul_launch
    path = str(tmp_path / "tiny.gguf")
    tensors = _write(path, oracle, with_experts=True)
    be = lp.Backend(0)
    with G.GgufFile(path) as f:
        for name, (fmt, rows, cols, q) in tensors.items():
            buf, dtype, shape = f.load(be, name)
            if fmt is None:
                assert dtype == lp.DType.F32 and np.array_equal(buf.download().view(np.float32), q)
                continue
            if isinstance(rows, tuple):
                continue
            assert int(dtype) == fmt and shape == (rows, cols)
            assert np.array_equal(buf.download(), q)                    # the layout lapid-quant itself would hold
            deq = be.alloc(rows * cols * 4)
            be.dequantize_into(dtype, buf, rows, cols, deq)
            want = oracle.dequantize(fmt, q, rows, cols)
            assert np.array_equal(deq.download().view(np.uint32), want.view(np.uint32).reshape(-1))
            x = O.normal(640, 2 * cols)
            out = be.alloc(2 * rows * 4)
            be.execute([matmul_launch(dtype, 2, rows, cols)], [be.upload(x), buf, out])
            y, _ = oracle.matmul(fmt, x, q, rows, cols, m=2)
            got = out.download().view(np.float32)
            rms = float(np.sqrt((y.astype(np.float64) ** 2).mean()))
            assert float((np.abs(got - y) / np.maximum(np.abs(y), rms)).max()) <= 2e-5
        # the expert stack: MatMulId over the loaded tensor
        fmt, (e, n, k), _, stack = tensors["blk.0.ffn_gate_exps.weight"]
        buf, dtype, shape = f.load(be, "blk.0.ffn_gate_exps.weight")
        assert shape == (e, n, k) and np.array_equal(buf.download(), stack)
        t, r = 2, 2
        x = O.normal(650, t * k)
        ids = np.array([[0, 2], [1, 0]], np.int32)
        out = be.alloc(t * r * n * 4)
        be.execute([matmul_id_launch(dtype, t, r, e, n, k)], [be.upload(x), buf, be.upload(ids), out])
        want = oracle.matmul_id(fmt, x, stack, ids, t, r, e, n, k)
        got = out.download().view(np.float32).reshape(t, r, n)
        rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
        assert float((np.abs(got - want) / np.maximum(np.abs(want), rms)).max()) <= 2e-5
        with pytest.raises(G.GgufError) as err:
            f.load(be, "missing")
        assert err.value.code == "not_found"
