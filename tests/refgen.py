"""Input generators of the reference's own tests, restated so that the ported tests feed the
oracle and the CUDA path the same values the reference's tests use.

* ``noise``  -- crates/lapid-quant/src/imp.rs:262-273 and src/kquant.rs:402-413 (xorshift64, seed.max(1))
* ``rnd``    -- crates/lapid-cpu/src/matmul/matmul_tests.rs:13-23 (seed * golden ratio | 1)
* ``make_blocks`` -- crates/lapid-cpu/src/kquant.rs:334-358 (xorshift32 bytes, fixed f16 d / dmin)
"""
import numpy as np

M64 = (1 << 64) - 1


def _xs64(s):
    s ^= (s << 13) & M64
    s ^= s >> 7
    s ^= (s << 17) & M64
    return s


def noise(n, seed, scale=1.0):
    s = max(seed, 1)
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = _xs64(s)
        v = np.float32(s >> 40) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0)
        out[i] = v * np.float32(scale)
    return out


def rnd(n, seed):
    s = ((seed * 0x9E3779B97F4A7C15) & M64) | 1
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = _xs64(s)
        out[i] = np.float32(s >> 40) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0)
    return out


def make_blocks(fmt_bytes, n_blocks, seed, d_off, dmin_off=None):
    """Pseudo-random block bytes with finite scales: d = f16(0.01), dmin = f16(0.004)."""
    v = np.empty(n_blocks * fmt_bytes, dtype=np.uint8)
    s = max(seed, 1)
    for i in range(v.size):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        v[i] = (s >> 8) & 0xFF
    d = np.array([0.01], dtype=np.float16).view(np.uint8)
    dm = np.array([0.004], dtype=np.float16).view(np.uint8)
    b = v.reshape(n_blocks, fmt_bytes)
    b[:, d_off:d_off + 2] = d
    if dmin_off is not None:
        b[:, dmin_off:dmin_off + 2] = dm
    return v


IQ_BLOCK_BYTES = {10: 66, 11: 82, 12: 98, 13: 74}   # IQ2_XXS, IQ2_S, IQ3_XXS, IQ2_XS by lapid dtype code


def iq_matrix(fmt, rows, cols, seed, pad=True):
    """Random i-quant blocks for a [rows, cols] matrix: every bit pattern of the index, sign and scale fields is a
    valid block, so the bytes are uniform; the f16 super-block scales cycle through magnitudes from 6e-8 (a denormal)
    to 7, both signs. The result is padded to the 256-byte multiple of ``layout(..).total``."""
    bb = IQ_BLOCK_BYTES[int(fmt)]
    nb = rows * cols // 256
    raw = np.random.default_rng(seed).integers(0, 256, nb * bb, dtype=np.uint8)
    ds = np.array([0.01, 0.25, 3e-5, -0.02, 6e-8, 1.5, 0.003, 7.0, 0.0], np.float16).view(np.uint8).reshape(-1, 2)
    b = raw.reshape(nb, bb)
    b[:, 0:2] = ds[np.arange(nb) % ds.shape[0]]
    if not pad:
        return raw
    return np.concatenate([raw, np.zeros((-raw.size) % 256, np.uint8)])


def iq_fixture(name):
    """The reference's golden file for one i-quant (crates/lapid-quant/tests/fixtures/iquant/<name>.bin, read by
    tests/iquant_golden.rs:36-52): sections of (block bytes of an 8 x 512 matrix quantized by ggml, the f32 values ggml
    dequantizes them to). Returns a list of (blocks u8, values f32)."""
    import os
    bb = {"iq2_xxs": 66, "iq2_xs": 74, "iq2_s": 82, "iq3_xxs": 98}[name]
    f = np.fromfile(os.path.join(os.path.dirname(__file__), "golden", "iquant", name + ".bin"), dtype=np.uint8)
    qn = 16 * bb
    sec = qn + 4 * 4096
    assert f.size % sec == 0
    return [(f[i * sec:i * sec + qn].copy(), f[i * sec + qn:(i + 1) * sec].copy().view(np.float32)) for i in range(f.size // sec)]
