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
