"""Regenerates ``tests/golden/golden.npz`` from the CPU oracle (``python tests/golden/make_golden.py``).

The reference cannot be built in this environment (no Rust toolchain) and checks in no golden
bytes for the K formats, so these vectors are outputs of the oracle restatement, itself pinned by
the reference's known-answer and property tests (tests/test_oracle.py). They freeze those
outputs: any later change of the oracle or of the CUDA path that moves a byte shows up here.

Contents, per format f in (int8, q4_k, q5_k, q6_k), with W = normal(seed 10+f, [24, 512], 0.02),
X3 = normal(seed 20, [3, 512]), X12 = normal(seed 21, [12, 512]):
  w_<f>     quantized bytes of W             (lapid_quant::quantize)
  deq_<f>   f32 bits of dequantize(w)        (lapid_quant::dequantize), as uint32
  y3_<f>    matmul(X3, w)  -- int8-activation decode path (batch*m <= 8)
  y12_<f>   matmul(X12, w) -- f32 path with fused multiply-add accumulation
plus the activation quantizer's output for X3: qa3 (int8), sa3 (f32 scales), bs3 (f32 sums).

``tests/golden/iquant/`` is different: those files are golden bytes the reference itself holds for the grid-based
i-quants (``crates/lapid-quant/tests/fixtures/iquant/``: blocks quantized and values dequantized by ggml, and the
codebook file ``grids.bin``; made by the reference's ``tools/iquant_golden/gen.sh`` from the llama.cpp commit its
``SOURCE`` file names). ``python tests/golden/make_golden.py --iquant <reference checkout>`` copies them byte for byte
(``input.bin``, the quantizers' input, is not used here: the i-quant quantizers are not restated) and refreshes the
copy of ``grids.bin`` the CUDA library embeds (``lapid_b200/csrc/iq_grids.bin``).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

N, K = 24, 512


def copy_iquant_fixtures(reference: str) -> None:
    import shutil
    src = os.path.join(reference, "crates", "lapid-quant", "tests", "fixtures", "iquant")
    dst = os.path.join(ROOT, "tests", "golden", "iquant")
    os.makedirs(dst, exist_ok=True)
    for name in ("grids.bin", "iq2_xxs.bin", "iq2_xs.bin", "iq2_s.bin", "iq3_xxs.bin"):
        shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
    shutil.copyfile(os.path.join(src, "grids.bin"), os.path.join(ROOT, "lapid_b200", "csrc", "iq_grids.bin"))
    print("copied the i-quant fixtures from", src)


def main():
    if len(sys.argv) >= 3 and sys.argv[1] == "--iquant":
        copy_iquant_fixtures(sys.argv[2])
        return
    o = O.load()
    out = {}
    x3 = O.normal(20, 3 * K).reshape(3, K)
    x12 = O.normal(21, 12 * K).reshape(12, K)
    qs = [o.quantize_row_sums(x3[r]) for r in range(3)]
    out["qa3"] = np.stack([q[0] for q in qs])
    out["sa3"] = np.stack([q[1] for q in qs])
    out["bs3"] = np.stack([q[2] for q in qs])
    for name, fmt in O.FORMATS.items():
        w = O.normal(10 + fmt, N * K, 0.02)
        qb = o.quantize(fmt, w, N, K)
        out[f"w_{name}"] = qb
        out[f"deq_{name}"] = o.dequantize(fmt, qb, N, K).view(np.uint32)
        y3, p3 = o.matmul(fmt, x3, qb, N, K, m=3)
        y12, p12 = o.matmul(fmt, x12, qb, N, K, m=12, fma=True)
        assert (p3, p12) == ("int8_act", "f32_act")
        out[f"y3_{name}"] = y3.reshape(3, N)
        out[f"y12_{name}"] = y12.reshape(12, N)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
