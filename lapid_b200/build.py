"""Builds ``liblapid_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python -m lapid_b200.build``. nvcc cross-compiles without a GPU. The objects land in
``lapid_b200/csrc/build/`` and the library beside this file, so it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "liblapid_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# per-file extras: the bit-exact files must never fuse multiply-adds
SOURCES = {
    "dequant.cu": ["-fmad=false"],
    "quantize.cu": ["-fmad=false"],
    "actquant.cu": ["-fmad=false"],
    "qgemv.cu": [],
    "qgemv_q4k.cu": [],
    "qgemv_q4k_mma.cu": [],
    "qgemv_kq_stream.cu": [],
    "qgemv_q6k_mma.cu": [],
    "qgemv_i8.cu": [],
    "qgemv_i4.cu": [],
    "qgemv_mxfp4.cu": [],
    "qgemv_mxfp4_mma.cu": [],
    "qgemv_iq.cu": [],
    "iquant.cu": ["-DLAPID_B200_IQ_GRIDS_FILE=" + os.path.join(CSRC, "iq_grids.bin")],
    "qgemv_i8_mma.cu": [],
    "qgemv_i4_mma.cu": [],
    "qgemm_f32.cu": [],
    "qgemm_tc.cu": [],
    "noalloc.cu": [],
    "glue.cu": [],
    "moe.cu": [],
    "tp_allreduce.cu": [],
    "backend.cc": ["-x", "cu"],
}


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    bdir = os.path.join(CSRC, "build")
    os.makedirs(bdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "lapid_b200.h"))
    headers.append(os.path.abspath(__file__))
    headers.append(os.path.join(CSRC, "iq_grids.bin"))  # embedded by iquant.cu
    jobs = []
    objs = []
    for src, extra in SOURCES.items():
        s = os.path.join(CSRC, src)
        o = os.path.join(bdir, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc(), *ARCH, *COMMON, *extra, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for out in ex.map(run, jobs):
            if verbose and out:
                print(out, file=sys.stderr)
    if force or jobs or _stale(OUT, objs):
        cmd = [nvcc(), *ARCH, "-shared", "-o", OUT, *objs, "-Xcompiler", "-fvisibility=hidden"]
        run(cmd)
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
