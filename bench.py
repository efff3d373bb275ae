#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (``config.workload = "decode_gemv_sweep"``): the decode GEMV sweep over
Llama-3-8B-shaped projections -- (N x K) in {4096x4096, 1024x4096, 14336x4096, 4096x14336},
batch M in {1, 2, 4, 8}, Q4_K weights -- 16 launches per step, each over its own weight copy
(311 MB of weights per step, 2.5x the L2, so every launch streams from HBM). Inputs are synthetic:
weights N(0, 0.02) quantized on the device by the library's own quantizer, activations N(0, 1).

  value        GB/s of algorithmic bytes (weights + 4MK + 4MN per GEMV) with everything resident
               in HBM; the step is one CUDA-graph replay of the 16 launches
  e2e          the same bytes through the C-ABI `execute` call with host buffers: one `write` of
               the activations from pinned memory, one `execute` (16 launches, waits), one
               `download` of the outputs -- per step, inside the timed region
  roofline     for the decode kernel with the larger share of the time (the sweep runs the dp4a
               kernel at M = 1 and the int8 tensor-core kernel at M >= 2): algorithmic bytes per
               launch / mean launch time over its cases, against the measured HBM copy bandwidth
  cpu_baseline the oracle's restatement of lapid-cpu's path, timed on this host's cores
  cases        per (format, shape, M) GB/s, each timed alone over cold weight copies

``--impl reference`` times the CPU restatement of lapid-cpu's path (the reference itself is Rust
and cannot be built where no Rust toolchain exists) on the same workload.
With --gpus N (torchrun, one rank per GPU) every rank streams its own copy of the sweep (the
column-parallel case: independent weight shards, no collective) -> weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096, "q/o"), (1024, 4096, "k/v"), (14336, 4096, "gate/up"), (4096, 14336, "down")]
MS = [1, 2, 4, 8]
FMT_NAMES = {4: "int8", 5: "int4", 6: "q4_k", 7: "q5_k", 8: "q6_k", 9: "mxfp4", 10: "iq2_xxs", 11: "iq2_s", 12: "iq3_xxs", 13: "iq2_xs"}
AOS_BLOCK = {6: (256, 144), 7: (256, 176), 8: (256, 210), 9: (32, 17), 10: (256, 66), 11: (256, 82), 12: (256, 98), 13: (256, 74)}


def weight_bytes(fmt: int, n: int, k: int) -> int:
    if fmt in AOS_BLOCK:
        b = n * k // AOS_BLOCK[fmt][0] * AOS_BLOCK[fmt][1]
    elif fmt == 5:
        b = (n * k // 2 + 255) // 256 * 256 + n * k // 32 * 2
    else:
        b = (n * k + 255) // 256 * 256 + n * k // 32 * 2
    return (b + 255) // 256 * 256


def algo_bytes(fmt: int, m: int, n: int, k: int) -> int:
    return weight_bytes(fmt, n, k) + 4 * m * k + 4 * m * n


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.nv or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        seen = set()
        for _, r in self.samples:
            for n, bit in names.items():
                if r & bit:
                    seen.add(n)
        mhz = sorted(s[0] for s in self.samples)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(seen), "samples": len(mhz)}


# ---------------------------------------------------------------------------------------------
def cpu_threads() -> int:
    """The host cores this process may use (a launcher may have set OMP_NUM_THREADS=1 for its workers)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def cpu_sweep(o, fmt, budget_s: float, max_steps: int, warm: int):
    """The oracle's timed copy of lapid-cpu's decode path over the 16-GEMV sweep on this host's cores. Every
    launch of a step has its own weight copy (16 matrices, 311 MB per step, cycled like the GPU arm's), so the
    last-level cache does not serve the weights. Returns (GB/s, ms per step, steps, cores)."""
    o.set_num_threads(cpu_threads())
    rng = np.random.default_rng(0)
    cases = [(m, n, k) for m in MS for (n, k, _) in SHAPES]
    base = {(n, k): o.quantize(fmt, rng.standard_normal(n * k, dtype=np.float32) * np.float32(0.02), n, k) for (n, k, _) in SHAPES}
    ws = [base[(n, k)].copy() for (m, n, k) in cases]   # distinct memory per launch
    xs = {(m, kk): rng.standard_normal(m * kk, dtype=np.float32) for m in MS for kk in (4096, 14336)}
    step_bytes = sum(algo_bytes(fmt, m, n, k) for (m, n, k) in cases)

    def step():
        for w, (m, n, k) in zip(ws, cases):
            o.matmul(fmt, xs[(m, k)], w, n, k, m=m)

    for _ in range(max(1, warm)):
        step()
    t0 = time.perf_counter()
    done = 0
    while done < max_steps:
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    return step_bytes / dt / 1e9, dt * 1e3, done, o.num_threads()


def run_reference(args, rank: int, world: int):
    """CPU arm: the oracle's restatement of lapid-cpu's decode path on the same 16 GEMVs, all host cores."""
    if rank != 0:
        return
    from oracle import oracle as O
    o = O.load(fast=True)
    fmt = 6
    val, ms, done, cores = cpu_sweep(o, fmt, budget_s=120.0, max_steps=max(1, args.steps), warm=min(max(args.warmup, 1), 3))
    cases = [(m, n, k) for m in MS for (n, k, _) in SHAPES]
    line = {
        "impl": "reference", "metric": "q4k_decode_gemv_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x q4_k -> f32", "data": "synthetic",
        "config": {"workload": "decode_gemv_sweep", "format": "q4_k", "shapes": [[n, k] for (n, k, _) in SHAPES],
                   "batch_m": MS, "launches_per_step": len(cases)},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{done} full steps of the 16-GEMV sweep, one weight copy per launch (311 MB per step, no reuse inside a step)"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "C restatement of lapid-cpu's int8-activation decode path (the Rust reference cannot be built here); "
                "gcc -O3 -march=native, OpenMP over output columns on every core this process may use"
                + (f"; ONE CPU copy of the sweep: a run on {args.gpus} GPUs streams {args.gpus} copies at once" if args.gpus > 1 else ""),
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    import lapid_b200 as lp
    from lapid_b200.backend import MatView, matmul_launch

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    be = lp.Backend(local_rank)
    for kv in list(filter(None, os.environ.get("LAPID_B200_OPTS", "").split(","))) + list(args.opt):  # e.g. "pdl=0,gemv=generic"
        key, _, val = kv.partition("=")
        be.set_option(key, val)
    stream = torch.cuda.Stream(device=dev)
    be.set_stream(stream.cuda_stream)
    peak, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()

    def quantized(fmt, n, k, seed):
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        if fmt >= 10:   # the i-quants have no quantizer here; every byte pattern is a valid block: random blocks, d = f16 0.01
            out = torch.zeros(weight_bytes(fmt, n, k), dtype=torch.uint8, device=dev)
            blocks = torch.randint(0, 256, (n * k // 256, AOS_BLOCK[fmt][1]), dtype=torch.uint8, device=dev, generator=g)
            blocks[:, 0] = 0x1F
            blocks[:, 1] = 0x21
            out[:blocks.numel()] = blocks.reshape(-1)
            torch.cuda.synchronize()
            return out
        w = torch.randn(n * k, device=dev, generator=g) * 0.02
        out = torch.empty(weight_bytes(fmt, n, k), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        be.quantize_into(fmt, be.wrap_tensor(w), n, k, be.wrap_tensor(out))
        return out

    fmt = 6
    cases = [(m, n, k) for m in MS for (n, k, _) in SHAPES]  # layer order: the projections of one batch size follow each other
    base = {(n, k): quantized(fmt, n, k, 100 + i) for i, (n, k, _) in enumerate(SHAPES)}
    # one distinct weight copy per launch; packed activations and outputs
    a_off, o_off, ao, oo = [], [], 0, 0
    for (m, n, k) in cases:
        a_off.append(ao)
        o_off.append(oo)
        ao += m * k
        oo += m * n
    g = torch.Generator(device=dev)
    g.manual_seed(200)
    acts = torch.randn(ao, device=dev, generator=g)
    outs = torch.zeros(oo, device=dev)
    wcopies = [base[(n, k)].clone() for (m, n, k) in cases]
    torch.cuda.synchronize()
    bufs = [be.wrap_tensor(acts), be.wrap_tensor(outs)] + [be.wrap_tensor(w) for w in wcopies]
    launches = []
    for i, (m, n, k) in enumerate(cases):
        l = matmul_launch(fmt, m, n, k, inputs=(0, 2 + i), output=1, out=MatView(o_off[i], m * n, n))
        import dataclasses as dc
        l = dc.replace(l, dims=dc.replace(l.dims, a=MatView(a_off[i], m * k, k)))
        launches.append(l)
    be.prepare(launches)
    step_bytes = sum(algo_bytes(fmt, m, n, k) for (m, n, k) in cases)
    run = be.packed(launches, bufs)

    # ---- device-resident timing: one CUDA graph replay per step
    be.take_launch_count()
    with torch.cuda.stream(stream):
        run()
    stream.synchronize()
    launches_per_step = be.take_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        be.set_stream(torch.cuda.current_stream().cuda_stream)
        run()
    be.set_stream(stream.cuda_stream)
    be.take_launch_count()

    sampler = ClockSampler(local_rank)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        stream.synchronize()
        barrier()
        sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        ev1.record(stream)
        stream.synchronize()
        ms_total = ev0.elapsed_time(ev1)
        # keep the same load running briefly so the clock sampler sees the GPU under this load
        t_end = time.perf_counter() + 0.4
        while time.perf_counter() < t_end:
            for _ in range(50):
                graph.replay()
            stream.synchronize()
        sampler.stop()
    barrier()
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end through the C ABI with host buffers
    be.set_stream(0)  # the device's own stream: execute() waits on it
    h_acts = torch.randn(ao).pin_memory()
    h_out = torch.empty(oo).pin_memory()
    e2e_bufs = [be.alloc(ao * 4), be.alloc(oo * 4)] + bufs[2:]
    arr, cb = be._pack(launches, e2e_bufs)
    from lapid_b200 import _lib
    lib = _lib.lib()

    def three_calls():   # Backend::write, execute, read one after the other
        be.write_ptr(e2e_bufs[0], 0, h_acts.data_ptr(), ao * 4)
        _lib.check(lib.lapid_b200_execute(be._h, arr, len(launches), cb, len(e2e_bufs)))
        be.download_ptr(e2e_bufs[1], h_out.data_ptr(), oo * 4)

    # the same step as ONE call of the public API: every launch's activations are a write tied to that launch, its
    # output a read tied to it; the library overlaps uploads, launches and downloads chunk by chunk
    io_writes = [(0, a_off[i] * 4, h_acts.data_ptr() + a_off[i] * 4, m * k * 4, i) for i, (m, n, k) in enumerate(cases)]
    io_reads = [(1, o_off[i] * 4, h_out.data_ptr() + o_off[i] * 4, m * n * 4, i) for i, (m, n, k) in enumerate(cases)]
    e2e_step = be.packed_io(launches, e2e_bufs, io_writes, io_reads, args.e2e_chunk)

    def timed(fn, steps):
        for _ in range(3):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        return (time.perf_counter() - t0) / steps

    e_steps = max(args.steps, 1)
    three_s = timed(three_calls, e_steps)
    h_out.zero_()
    e2e_s = timed(e2e_step, e_steps)
    if world > 1:
        t = torch.tensor([e2e_s, three_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, three_s = float(t[0].item()), float(t[1].item())
    e2e_val = world * step_bytes / e2e_s / 1e9
    be.set_stream(stream.cuda_stream)

    # ---- outside the timed regions: every launch of the sweep against the CPU oracle (resident path: the
    #      outputs of the last graph replay; end-to-end path: what the last download brought back)
    check = None
    if rank == 0 and not args.no_check:
        try:
            stream.synchronize()
            check = {"sweep": check_sweep(fmt, cases, base, acts.cpu().numpy(), outs.cpu().numpy(), a_off, o_off),
                     "e2e": check_sweep(fmt, cases, base, h_acts.numpy(), h_out.numpy(), a_off, o_off),
                     "bar": "max_rel = max|got - ref| / max(|ref|, rms(ref)) against the CPU oracle's int8-activation path; "
                            "decode bar 1e-3 (tests assert 2e-5); prefill (bf16 operands) rel_l2 <= 4e-3"}
        except Exception as e:
            check = {"error": f"{type(e).__name__}: {e}"[:300]}

    # ---- 70B-shaped layer stack, tensor-parallel over the ranks (all ranks take part)
    tp_obj = None
    if not args.no_tp:
        try:
            tp_obj = measure_tp70b(be, stream, dev, rank, world, quantized, check=not args.no_check)
        except Exception as e:  # reported, never fatal for the headline line
            tp_obj = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank != 0:
        return

    prefill_rows = None
    if world == 1 and not args.no_prefill:
        prefill_rows = measure_prefill(be, stream, dev, base, quantized, check=not args.no_check)
    stack_obj = None
    if world == 1 and not args.no_stack:
        try:
            stack_obj = measure_stack8b(be, stream, dev, quantized, peak, check=not args.no_check)
        except Exception as e:  # reported, never fatal for the headline line
            stack_obj = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()

    moe_rows = None
    if world == 1 and not args.no_moe:
        try:
            moe_rows = measure_moe(be, stream, dev, quantized, peak)
        except Exception as e:  # reported, never fatal for the headline line
            moe_rows = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()

    # ---- per-case timing over cold copies (rank 0, N = 1 only): the kbench method scaled to B200's L2
    case_rows = []
    roof = None
    roof_kernel, roof_traffic, roof_detail = None, None, None
    if world == 1 and not args.no_cases:
        POOL = 512 << 20
        for f in (6, 8, 4, 7, 5, 9, 10, 12):   # Q4_K, Q6_K, Int8 (the benchmark's formats), then Q5_K, Int4, MXFP4, IQ2_XXS, IQ3_XXS
            for si, (n, k, tag) in enumerate(SHAPES):
                wq = base[(n, k)] if f == 6 else quantized(f, n, k, 300 + si)
                wb = wq.numel()
                copies = max(2, min(256, -(-POOL // wb)))
                pool = wq.repeat(copies).view(copies, wb)
                for m in MS:
                    a = torch.randn(m * k, device=dev)
                    o = torch.zeros(m * n, device=dev)
                    torch.cuda.synchronize()
                    cb_ = [be.wrap_tensor(a), be.wrap_tensor(o)] + [be.wrap_tensor(pool[c]) for c in range(copies)]
                    ls = [matmul_launch(f, m, n, k, inputs=(0, 2 + c), output=1) for c in range(copies)]
                    be.prepare(ls)
                    rn = be.packed(ls[:1], cb_)
                    with torch.cuda.stream(stream):
                        rn()  # first use of a kernel variant sets its attributes: keep that out of the capture
                    stream.synchronize()
                    rn = be.packed(ls, cb_)
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=stream):
                        be.set_stream(torch.cuda.current_stream().cuda_stream)
                        rn()
                    be.set_stream(stream.cuda_stream)
                    with torch.cuda.stream(stream):
                        for _ in range(3):
                            gr.replay()
                        times = []
                        for _ in range(7):
                            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                            e0.record(stream)
                            gr.replay()
                            e1.record(stream)
                            stream.synchronize()
                            times.append(e0.elapsed_time(e1) / copies)
                    times.sort()
                    us = times[len(times) // 2] * 1e3
                    gbs = algo_bytes(f, m, n, k) / (us * 1e-6) / 1e9
                    case_rows.append({"fmt": FMT_NAMES[f], "n": n, "k": k, "m": m, "us": round(us, 3),
                                      "gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "kernel": gemv_kernel_name(f, m, n, k)})
                    del gr, rn, cb_, ls
                del pool
                torch.cuda.empty_cache()
        # the sweep runs two GEMV kernels (by row count); the roofline is that of the one with the
        # larger share of the time, the other is listed beside it
        q4 = [r for r in case_rows if r["fmt"] == "q4_k"]
        by_kernel = {}
        for r in q4:
            e = by_kernel.setdefault(r["kernel"], {"bytes": 0, "us": 0.0, "launches": 0})
            e["bytes"] += algo_bytes(6, r["m"], r["n"], r["k"])
            e["us"] += r["us"]
            e["launches"] += 1
        roof_kernel = max(by_kernel, key=lambda kname: by_kernel[kname]["us"])
        e = by_kernel[roof_kernel]
        roof = e["bytes"] / (e["us"] * 1e-6) / 1e9
        ratio = DRAM_TRAFFIC_RATIO.get(roof_kernel)
        roof_traffic = ratio * e["bytes"] / e["launches"] if ratio is not None else None
        roof_detail = [{"kernel": kname, "launches": v["launches"], "us": round(v["us"], 2),
                        "achieved": round(v["bytes"] / (v["us"] * 1e-6) / 1e9, 1),
                        "frac": round(v["bytes"] / (v["us"] * 1e-6) / 1e9 / peak, 4)} for kname, v in by_kernel.items()]

        # the north star's own case, one row on the large shapes, listed beside the aggregates
        for r in q4:
            if r["m"] == 1 and r["n"] * r["k"] >= 4096 * 14336:
                roof_detail.append({"kernel": r["kernel"], "case": f"M=1 {r['n']}x{r['k']}", "launches": 1, "us": r["us"],
                                    "achieved": r["gbs"], "frac": r["frac"]})

    achieved = roof if roof is not None else value / world
    line = {
        "metric": "q4k_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / published_baseline()) if published_baseline() else None, "dtype": "int8 x q4_k -> f32", "data": "synthetic",
        "config": {"workload": "decode_gemv_sweep", "format": "q4_k", "shapes": [[n, k] for (n, k, _) in SHAPES],
                   "batch_m": MS, "launches_per_step": len(cases), "weight_bytes_per_step": sum(w.numel() for w in wcopies),
                   "l2": "every launch has its own weight copy; 311 MB per step > 126 MB L2", "cuda_graph": True,
                   "parallelism": f"replicas x{world} (column-parallel shards, no collective)" if world > 1 else "single"},
        "clocks": sampler.summary(),
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": ao * 4, "d2h_bytes_per_step": oo * 4,
                "ms_per_step": e2e_s * 1e3,
                "calls_per_step": "one execute_io: 16 writes, 16 launches in " + (f"chunks of {args.e2e_chunk}" if args.e2e_chunk else "three chunks of about equal transfer bytes (the library's choice)") + ", 16 reads (a chunk's adjacent transfers go as one copy; "
                                  "uploads, launches and downloads of different chunks overlap); waits",
                "three_calls": {"value": world * step_bytes / three_s / 1e9, "ms_per_step": three_s * 1e3,
                                "calls_per_step": "write + execute(16 launches, waits) + download, one after the other"}},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": roof_traffic, "peak_kind": peak_kind, "kernel": roof_kernel, "by_kernel": roof_detail,
                     "what": "Q4_K decode launches of the kernel with the larger time share (act-quant pre-pass included): "
                             "algorithmic bytes / mean launch time over its cases; traffic is MODELLED, not measured in this run: "
                             "mean algorithmic bytes per launch x the DRAM-bytes / algorithmic-bytes ratio of the ncu capture "
                             "summarised under profiles/ (null when that kernel has no capture)"},
    }
    if world > 1 and isinstance(tp_obj, dict) and "decode_b1" in tp_obj:
        line["config"]["tp70b"] = {"decode_tok_s": tp_obj["decode_b1"]["tok_s"],
                                   "decode_frac_of_hbm_ceiling": tp_obj["decode_b1"].get("frac_of_hbm_ceiling"),
                                   "prefill_m512_tok_s": tp_obj.get("prefill_m512", {}).get("tok_s"),
                                   "prefill_collective_share": tp_obj.get("prefill_m512", {}).get("collective_share"),
                                   "note": "the headline value is a communication-free replica run; the tensor-parallel stack "
                                           "with real exchanges is this object (details under tp70b)"}
    if case_rows:
        line["cases"] = case_rows
    if prefill_rows:
        line["prefill"] = prefill_rows
    if stack_obj:
        line["stack8b"] = stack_obj
    if moe_rows:
        line["matmul_id"] = moe_rows
    if tp_obj:
        line["tp70b"] = tp_obj
    if check is not None:
        if prefill_rows:
            check["prefill"] = [r["check"] for r in prefill_rows if "check" in r]
        if isinstance(stack_obj, dict) and "check" in stack_obj:
            check["stack8b"] = stack_obj["check"]
        if isinstance(tp_obj, dict) and "check" in tp_obj:
            check["tp70b"] = tp_obj["check"]
        decode = [check[kk]["max_rel"] for kk in ("sweep", "e2e", "stack8b") if isinstance(check.get(kk), dict) and "max_rel" in check[kk]]
        check["decode_worst_max_rel"] = max(decode) if decode else None
        check["prefill_worst_rel_l2"] = max([c["rel_l2"] for c in check.get("prefill", [])], default=None)
        line["check"] = check
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(cases, fmt)
    print(json.dumps(line), flush=True)


def gemv_kernel_name(fmt: int, m: int, n: int = 0, k: int = 0) -> str:
    """The kernel a decode launch of `m` rows takes with the library's default options when, as in the per-case
    timing, its activations were quantized at the head of the launch list (so it may run ahead of its predecessor)."""
    units = -(-n // 128) * -(-(k // 256) // 2)   # 128-row x 512-k units of the balanced-stream kernel
    if fmt == 6:
        if m >= 2:
            return "qgemv_kq_stream_kernel<q4_k>" if units >= 2 * 148 else "qgemv_q4k_mma_kernel"
        return "qgemv_kq_fast_kernel<q4_k>"
    small = m <= 4 and n * k <= (6 << 20)   # small matrices at three and four rows stay on the dp4a kernel
    if fmt == 8:
        return "qgemv_q6k_mma_kernel" if m >= 3 and not small else "qgemv_kq_fast_kernel<q6_k>"
    if fmt == 7:
        return "qgemv_kq_stream_kernel<q5_k>" if m >= 3 and not small else "qgemv_kq_fast_kernel<q5_k>"
    if fmt == 5:
        return "qgemv_i4_mma_kernel" if m >= 2 else ("qgemv_i8_fast_kernel<int4>" if k % 512 == 0 else "qgemv_i4_kernel")
    if fmt == 9:
        return "qgemv_mxfp4_mma_kernel" if m >= 3 and k % 512 == 0 else "qgemv_mxfp4_kernel"
    if fmt >= 10:
        return "qgemv_iq_kernel"
    return "qgemv_i8_mma_kernel" if m >= 2 else "qgemv_i8_fast_kernel"


# dram__bytes_read.sum + dram__bytes_write.sum of one launch / algorithmic bytes of that launch, from the ncu
# captures summarised under profiles/ (weights are read once; the outputs stay in L2). A kernel without a
# capture reports no traffic.
DRAM_TRAFFIC_RATIO = {"qgemv_kq_stream_kernel<q4_k>": 0.986, "qgemv_q4k_mma_kernel": 0.985, "qgemv_kq_fast_kernel<q4_k>": 0.9985}


def max_rel(got, ref) -> float:
    """max |got - ref| / max(|ref|, rms(ref)): the parity tests' per-element measure."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = float(np.sqrt((ref ** 2).mean()))
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), max(rms, 1e-30))).max())


def rel_l2(got, ref) -> float:
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.sqrt(((got - ref) ** 2).sum() / max((ref ** 2).sum(), 1e-30)))


def published_baseline():
    """BASELINE.json's published number for this metric, if it holds one (it holds none for B200)."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            pub = json.load(f).get("published") or {}
        v = pub.get("q4k_decode_gemv_hbm_gbs")
        return float(v) if v else None
    except Exception:
        return None


def check_sweep(fmt, cases, base, acts, outs, a_off, o_off):
    """Every launch of the sweep against the oracle: the worst max_rel per kernel and overall."""
    from oracle import oracle as O
    o = O.load(fast=True)
    o.set_num_threads(cpu_threads())
    wh = {nk: t.cpu().numpy() for nk, t in base.items()}
    by_kernel, worst = {}, 0.0
    for i, (m, n, k) in enumerate(cases):
        want, _ = o.matmul(fmt, acts[a_off[i]:a_off[i] + m * k], wh[(n, k)], n, k, m=m)
        mr = max_rel(outs[o_off[i]:o_off[i] + m * n], want)
        name = "decode kernels for 3..8 rows" if m >= 3 else gemv_kernel_name(fmt, m, n, k) if m == 1 else "two rows (kernel chosen by the launch list)"
        by_kernel[name] = max(by_kernel.get(name, 0.0), mr)
        worst = max(worst, mr)
    return {"launches_checked": len(cases), "max_rel": worst, "by_kernel": by_kernel}


def _event_time(stream, fn, reps, warm=2):
    import torch
    with torch.cuda.stream(stream):
        for _ in range(warm):
            fn()
        stream.synchronize()
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            stream.synchronize()
            ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def _graph_times(be, stream, run, reps, warm=3):
    """Captures `run` (which queues work through the library on the current stream) in a CUDA graph and
    times `reps` replays with events: (median ms, min ms)."""
    import torch
    with torch.cuda.stream(stream):
        run()   # first use of a kernel variant sets its attributes: keep that out of the capture
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        be.set_stream(torch.cuda.current_stream().cuda_stream)
        run()
    be.set_stream(stream.cuda_stream)
    ts = []
    with torch.cuda.stream(stream):
        for _ in range(warm):
            graph.replay()
        stream.synchronize()
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            stream.synchronize()
            ts.append(e0.elapsed_time(e1))
    del graph
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def measure_prefill(be, stream, dev, base, quantized, check=True):
    """Prefill GEMM (tcgen05): Q4_K at M in {64, 512, 2048}, Q6_K and Q5_K at M in {512, 2048} on the gate/up
    and down shapes; five weight copies are cycled (165 MB > L2) inside one CUDA graph, 12 replays: median and
    best. TFLOP/s = 2*M*N*K / time, against the measured bf16 peaks. One Q4_K row per shape is checked
    against the oracle's f32 path on a 128-row slice of the weights (outside the timed region)."""
    import torch
    from lapid_b200.backend import matmul_launch
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        burst, sustained = float(pk["bf16_tflops"]), float(pk["bf16_tflops_sustained"])
    except Exception:
        burst, sustained = 1590.0, 1400.0
    rows = []
    for fmt, (n, k) in [(f, s) for f in (6, 8, 7) for s in [(14336, 4096), (4096, 14336)]]:
        copies = 5
        wq = base[(n, k)] if fmt == 6 else quantized(fmt, n, k, 700 + n)
        pool = wq.repeat(copies).view(copies, -1)
        for m in ((64, 512, 2048) if fmt == 6 else (512, 2048)):
            a = torch.randn(m * k, device=dev)
            o = torch.zeros(m * n, device=dev)
            torch.cuda.synchronize()
            bufs = [be.wrap_tensor(a), be.wrap_tensor(o)] + [be.wrap_tensor(pool[c]) for c in range(copies)]
            ls = [matmul_launch(fmt, m, n, k, inputs=(0, 2 + c), output=1) for c in range(copies)]
            be.prepare(ls)
            med, best = _graph_times(be, stream, be.packed(ls, bufs), 12)
            ms, ms_best = med / copies, best / copies
            tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            row = {"fmt": FMT_NAMES[fmt], "m": m, "n": n, "k": k, "us": round(ms * 1e3, 1), "us_best": round(ms_best * 1e3, 1),
                   "tflops": round(tf, 1), "tflops_best": round(2.0 * m * n * k / (ms_best * 1e-3) / 1e12, 1),
                   "frac_burst": round(tf / burst, 4), "frac_sustained": round(tf / sustained, 4),
                   "operands": "bf16 (f32 accumulate in TMEM)", "timing": "CUDA graph of 5 launches over 5 weight copies, 12 replays"}
            if check and fmt == 6 and m == 512:
                from oracle import oracle as O
                orc = O.load(fast=True)
                orc.set_num_threads(cpu_threads())
                j0, rws = n // 2 + 64, 128
                rb = k // 256 * 144
                part = wq[j0 * rb:(j0 + rws) * rb].cpu().numpy()
                want, _ = orc.matmul(6, a.cpu().numpy(), np.concatenate([part, np.zeros((-part.size) % 256, np.uint8)]), rws, k, m=m)
                got = o.view(m, n)[:, j0:j0 + rws].cpu().numpy()
                row["check"] = {"case": f"q4_k M={m} {n}x{k}, weight rows [{j0}, {j0 + rws})", "rel_l2": rel_l2(got, want),
                                "max_rel": max_rel(got, want)}
            rows.append(row)
        del pool
    return rows


def measure_moe(be, stream, dev, quantized, peak):
    """Kernel::MatMulId (the mixture-of-experts matmul) on two expert-stack shapes, Q4_K: 8 experts of
    14336 x 4096 with 2 slots per token, and 128 experts of 768 x 2048 with 8 slots. Decode launches
    (int8-activation arithmetic) report algorithmic GB/s = (routed experts' bytes + activations + outputs)
    / time, prefill launches (device-side routing + grouped tcgen05 GEMM) report TFLOP/s = 2 * pairs * n * k
    / time. Several copies of the stack (or disjoint id sets) are cycled so that weights come from HBM."""
    import torch
    from lapid_b200.backend import matmul_id_launch
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            burst = float(json.load(f)["bf16_tflops"])
    except Exception:
        burst = 1590.0
    rows = []
    for tag, e, r, n, k, copies in (("8x[14336,4096] top-2", 8, 2, 14336, 4096, 2), ("128x[768,2048] top-8", 128, 8, 768, 2048, 5)):
        one = weight_bytes(6, n, k)
        stack = quantized(6, e * n, k, 900 + e)          # K-quant stacks are dense: [e*n, k] quantized as one matrix
        pool = stack.repeat(copies).view(copies, -1)
        for t in (1, 4, 512):
            pairs = t * r
            g = torch.Generator(device="cpu")
            g.manual_seed(17 * t + e)
            x = torch.randn(t * k, device=dev)
            out = torch.zeros(pairs * n, device=dev)
            sets = 4
            id_sets = []
            for s_ in range(sets):       # distinct experts per token; decode sets are disjoint where the stack allows
                rows_ = [((torch.randperm(e, generator=g)[:r] if t > 1 else (torch.arange(r) + s_ * r) % e)) for _ in range(t)]
                id_sets.append(torch.stack(rows_).to(torch.int32).reshape(-1).to(dev))
            torch.cuda.synchronize()
            bufs = [be.wrap_tensor(x), be.wrap_tensor(out)] + [be.wrap_tensor(pool[c]) for c in range(copies)] + \
                   [be.wrap_tensor(i_) for i_ in id_sets]
            ls = [matmul_id_launch(6, t, r, e, n, k, inputs=(0, 2 + (j % copies), 2 + copies + (j % sets)), output=1)
                  for j in range(copies * sets)]
            be.prepare(ls)
            run = be.packed(ls, bufs)
            be.take_launch_count()
            with torch.cuda.stream(stream):
                run()
            stream.synchronize()
            kernels = be.take_launch_count() // len(ls)
            graph = torch.cuda.CUDAGraph()   # decode-sized launches are shorter than a host-side launch
            with torch.cuda.graph(graph, stream=stream):
                be.set_stream(torch.cuda.current_stream().cuda_stream)
                run()
            be.set_stream(stream.cuda_stream)
            ms = _event_time(stream, graph.replay, 5) / len(ls)
            del graph, run
            used = min(pairs, e) if t > 1 else r
            row = {"stack": tag, "fmt": "q4_k", "t": t, "r": r, "us": round(ms * 1e3, 2), "kernels_per_launch": kernels}
            if t <= 8:
                b = used * one + 4 * t * k + 4 * pairs * n
                row.update({"path": "decode (int8 activations)", "gbs": round(b / (ms * 1e-3) / 1e9, 1),
                            "frac_of_measured_hbm": round(b / (ms * 1e-3) / 1e9 / peak, 4)})
            else:
                tf = 2.0 * pairs * n * k / (ms * 1e-3) / 1e12
                row.update({"path": "prefill (routed, bf16 tensor cores)", "tflops": round(tf, 1), "frac_burst": round(tf / burst, 4)})
            rows.append(row)
            del bufs, ls
        del pool, stack
        torch.cuda.empty_cache()
    return rows


def measure_stack8b(be, stream, dev, quantized, peak, check=True):
    """Every quantized projection of one decode token through a 32-layer Llama-3-8B-shaped stack plus
    the output head, as ONE launch list through the C ABI (225 MatMul launches, batch 1 and 8).

    Q4_K_M-style mix: Q6_K for attn_v, for ffn_down in the `use_more_bits` layers and for the head,
    Q4_K elsewhere. The projections are chained by real data (x -> q,k,v; q_out -> o; o_out -> gate,
    up; gate_out -> down -> next layer's x), so every launch but the first waits for its producer;
    attention mixing, normalisation and the SwiGLU product are not part of this path. All 4.6 GB of
    weights are distinct and resident; a token streams each of them once.
    """
    import torch
    from lapid_b200 import tp
    from lapid_b200.backend import matmul_launch
    shape, n_layers, vocab = tp.LLAMA3_8B, 32, 128256
    d = shape.d_model
    weights, formats, token_bytes = [], [], 0
    for i in range(n_layers):
        f = {name: tp.q4km_format(name, i, n_layers) for name, _, _, _ in shape.projections()}
        w = {name: quantized(f[name], n, k, 4000 + 8 * i + j) for j, (name, n, k, _) in enumerate(shape.projections())}
        token_bytes += sum(t.numel() for t in w.values())
        weights.append(w)
        formats.append(f)
    head = quantized(8, vocab, d, 4999)
    token_bytes += head.numel()
    out = {"layers": n_layers, "head_rows": vocab, "weight_bytes_per_token": token_bytes,
           "launches_per_token": 7 * n_layers + 1,
           "ceiling_tok_s_b1": round(peak * 1e9 / token_bytes, 1)}
    for m in (1, 8):
        bufs, launches, keep = [], [], []

        def buf(t):
            keep.append(t)
            bufs.append(be.wrap_tensor(t))
            return len(bufs) - 1

        g = torch.Generator(device=dev)
        g.manual_seed(5000 + m)
        x = buf(torch.randn(m * d, device=dev, generator=g))
        dims = {name: (n, k) for name, n, k, _ in shape.projections()}
        for i in range(n_layers):
            wid = {name: buf(weights[i][name]) for name in dims}
            oid = {name: buf(torch.zeros(m * dims[name][0], device=dev)) for name in dims}
            src = {"q": x, "k": x, "v": x, "o": oid["q"], "gate": oid["o"], "up": oid["o"], "down": oid["gate"]}
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                n, k = dims[name]
                launches.append(matmul_launch(formats[i][name], m, n, k, inputs=(src[name], wid[name]), output=oid[name]))
            x = oid["down"]
        logits = buf(torch.zeros(m * vocab, device=dev))
        launches.append(matmul_launch(8, m, vocab, d, inputs=(x, buf(head)), output=logits))
        torch.cuda.synchronize()
        be.prepare(launches)
        run = be.packed(launches, bufs)
        be.take_launch_count()
        with torch.cuda.stream(stream):
            run()
        stream.synchronize()
        kernels = be.take_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            be.set_stream(torch.cuda.current_stream().cuda_stream)
            run()
        be.set_stream(stream.cuda_stream)
        ms = _event_time(stream, graph.replay, 7, warm=3)
        out[f"decode_b{m}"] = {"ms_per_token_step": round(ms, 4), "tok_s": round(m / (ms * 1e-3), 1),
                               "hbm_gbs": round(token_bytes / (ms * 1e-3) / 1e9, 1),
                               "frac_of_measured_hbm": round(token_bytes / (ms * 1e-3) / 1e9 / peak, 4),
                               "kernels_per_token": kernels}
        if check:
            # outside the timed region: the last layer's down projection and the output head of the replayed token
            # against the oracle, each on the input that launch actually read
            from oracle import oracle as O
            orc = O.load(fast=True)
            orc.set_num_threads(cpu_threads())
            stream.synchronize()
            i = n_layers - 1
            n_dn, k_dn = dims["down"]
            gate_out, down_out, logits_t = keep[oid["gate"]], keep[oid["down"]], keep[logits]   # `keep` and `bufs` share indices
            want_dn, _ = orc.matmul(formats[i]["down"], gate_out.cpu().numpy(), weights[i]["down"].cpu().numpy(), n_dn, k_dn, m=m)
            want_hd, _ = orc.matmul(8, down_out.cpu().numpy(), head.cpu().numpy(), vocab, d, m=m)
            mr = max(max_rel(down_out.cpu().numpy(), want_dn), max_rel(logits_t.cpu().numpy(), want_hd))
            out.setdefault("check", {"what": "last layer's ffn_down and the 128256 x 4096 Q6_K head vs the oracle, batch 1 and 8", "max_rel": 0.0})
            out["check"]["max_rel"] = max(out["check"]["max_rel"], mr)
        del graph, run, bufs, keep, launches
        torch.cuda.empty_cache()
    return out


def measure_tp70b(be, stream, dev, rank, world, quantized, check=True):
    """Llama-70B-shaped layer stack (80 layers: d_model 8192, 64/8 heads of 128, FFN 28672), Q4_K_M-style
    mix (Q6_K for attn_v and for ffn_down in half of the layers), tensor-parallel over `world` ranks:
    column-parallel q/k/v/gate/up, row-parallel o/down with an NCCL all-reduce. Eight distinct layer
    weight sets are cycled so the weights always come from HBM. One token = 80 layers, one CUDA graph."""
    import torch
    import torch.distributed as dist
    from lapid_b200 import tp
    shape, n_layers, n_sets = tp.LLAMA_70B, 80, 8
    weights, formats, wbytes = [], [], 0
    for s_ in range(n_sets):
        w, f = {}, {}
        for i, (name, n, k, kind) in enumerate(shape.projections()):
            fmt = tp.Q6_K if name == "v" or (name == "down" and s_ % 2 == 1) else tp.Q4_K
            nl, kl = tp.local_shape(name, n, k, kind, world)
            # random-init weights: a shard of a random matrix is a random matrix of the shard's shape
            w[name] = quantized(fmt, nl, kl, 5000 + 97 * rank + 10 * s_ + i)
            f[name] = fmt
            wbytes += w[name].numel()
        weights.append(w)
        formats.append(f)
    token_bytes = wbytes * n_layers // n_sets
    out = {"layers": n_layers, "weight_sets_cycled": n_sets, "weight_bytes_per_token_per_gpu": token_bytes, "tp": world,
           "collective": ("decode: partials pushed over peer-mapped memory from the GEMV epilogue and summed by the "
                          "following rms_norm (2 per layer, no kernel of their own); prefill: nccl all_reduce") if world > 1 else "none"}
    peer = None
    if world > 1:
        try:
            peer = tp.PeerAllReduce(be, rank, world, dev)
        except Exception as e:
            out["peer_all_reduce_error"] = f"{type(e).__name__}: {e}"[:200]
    # decode_b1: the row-parallel GEMVs push their partials from their epilogue and the following
    # rms_norm sums them (no all-reduce kernel); _allreduce_kernel: the library's stand-alone one-shot
    # all-reduce; _nccl: the library collective, for comparison
    # _prepass: the same stack with a quantizing pre-pass kernel in front of every projection group instead
    # of the rms_norm / silu_mul kernels writing the quantized operand themselves
    variants = [(1, "decode_b1", peer, True, True, False), (1, "decode_b1_prepass", peer, True, False, False),
                (512, "prefill_m512", peer, False, True, False)]
    if world > 1:
        variants.append((512, "prefill_m512_no_collective", peer, False, True, True))   # timing only: what the all-reduces cost
    if world > 1 and peer is not None:
        variants.insert(2, (1, "decode_b1_allreduce_kernel", peer, False, True, False))
        variants.insert(3, (1, "decode_b1_nccl", None, False, True, False))
    for m, key, reducer, fused, fuse_act, skip in variants:
        layers = tp.GpuTpLayers(be, shape, world, rank, m, weights, formats, peer_all_reduce=reducer, fused=fused, fuse_act=fuse_act,
                                skip_collective=skip)
        layers.h.normal_()
        torch.cuda.synchronize()
        run = lambda: layers.token(n_layers)
        graph = None
        with torch.cuda.stream(stream):
            run()
        stream.synchronize()
        try:   # one token = one CUDA graph (NCCL's all-reduce is captured with the rest)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                be.set_stream(torch.cuda.current_stream().cuda_stream)
                run()
            be.set_stream(stream.cuda_stream)
            run = graph.replay
        except Exception as e:
            out["graph_error"] = str(e)[:200]
            graph = None
            be.set_stream(stream.cuda_stream)
            run = lambda: layers.token(n_layers)
        if world > 1:
            dist.barrier()
        ms = _event_time(stream, run, 5 if m == 1 else 3, warm=2 if m == 1 else 1)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        row = {"ms_per_token_step": round(ms, 4), "tok_s": round(m / (ms * 1e-3), 2), "cuda_graph": graph is not None}
        if m == 1:
            row["hbm_gbs_per_gpu"] = round(token_bytes / (ms * 1e-3) / 1e9, 1)
            row["frac_of_hbm_ceiling"] = round(token_bytes / (ms * 1e-3) / 1e9 / measured_peaks()[0], 4)
        else:
            fl = 2.0 * m * sum(n * k for _, n, k, _ in shape.projections()) * n_layers
            row["tflops_total"] = round(fl / (ms * 1e-3) / 1e12, 1)
        out[key] = row
        del layers, graph
        torch.cuda.empty_cache()
    if "prefill_m512_no_collective" in out:
        a, b = out["prefill_m512"]["ms_per_token_step"], out["prefill_m512_no_collective"]["ms_per_token_step"]
        out["prefill_m512"]["collective_share"] = round(max(0.0, a - b) / a, 4)
    if check and world > 1:
        try:
            out["check"] = tp_check(be, stream, dev, rank, world, quantized, peer)
        except Exception as e:
            out["check"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


def tp_check(be, stream, dev, rank, world, quantized, peer):
    """Tensor-parallel correctness at this world size, outside any timed region: one 70B-shaped layer whose shards
    are cut from COMMON full matrices (every rank makes the same full matrices from the same seeds and keeps its
    shard), run sharded on all ranks and unsharded on rank 0. `first_exchange`: h + sum over ranks of o, whose inputs
    are the same on both sides, so only the order of f32 sums differs (bar 1e-5); `layer`: the whole layer step,
    where those differences pass the int8 activation quantizer of the later projections (bar rel_l2 1e-2)."""
    import torch
    import torch.distributed as dist
    from lapid_b200 import tp
    shape = tp.LLAMA_70B
    full, fmts, shard = {}, {}, {}
    for i, (name, n, k, kind) in enumerate(shape.projections()):
        fmts[name] = tp.Q6_K if name in ("v", "down") else tp.Q4_K
        full[name] = quantized(fmts[name], n, k, 9000 + i)   # the same matrix on every rank
        cut = tp.shard_rows if kind == "column" else tp.shard_cols
        shard[name] = cut(fmts[name], full[name], n, k, rank, world)[0]
    res = {"what": "sharded layer (all ranks) vs unsharded layer (rank 0), shards cut from common full matrices", "tp": world}
    for m, key in ((1, "decode_b1"), (512, "prefill_m512")):
        g = torch.Generator(device=dev)
        g.manual_seed(77 + m)
        h0 = torch.randn(m, shape.d_model, device=dev, generator=g)
        got = {}
        sharded = tp.GpuTpLayers(be, shape, world, rank, m, [shard], [fmts], peer_all_reduce=peer, fused=(m == 1), fuse_act=True)
        for part in ("first_exchange", "layer"):
            sharded.h.copy_(h0)
            torch.cuda.synchronize()
            dist.barrier()
            with torch.cuda.stream(stream):
                t = sharded.first_row_parallel() if part == "first_exchange" else sharded.token(1)
            stream.synchronize()
            got[part] = t.clone()
        del sharded
        dist.barrier()
        if rank == 0:
            single = tp.GpuTpLayers(be, shape, 1, 0, m, [full], [fmts], fuse_act=True)
            row = {}
            for part in ("first_exchange", "layer"):
                single.h.copy_(h0)
                torch.cuda.synchronize()
                with torch.cuda.stream(stream):
                    t = single.first_row_parallel() if part == "first_exchange" else single.token(1)
                stream.synchronize()
                row[part] = {"max_rel": max_rel(got[part].cpu().numpy(), t.cpu().numpy()),
                             "rel_l2": rel_l2(got[part].cpu().numpy(), t.cpu().numpy())}
            res[key] = row
            del single
        torch.cuda.empty_cache()
        dist.barrier()
    return res


def run_case(args):
    """One matmul case through the C ABI: `reps` executes of `copies` launches (each over its own weight copy, so a
    decode launch streams from HBM), then the same list as a CUDA graph, timed with events. Prints one JSON row."""
    import torch
    import lapid_b200 as lp
    from lapid_b200 import quant
    from lapid_b200.backend import matmul_id_launch, matmul_launch
    parts = args.case.split(",")
    names = {v: kk for kk, v in FMT_NAMES.items()}
    fmt, (m, n, k) = names[parts[0]], [int(x) for x in parts[1:4]]
    copies = int(parts[4]) if len(parts) > 4 else 6
    reps = int(parts[5]) if len(parts) > 5 else 2
    be = lp.Backend(0)
    for kv in list(filter(None, os.environ.get("LAPID_B200_OPTS", "").split(","))) + list(args.opt):
        key, _, val = kv.partition("=")
        be.set_option(key, val)
    stream = torch.cuda.Stream()
    be.set_stream(stream.cuda_stream)
    e, r = args.experts, args.slots
    one = quant.layout(fmt, n, k).total
    stack = torch.empty((e or 1) * one, dtype=torch.uint8, device="cuda")
    for x in range(e or 1):
        if fmt >= 10:   # the i-quants have no quantizer here; every byte pattern is a valid block: random blocks, small f16 scales
            g = torch.Generator(device="cuda")
            g.manual_seed(7 + x)
            blocks = torch.randint(0, 256, (n * k // 256, AOS_BLOCK[fmt][1]), dtype=torch.uint8, device="cuda", generator=g)
            blocks[:, 0] = 0x1F          # d = f16 0x211F, about 0.01
            blocks[:, 1] = 0x21
            stack[x * one:x * one + blocks.numel()] = blocks.reshape(-1)
            torch.cuda.synchronize()
            continue
        w = torch.randn(n * k, device="cuda") * 0.02
        torch.cuda.synchronize()
        be.quantize_into(fmt, be.wrap_tensor(w), n, k, be.wrap_tensor(stack[x * one:(x + 1) * one]))
    pool = stack.repeat(copies).view(copies, -1)
    a = torch.randn(m * k, device="cuda")
    if e:
        g = torch.Generator()
        g.manual_seed(1)
        ids = torch.stack([torch.randperm(e, generator=g)[:r] for _ in range(m)]).to(torch.int32).reshape(-1).cuda()
        o = torch.zeros(m * r * n, device="cuda")
        torch.cuda.synchronize()
        bufs = [be.wrap_tensor(a), be.wrap_tensor(o), be.wrap_tensor(ids)] + [be.wrap_tensor(pool[c]) for c in range(copies)]
        launches = [matmul_id_launch(fmt, m, r, e, n, k, inputs=(0, 3 + c, 2), output=1) for c in range(copies)]
    else:
        o = torch.zeros(m * n, device="cuda")
        torch.cuda.synchronize()
        bufs = [be.wrap_tensor(a), be.wrap_tensor(o)] + [be.wrap_tensor(pool[c]) for c in range(copies)]
        launches = [matmul_launch(fmt, m, n, k, inputs=(0, 2 + c), output=1) for c in range(copies)]
    be.prepare(launches)
    run = be.packed(launches, bufs)
    be.take_launch_count()
    with torch.cuda.stream(stream):
        for _ in range(reps):
            run()
    stream.synchronize()
    kernels = be.take_launch_count() // max(1, reps)
    med, best = _graph_times(be, stream, run, 9)
    us, us_best = med / copies * 1e3, best / copies * 1e3
    row = {"case": args.case, "experts": e, "copies": copies, "reps": reps, "kernels_per_list": kernels, "us_per_launch": round(us, 3),
           "us_per_launch_best": round(us_best, 3), "checksum": float(o.abs().sum())}
    if not e and m <= 8:
        peak, kind = measured_peaks()
        gbs = algo_bytes(fmt, m, n, k) / (us * 1e-6) / 1e9
        row.update({"gbs": round(gbs, 1), "frac_of_hbm": round(gbs / peak, 4), "peak_kind": kind})
    elif not e:
        row["tflops"] = round(2.0 * m * n * k / (us * 1e-6) / 1e12, 1)
    if args.trace:
        row["timeline"] = stream_kernel_timeline(be, stream, run, copies)
    print(json.dumps(row), flush=True)


def stream_kernel_timeline(be, stream, run, launches, mhz=1965.0):
    """Per-CTA timeline of the balanced-stream decode kernel over one CUDA-graph replay of `run` (the library's
    diagnostics call: `lapid_b200_decode_trace_begin` / `_read`). Microseconds; SM clock cycles are converted with the
    maximum SM clock. Per launch: CTAs, when they entered and left (5 % / median / 95 % of the CTAs, relative to the first
    entry of the first launch), and the means of a CTA's phases -- entry to first data, first data to the end of its
    span (`work`), the rest (`after`: staging or hand-over, waits, stores), of which it waited for data (`starved`)."""
    import torch
    with torch.cuda.stream(stream):
        run()
    stream.synchronize()
    be.decode_trace_begin(launches)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        be.set_stream(torch.cuda.current_stream().cuda_stream)
        run()
    be.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(4):
            graph.replay()
    stream.synchronize()
    t = be.decode_trace_read(launches).astype(np.int64)
    be.decode_trace_begin(0)
    del graph
    out, base = [], None
    pct = lambda x: [round(float(np.percentile(x, q)), 2) for q in (5, 50, 95)]
    for i in range(t.shape[0]):
        r = t[i]
        r = r[r[:, 1] != 0]   # rows of CTAs that ran
        if not len(r):
            continue
        base = int(r[:, 0].min()) if base is None else base
        cyc = lambda a, b: (r[:, b] - r[:, a]) / mhz
        out.append({"launch": i, "ctas": int(len(r)), "units_per_cta": [int(r[:, 9].min()), int(r[:, 9].max())],
                    "entry_us": pct((r[:, 0] - base) / 1e3), "exit_us": pct((r[:, 7] - base) / 1e3), "last_exit_us": round(float((r[:, 7] - base).max()) / 1e3, 2),
                    "mean_us": {"life": round(float(cyc(1, 6).mean()), 2), "first_data": round(float(cyc(1, 3).mean()), 2),
                                "work": round(float(cyc(3, 4).mean()), 2), "after": round(float(cyc(4, 6).mean()), 2),
                                "starved": round(float((r[:, 10] / mhz).mean()), 2)}})
    return out


def cpu_baseline(cases, fmt):
    """The oracle's timed copy on this host's cores: a bounded sample (about 10 s) of full steps of the same sweep."""
    from oracle import oracle as O
    o = O.load(fast=True)
    val, ms, done, cores = cpu_sweep(o, fmt, budget_s=10.0, max_steps=50, warm=1)
    return {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{done} full steps of the 16-GEMV Q4_K sweep (one weight copy per launch), {ms:.1f} ms per step"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cases", action="store_true", help="skip the per-case breakdown")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM rows")
    ap.add_argument("--no-tp", action="store_true", help="skip the 70B-shaped tensor-parallel layer stack")
    ap.add_argument("--no-moe", action="store_true", help="skip the MatMulId (mixture-of-experts) measurements")
    ap.add_argument("--no-stack", action="store_true", help="skip the 32-layer 8B-shaped projection stack")
    ap.add_argument("--no-check", action="store_true", help="skip the result checks against the CPU oracle (they run outside the timed regions)")
    ap.add_argument("--case", default=None, metavar="FMT,M,N,K[,COPIES[,REPS]]",
                    help="run ONE matmul case instead of the benchmark (e.g. q4_k,8,14336,4096,6,2): REPS executes of COPIES launches, "
                         "each over its own weight copy, then a timed CUDA-graph replay; small enough to sit under a profiler")
    ap.add_argument("--trace", action="store_true", help="--case: add the per-CTA timeline of the balanced-stream decode kernel (one more graph replay)")
    ap.add_argument("--experts", type=int, default=0, help="--case: MatMulId over a stack of this many matrices (0: a plain MatMul)")
    ap.add_argument("--slots", type=int, default=2, help="--case with --experts: experts per token")
    ap.add_argument("--opt", action="append", default=[], help="device option key=value (repeatable)")
    ap.add_argument("--e2e-chunk", type=int, default=0, help="launches per chunk of the end-to-end step's pipelined call (0: the library picks)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.case:
        run_case(args)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
