"""Runs a few launches of ONE matmul case through the C ABI, small enough to sit under a profiler.

    python -m lapid_b200.profile_case --fmt q4_k --m 1 --n 14336 --k 4096 [--copies 6] [--reps 2]
    python -m lapid_b200.profile_case --fmt q4_k --experts 8 --slots 2 --m 512 --n 14336 --k 4096 --copies 1

With `--experts E --slots R` the case is a MatMulId launch: `--m` tokens, R distinct random experts
per token out of a stack of E matrices [n, k].

Weights are N(0, 0.02) quantized on the device; each launch of a repetition reads its own weight
copy, so with `--copies 6` of a 33 MB matrix a decode launch streams from HBM, not from L2.
"""
from __future__ import annotations

import argparse

FMTS = {"int8": 4, "q4_k": 6, "q5_k": 7, "q6_k": 8}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--fmt", default="q4_k", choices=sorted(FMTS))
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--copies", type=int, default=6)
    ap.add_argument("--reps", type=int, default=2)
    ap.add_argument("--experts", type=int, default=0, help="MatMulId: matrices in the stack (0: a plain MatMul)")
    ap.add_argument("--slots", type=int, default=2, help="MatMulId: experts per token")
    ap.add_argument("--opt", action="append", default=[], help="device option key=value")
    args = ap.parse_args()

    import torch
    import lapid_b200 as lp
    from lapid_b200 import quant
    from lapid_b200.backend import matmul_id_launch, matmul_launch

    fmt, m, n, k = FMTS[args.fmt], args.m, args.n, args.k
    be = lp.Backend(0)
    for kv in args.opt:
        key, _, val = kv.partition("=")
        be.set_option(key, val)
    if args.experts:
        e, r = args.experts, args.slots
        one = quant.layout(fmt, n, k).total
        stack = torch.empty(e * one, dtype=torch.uint8, device="cuda")
        for x in range(e):
            w = torch.randn(n * k, device="cuda") * 0.02
            torch.cuda.synchronize()
            be.quantize_into(fmt, be.wrap_tensor(w), n, k, be.wrap_tensor(stack[x * one:(x + 1) * one]))
        pool = stack.repeat(args.copies).view(args.copies, -1)
        g = torch.Generator()
        g.manual_seed(1)
        ids = torch.stack([torch.randperm(e, generator=g)[:r] for _ in range(m)]).to(torch.int32).reshape(-1).cuda()
        a = torch.randn(m * k, device="cuda")
        o = torch.zeros(m * r * n, device="cuda")
        torch.cuda.synchronize()
        bufs = [be.wrap_tensor(a), be.wrap_tensor(o), be.wrap_tensor(ids)] + [be.wrap_tensor(pool[c]) for c in range(args.copies)]
        launches = [matmul_id_launch(fmt, m, r, e, n, k, inputs=(0, 3 + c, 2), output=1) for c in range(args.copies)]
        be.prepare(launches)
        for _ in range(args.reps):
            be.execute(launches, bufs)
        print("ok", float(o.abs().sum()))
        return
    w = torch.randn(n * k, device="cuda") * 0.02
    q = torch.empty(quant.layout(fmt, n, k).total, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    be.quantize_into(fmt, be.wrap_tensor(w), n, k, be.wrap_tensor(q))
    pool = q.repeat(args.copies).view(args.copies, -1)
    a = torch.randn(m * k, device="cuda")
    o = torch.zeros(m * n, device="cuda")
    torch.cuda.synchronize()
    bufs = [be.wrap_tensor(a), be.wrap_tensor(o)] + [be.wrap_tensor(pool[c]) for c in range(args.copies)]
    launches = [matmul_launch(fmt, m, n, k, inputs=(0, 2 + c), output=1) for c in range(args.copies)]
    be.prepare(launches)
    for _ in range(args.reps):
        be.execute(launches, bufs)
    print("ok", float(o.abs().sum()))


if __name__ == "__main__":
    main()
