"""Run one Q4_K matmul shape on cuda:0 a few times and report its time.

    python -m backpack_b200.run_case N K M [--reps R] [--variant auto|fp32|stream]
                                           [--prefill-mode f16x3|f16|bf16] [--qtype q4k|q5k|q6k|q6kp]
                                           [--opt ID=VALUE ...]
                                           [--experts E --tokens T --topk R [--flush]]

A small driver for profilers and quick checks: seeded synthetic weights and
activations (backpack_b200.synth), `reps` back-to-back calls through the C ABI,
CUDA-event timing of the last `reps - 1` calls.  With --experts the weight is a stack of
E matrices of N rows and every call is the expert-indexed matmul of T tokens routed to R
experts each (a new seeded routing per call; --flush writes 256 MB between calls so that no
expert of an earlier call is still in L2; the time then includes that write).
"""
from __future__ import annotations

import argparse

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("M", type=int)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--variant", default="auto", choices=["auto", "fp32", "stream"])
    ap.add_argument("--prefill-mode", default="f16x3", choices=["f16x3", "f16", "bf16"],
                    help="precision mode of the tensor-core kernel (large M)")
    ap.add_argument("--qtype", default="q4k", choices=["q4k", "q5k", "q6k", "q6kp"],
                    help="weight format (q6kp: Q6_K in the padded device layout of the streaming kernel)")
    ap.add_argument("--opt", action="append", default=[], metavar="ID=VALUE",
                    help="set a numbered library option (see include/bpq4k.h), e.g. --opt 10=8 for 8 warps")
    ap.add_argument("--experts", type=int, default=0, help="expert-indexed form: number of stacked matrices of N rows")
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--flush", action="store_true", help="write a 256 MB buffer between calls")
    args = ap.parse_args()

    import torch

    import backpack_b200 as bp
    from backpack_b200 import q4k, synth

    ctx = bp.Q4KContext(0)
    ctx.set_option(q4k.OPT_GEMV_VARIANT, {"auto": q4k.GEMV_AUTO, "fp32": q4k.GEMV_FP32, "stream": q4k.GEMV_STREAM}[args.variant])
    ctx.set_option(q4k.OPT_PREFILL_MODE, {"f16x3": q4k.PREFILL_F16X3, "f16": q4k.PREFILL_F16, "bf16": q4k.PREFILL_BF16}[args.prefill_mode])
    for kv in args.opt:
        k, v = kv.split("=")
        ctx.set_option(int(k), int(v))
    qtype = {"q4k": q4k.Q4_K, "q5k": q4k.Q5_K, "q6k": q4k.Q6_K, "q6kp": q4k.Q6_K_PADDED}[args.qtype]
    ftype = q4k.Q6_K if qtype == q4k.Q6_K_PADDED else qtype   # the file format behind the device layout
    if args.experts:
        run_experts(args, ctx, torch, bp, synth, qtype, ftype)
        return
    w = ctx.upload(bp.pack_kq(qtype, synth.make_kq_weights(ftype, args.N, args.K, 0), args.N, args.K))
    x = torch.from_numpy(synth.make_activations(args.M, args.K, 1)).cuda()
    y = torch.zeros(args.M, args.N, device="cuda")
    ctx.matmul(x, w, out=y)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(max(args.reps - 1, 1)):
        ctx.matmul(x, w, out=y)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / max(args.reps - 1, 1)
    nbytes = synth.kq_algorithmic_bytes(ftype, args.M, args.N, args.K)
    print(f"N={args.N} K={args.K} M={args.M}: {us:.2f} us/call, {nbytes / us / 1e3:.1f} GB/s algorithmic "
          f"(back-to-back calls on one weight: L2-warm if it fits), checksum {float(y.double().abs().sum()):.6e}")


def run_experts(args, ctx, torch, bp, synth, qtype, ftype) -> None:
    E, N, K, T, R = args.experts, args.N, args.K, args.tokens, args.topk
    w = ctx.upload(bp.pack_kq(qtype, synth.make_kq_weights(ftype, E * N, K, 0), E * N, K))
    x = torch.from_numpy(synth.make_activations(T, K, 1)).cuda()
    x_rows = torch.arange(T, device="cuda", dtype=torch.int32).repeat_interleave(R)
    reps = max(args.reps, 2)
    routes = [synth.make_moe_routing(T, E, R, 10 + i).reshape(-1) for i in range(reps)]
    offs = [torch.from_numpy((r * N).astype(np.int32)).cuda() for r in routes]
    y = torch.zeros(T * R, N, device="cuda")
    junk = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if args.flush else None
    ctx.matmul_moe(x, w, N, offs[0], x_rows=x_rows, out=y)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(1, reps):
        if junk is not None:
            junk.fill_(i)
        ctx.matmul_moe(x, w, N, offs[i], x_rows=x_rows, out=y)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps - 1)
    distinct = float(np.mean([len(np.unique(r)) for r in routes[1:]]))
    per_expert = synth.kq_weight_bytes(ftype, N, K)
    print(f"{E} experts of {N}x{K}, {T} tokens x {R} experts ({T * R} slots, {distinct:.1f} distinct): {us:.2f} us/call"
          f"{' including the flush' if args.flush else ''}; weight bytes per call {distinct * per_expert / 1e6:.1f} MB distinct, "
          f"{T * R * per_expert / 1e6:.1f} MB by slots; checksum {float(y.double().abs().sum()):.6e}")


if __name__ == "__main__":
    main()
