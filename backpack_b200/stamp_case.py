"""Where the microseconds of a decode step go: in-kernel time stamps of every launch of the step.

    python -m backpack_b200.stamp_case [8b|fused|70b] [ID=VALUE ...]

Runs the configuration-1 projections (eight launches), the same with Q+K+V and gate+up fused by rows (five), or the
Llama-3-70B shapes, M = 1, as a CUDA graph of two consecutive steps with BPQ4K_OPT_STREAM_STAMPS on, and prints per
launch of the replayed graph, in microseconds: when its first CTA started, when the preceding kernel released it
(first and last CTA), how long the staging of the activation row took, the streaming loop of thread 0 of each CTA
(median and slowest CTA; each tile's reduction included), the K-split tile after it, the end of the last CTA, the gap
between the previous launch's end and this launch's release, and the span from release to end.  ID=VALUE sets a
numbered library option first (see include/bpq4k.h).  A profiling aid beside run_case.py; needs a B200.
"""
from __future__ import annotations

import sys

import numpy as np


def main() -> None:
    import torch

    import backpack_b200 as bp
    from backpack_b200 import q4k, synth

    which = sys.argv[1] if len(sys.argv) > 1 and "=" not in sys.argv[1] else "8b"
    shapes = {"8b": synth.LLAMA3_8B, "70b": synth.LLAMA3_70B,
              "fused": [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336),
                        ("lm_head", 128256, 4096)]}[which]
    ctx = bp.Q4KContext(0, stamps=True)      # libbpq4k_stamps.so: the product library with the stamps compiled in
    dev = "cuda:0"
    for kv in sys.argv[1:]:
        if "=" in kv:
            k, v = kv.split("=")
            ctx.set_option(int(k), int(v))
    W = {n: ctx.upload(bp.pack_q4k(synth.make_q4k_weights(N, K, i + 1), N, K)) for i, (n, N, K) in enumerate(shapes)}
    X = {n: torch.randn(1, K, device=dev) for n, N, K in shapes}
    Y = {n: torch.zeros(1, N, device=dev) for n, N, K in shapes}
    reps = 2
    L = reps * len(shapes)
    slots = 2 * L + 8

    def step():
        for _ in range(reps):
            for n, _, _ in shapes:
                ctx.matmul(X[n], W[n], out=Y[n])

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        ctx.set_option(q4k.OPT_STREAM_STAMPS, slots)      # the capture below gets slots 0 .. L-1
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            step()
        for _ in range(3):
            g.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        g.replay()
        e1.record(stream)
        stream.synchronize()
    print(f"graph of {reps} steps: {e0.elapsed_time(e1) * 1e3 / reps:.2f} us per step")
    ts, _ = ctx.stream_stamps(slots)
    ctx.set_option(q4k.OPT_STREAM_STAMPS, 0)
    base, prev_end = None, None
    print(f"{'launch':10s} {'CTAs':>4s} | {'start':>7s} {'released':>8s} {'(last)':>7s} | {'stage':>6s} {'loop med':>8s} {'loop max':>8s} {'tail':>5s} | "
          f"{'end':>7s} {'gap':>5s} {'span':>6s} | ends: first / median")
    for i in range(L):
        name = shapes[i % len(shapes)][0]
        grid = int(ts[i, 0, 7] >> np.uint64(32))
        if grid == 0:
            print(f"{name:10s} (not stamped: not the single-row streaming kernel)")
            continue
        t = ts[i, :min(grid, 160), :6].astype(np.int64)
        if base is None:
            base = t[:, 0].min()
        t = (t - base) / 1e3
        rel0, rel1 = t[:, 2].min(), t[:, 2].max()
        stage = np.median(t[:, 3] - t[:, 2])
        loop = t[:, 4] - t[:, 3]
        tail = np.median(t[:, 5] - t[:, 4])
        end = t[:, 5].max()
        gap = rel0 - prev_end if prev_end is not None else float("nan")
        print(f"{name:10s} {grid:4d} | {t[:, 0].min():7.2f} {rel0:8.2f} {rel1:7.2f} | {stage:6.2f} {np.median(loop):8.2f} {loop.max():8.2f} {tail:5.2f} | "
              f"{end:7.2f} {gap:5.2f} {end - rel0:6.2f} | {t[:, 5].min():7.2f} / {np.median(t[:, 5]):7.2f}")
        prev_end = end


if __name__ == "__main__":
    main()
