"""Interleaved A/B of library option sets on the decode step.

    python -m backpack_b200.step_ab NAME:ID=VALUE,ID=VALUE [NAME2:...] [--branches]

Every option set (NAME: alone = the defaults; IDs as in include/bpq4k.h) is captured as two CUDA graphs of ten
consecutive steps, M = 1 -- the eight projections of configuration 1, and the same bytes with Q+K+V and gate+up fused by
rows (five launches) -- and the graphs are replayed in turn, twelve rounds, so that every set sees the same clocks and
the same neighbours; the median microseconds per step of each is printed.  Every projection has its own weight
(418 MB per step, nothing stays in L2).  --branches adds the eight-launch step with the independent projections
(q, k, v; gate, up) on parallel branches of the graph.  A tuning aid beside run_case.py; needs a B200.
"""
from __future__ import annotations

import sys

import numpy as np


def main() -> None:
    import torch

    import backpack_b200 as bp
    from backpack_b200 import synth

    args = [a for a in sys.argv[1:] if a != "--branches"]
    branches = "--branches" in sys.argv[1:]
    cfgs = []
    for a in args or ["defaults:"]:
        name, _, rest = a.partition(":")
        cfgs.append((name, [tuple(int(x) for x in kv.split("=")) for kv in rest.split(",") if kv]))
    ctx = bp.Q4KContext(0)
    dev = "cuda:0"
    S8 = synth.LLAMA3_8B
    S5 = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336), ("lm_head", 128256, 4096)]
    W = {n: ctx.upload(bp.pack_q4k(synth.make_q4k_weights(N, K, i + 1), N, K)) for i, (n, N, K) in enumerate(S8 + S5[:1] + S5[2:3])}
    X = {K: torch.randn(1, K, device=dev) for K in {k for _, _, k in S8}}
    Y = {n: torch.zeros(1, w.N, device=dev) for n, w in W.items()}
    main_s, s1, s2 = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    reps = 10

    def mm(n, st=main_s):
        with torch.cuda.stream(st):
            ctx.matmul(X[W[n].K], W[n], out=Y[n])

    def fork(group, streams):
        ev = torch.cuda.Event()
        ev.record(main_s)
        for st in streams[1:len(group)]:
            st.wait_event(ev)
        for n, st in zip(group, streams):
            mm(n, st)
        for st in streams[1:len(group)]:
            e = torch.cuda.Event()
            e.record(st)
            main_s.wait_event(e)

    def eight():
        for n, _, _ in S8:
            mm(n)

    def five():
        for n, _, _ in S5:
            mm(n)

    def eight_branches():
        fork(["q", "k", "v"], [main_s, s1, s2])
        mm("o")
        fork(["gate", "up"], [main_s, s1])
        mm("down")
        mm("lm_head")

    forms = [("8 launches", eight), ("5 launches", five)] + ([("8, parallel branches", eight_branches)] if branches else [])
    touched = sorted({o for _, opts in cfgs for o, _ in opts})
    defaults = {o: ctx.get_option(o) for o in touched}
    graphs = {}
    with torch.cuda.stream(main_s):
        for name, opts in cfgs:
            for o, v in defaults.items():
                ctx.set_option(o, v)
            for o, v in opts:
                ctx.set_option(o, v)
            for fname, fn in forms:
                try:
                    fn()                     # eager first: an option set a shape cannot take fails here, outside any capture
                except Exception as e:       # noqa: BLE001
                    print(f"{name}: {fname}: not applicable ({e})", flush=True)
                    continue
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=main_s):
                    for _ in range(reps):
                        fn()
                graphs[(name, fname)] = g
        for o, v in defaults.items():
            ctx.set_option(o, v)
        res = {k: [] for k in graphs}
        for it in range(12):
            for k, g in graphs.items():
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g.replay()
                e0.record(main_s)
                g.replay()
                e1.record(main_s)
                main_s.synchronize()
                if it >= 2:
                    res[k].append(e0.elapsed_time(e1) * 1e3 / reps)
    for name, _ in cfgs:
        print(f"{name:16s} " + "   ".join(f"{fname}: {np.median(res[(name, fname)]):7.2f} us (min {min(res[(name, fname)]):7.2f})"
                                          for fname, _ in forms if (name, fname) in res), flush=True)
    assert ctx.device_status() == 0


if __name__ == "__main__":
    main()
