"""Benchmark of the Q4_K matmul path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload (``config.workload``): the decode projections of a Llama-3-8B-shaped
model, M = 1, GGUF Q4_K weights -- q 4096x4096, k/v 1024x4096, o 4096x4096,
gate/up 14336x4096, down 4096x14336, lm_head 128256x4096 -- random weights and
N(0,1) activations from seeded generators (no model files are involved).  One
step = one pass over all eight projections, each with its own activation and
output buffer.  The weights of one pass (418 MB) exceed the 126 MB L2, so every
launch streams its weights from HBM.

``value``     whole-job algorithmic GB/s (weights + activations + outputs moved
              once) with everything resident in HBM, the step replayed from a
              CUDA graph, timed with CUDA events; max over ranks.
``e2e``       the same metric through the host-buffer C-ABI call
              (bpq4k_matmul_host_batch_f32, one call per step): every step moves
              the activations from pinned host memory to the device (one gather
              kernel), runs the kernels on the resident weights, writes the
              outputs to pinned host memory (one scatter kernel) and waits; the
              library replays that list from a CUDA graph once it has seen it
              twice.
``roofline``  the dominant kernel (the streaming matmul kernel) against the
              measured HBM copy bandwidth.
``cpu_baseline`` the reference's own CPU code for the path (dequant_kquant +
              float dot) timed on this machine's host cores on a bounded sample.

``prefill``   (1 GPU) the same projections at M = 512 through the tensor-core
              kernel, useful TFLOP/s per precision mode.
``per_shape``  (1 GPU) every distinct projection shape of the step alone, HBM-cold.
``fused_projections`` (1 GPU) the step with Q+K+V and gate+up fused by rows.
``kquant_siblings``   (1 GPU) the output head in Q5_K and Q6_K, M = 1.
``fused_prologues``   (1 GPU) launch time with and without a fused RMSNorm /
              silu*up prologue and residual epilogue.
``routed_experts``    (1 GPU) configuration 3: one routed-expert layer (128 experts,
              8 tokens x 8 experts), the matmuls alone and the whole step.
``gguf_upload``       (1 GPU) file -> HBM rate of the GGUF tensor loader.

With N > 1 ranks every rank holds its own row shard of each projection (the
shard has the single-GPU shape, i.e. the global matrix has N times the rows:
weak scaling).  ``--gather peer`` (default): the matmul epilogue stores each
output slice straight into every rank's gather buffer over peer memory and one
bounded flag barrier closes the step, all inside one CUDA graph.
``--gather nccl``: one NCCL all-gather per projection, launched eagerly.

``--impl reference`` times the reference's CPU implementation only (rank 0).
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from backpack_b200 import synth  # noqa: E402

METRIC = "q4k_matmul_m1_algorithmic_bandwidth"
UNIT = "GB/s"
WORKLOAD = "llama3-8b decode projections, M=1, Q4_K (config 1)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# DRAM read+write bytes of the streaming kernel divided by its algorithmic bytes, from one ncu capture
# on a 151 MB case (65536 x 4096, M = 1); traffic grows with the rows, so a launch's traffic is this
# ratio times its algorithmic bytes.
TRAFFIC_RATIO = 1.022


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAKS["hbm_gbs"], "fallback"


def step_bytes(M=1):
    return sum(synth.algorithmic_bytes(M, N, K) for _, N, K in synth.LLAMA3_8B)


def weight_bytes_total():
    return sum(synth.weight_bytes(N, K) for _, N, K in synth.LLAMA3_8B)


# --------------------------------------------------------------------------
# clocks (read-only NVML sampling during the timed regions)
# --------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.dev))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# --------------------------------------------------------------------------
# CPU baseline / reference arm
# --------------------------------------------------------------------------
def cpu_pass(kind_ref: bool, threads: int, shapes, weights, xs):
    from oracle import q4k_oracle as orc

    t0 = time.perf_counter()
    for (name, N, K) in shapes:
        orc.matmul(xs[name], weights[name], None, N, K, threads=threads, use_ref=kind_ref)
    return time.perf_counter() - t0


def cpu_baseline(budget_s: float, shapes, weights, xs):
    """Time the reference's CPU path on a bounded sample: whole passes over `shapes`, row-parallel over all
    host cores, and one pass on a single thread (the reference itself runs this code single-threaded)."""
    from oracle import q4k_oracle as orc

    kind_ref = orc.ref_available()
    cores = os.cpu_count() or 1
    best, reps, spent = None, 0, 0.0
    while reps < 2 or (spent < budget_s and reps < 50):
        dt = cpu_pass(kind_ref, cores, shapes, weights, xs)
        best = dt if best is None else min(best, dt)
        spent += dt
        reps += 1
    nbytes = sum(synth.algorithmic_bytes(1, N, K) for _, N, K in shapes)
    single = cpu_pass(kind_ref, 1, shapes, weights, xs)
    return {"value": nbytes / best / 1e9, "unit": UNIT, "cores": cores,
            "kind": "reference" if kind_ref else "port",
            "sample": f"{reps} passes over {len(shapes)} projections ({nbytes / 1e6:.0f} MB each), best pass",
            "single_thread": {"value": nbytes / single / 1e9, "unit": UNIT, "cores": 1,
                              "sample": "one pass over the same projections on one thread, as the reference runs it"}}


def make_host_inputs(shapes, config_tag, rank=0):
    weights, xs = {}, {}
    for name, N, K in shapes:
        weights[name] = synth.make_q4k_weights(N, K, synth.shape_seed(config_tag, name) + rank)
        xs[name] = synth.make_activations(1, K, synth.shape_seed(config_tag, name + ".x") + rank)
    return weights, xs


def run_reference_arm(args, rank):
    """The reference's CPU implementation of the path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    shapes = list(synth.LLAMA3_8B)
    weights, xs = make_host_inputs(shapes, "config1")
    from oracle import q4k_oracle as orc

    kind_ref = orc.ref_available()
    cores = os.cpu_count() or 1
    steps, warm = max(args.steps, 1), max(args.warmup, 0)
    # Bound the run: if (steps + warmup) full passes would take more than the
    # budget, each step processes the same leading fraction of every projection's rows.
    t_full = cpu_pass(kind_ref, cores, shapes, weights, xs)
    frac = min(1.0, args.ref_budget / ((steps + warm) * t_full))
    if frac < 1.0:
        shapes = [(n, max(min(N, 8 * cores), int(N * frac)), K) for n, N, K in shapes]
        weights = {n: weights[n][:N] for n, N, K in shapes}
    nbytes = sum(synth.algorithmic_bytes(1, N, K) for _, N, K in shapes)
    for _ in range(warm):
        cpu_pass(kind_ref, cores, shapes, weights, xs)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_pass(kind_ref, cores, shapes, weights, xs)
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    sample = (f"each step = the leading {100 * nbytes / step_bytes():.1f}% of the rows of all 8 projections "
              f"({nbytes / 1e6:.1f} MB), all host threads")
    line = {
        "metric": METRIC, "value": val, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": 1, "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "reference" if kind_ref else "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def capture_steps(torch, stream, one_step, n):
    """One CUDA graph of `n` consecutive steps.  A decode loop replays a graph of hundreds of launches per token; a
    graph of a single 8-launch step would pay the replay boundary (no dependent-launch overlap across it) every
    eight launches, which no caller of the path does."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for _ in range(n):
            one_step()
    return g


def timed_groups(torch, dist, stream, run_step, steps, groups, world, dev, after_step=None, steps_per_call=1):
    """`groups` back-to-back groups of exactly `steps` steps, each group between two CUDA events on `stream`
    (`run_step` performs `steps_per_call` steps: a replay of a graph of that many).
    Several ranks: a host barrier, then one untimed call (its flag barriers, or its collectives, line the
    devices up), then the groups; every group's time is the maximum over ranks.  Returns the per-group
    milliseconds (max over ranks)."""
    assert steps % steps_per_call == 0
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    run_step()
    if after_step:
        after_step(steps_per_call)
    evs = []
    for _ in range(groups):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps // steps_per_call):
            run_step()
        e1.record(stream)
        evs.append((e0, e1))
    stream.synchronize()
    if after_step:
        after_step(steps * groups)
    ms = torch.tensor([a.elapsed_time(b) for a, b in evs], dtype=torch.float64, device=dev)
    if dist:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
    torch.cuda.synchronize()
    return [float(v) for v in ms.cpu()]


def wall_groups(torch, dist, run_step, steps, groups, dev):
    """Host-clock version for the end-to-end passes (each pass ends with its own wait): per-group seconds,
    maximum over ranks."""
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    run_step()
    out = []
    for _ in range(groups):
        t0 = time.perf_counter()
        for _ in range(steps):
            run_step()
        out.append(time.perf_counter() - t0)
    t = torch.tensor(out, dtype=torch.float64, device=dev)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
    return [float(v) for v in t.cpu()]


def check_all_slots(torch, dist, rank, world, dev, names, dims, xs_h, weights_h, slices_of, M=1):
    """Before timing: every rank computes the expected values of ITS OWN slice with the CPU checker, the
    expectations are all-gathered, and every rank compares EVERY slot of its gather buffer (its own slice
    and the ones that arrived from the peers) with them."""
    from oracle import q4k_oracle as orc

    worst_rel, worst_abs, n = 0.0, 0.0, 0
    for name in names:
        N, K = dims[name]
        want_own = torch.from_numpy(orc.matmul(xs_h[name], weights_h[name], None, N, K, threads=4)).to(dev)
        if world > 1:
            want = torch.empty((world,) + tuple(want_own.shape), dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(want.view(-1), want_own.reshape(-1))
        else:
            want = want_own.unsqueeze(0)
        got = slices_of(name).reshape(want.shape)
        for p in range(world):
            rel = float((got[p] - want[p]).norm() / want[p].norm())
            mx = float((got[p] - want[p]).abs().max())
            assert rel <= 1e-3 and mx <= 2e-2, f"parity check failed before timing: {name} slot {p} on rank {rank}: rel_l2={rel} max_abs={mx}"
            worst_rel, worst_abs, n = max(worst_rel, rel), max(worst_abs, mx), n + 1
    return {"slots_checked_per_rank": n, "projections": list(names), "worst_rel_l2": worst_rel, "worst_max_abs": worst_abs,
            "against": "CPU checker, every rank's slice (expected values all-gathered)"}


def run_gpu_arm(args, rank, world, local_rank):
    import torch

    import backpack_b200 as bp

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    # the clock sampler starts NVML here, long before any timed region (its start-up takes milliseconds
    # and differs between ranks)
    sampler = ClockSampler(local_rank)
    ctx = bp.Q4KContext(local_rank)
    if args.no_pdl:
        from backpack_b200 import q4k as _q4k

        ctx.set_option(_q4k.OPT_STREAM_NO_PDL, 1)
    shapes = synth.LLAMA3_8B
    dims = {n: (N, K) for n, N, K in shapes}
    weights_h, xs_h = make_host_inputs(shapes, "config1", rank)
    dev = f"cuda:{local_rank}"
    from backpack_b200 import sharded

    steps, groups = max(args.steps, 1), max(args.groups, 1)
    W, X, Y, Yall, lin = {}, {}, {}, {}, {}
    pg = None
    if world > 1 and args.gather == "peer":
        # fused all-gather: the matmul epilogue stores every slice into all ranks' gather buffers
        pg = sharded.PeerGather(ctx, world, rank, {name: (1, N) for name, N, _ in shapes})
    # all activation vectors in one device buffer (64-float aligned views), so that the end-to-end pass of the
    # multi-rank run can bring them up with one copy
    x_off, x_total = {}, 0
    for name, _, K in shapes:
        x_off[name] = x_total
        x_total += (K + 63) // 64 * 64
    X_all = torch.zeros(x_total, dtype=torch.float32, device=dev)
    for name, N, K in shapes:
        W[name] = ctx.upload(bp.pack_q4k(weights_h[name], N, K))
        X[name] = X_all[x_off[name]: x_off[name] + K].view(1, K)
        X[name].copy_(torch.from_numpy(xs_h[name]))
        if world > 1:
            # weak scaling: this rank's shard has the single-GPU shape, the global matrix has world*N rows
            Yall[name] = torch.zeros((world, 1, N), dtype=torch.float32, device=dev)
            lin[name] = sharded.ShardedQ4KLinear(
                world * N, K, world, rank, W[name],
                lambda x, shard, out=None: ctx.matmul(x, shard, out=out))
        Y[name] = torch.zeros(1, N, dtype=torch.float32, device=dev)

    def one_pass():
        for name, N, K in shapes:
            if pg is not None:
                pg.matmul(name, X[name], W[name])               # local product, slices stored to every rank
            elif world > 1:
                lin[name].forward(X[name], Yall[name])          # local product + NCCL all-gather of the slices
            else:
                ctx.matmul(X[name], W[name], out=Y[name])
        if pg is not None:
            pg.barrier()                                        # one bounded flag barrier per step

    # correctness before timing: every slot of the gathered k and lm_head outputs (on one GPU: those two outputs)
    one_pass()
    torch.cuda.synchronize()
    parity = check_all_slots(
        torch, dist, rank, world, dev, ("k", "lm_head"), dims, xs_h, weights_h,
        (lambda n: pg.gathered(n)) if pg is not None else (lambda n: Yall[n]) if world > 1 else (lambda n: Y[n]))
    assert ctx.device_status() == 0

    # ---- resident (graph-replayed) timing --------------------------------
    stream = torch.cuda.Stream()
    graph = None
    sampler.start()
    with torch.cuda.stream(stream):
        for _ in range(3):
            one_pass()
        stream.synchronize()
        if world == 1 or args.graph_multi or pg is not None:
            graph = torch.cuda.CUDAGraph()
            steps_before = pg.steps if pg is not None else 0
            with torch.cuda.graph(graph, stream=stream):
                one_pass()
            if pg is not None:
                pg.steps = steps_before                         # capturing enqueued nothing
        # (NCCL gather: the step is timed as eager launches unless --graph-multi is given; capturing the NCCL
        # all-gathers together with the dependent-launch kernels into one graph did not complete on this pool)
        run_step = graph.replay if graph is not None else one_pass
        note = pg.note_replays if (pg is not None and graph is not None) else None
        for _ in range(max(args.warmup, 3)):
            run_step()
        if note:
            note(max(args.warmup, 3))
        stream.synchronize()
        ctx.launch_count(reset=True)
        if graph is not None:
            # the timed groups replay ONE graph of `steps` steps each
            steps_before = pg.steps if pg is not None else 0
            graph_k = capture_steps(torch, stream, one_pass, steps)
            if pg is not None:
                pg.steps = steps_before
            group_ms = timed_groups(torch, dist, stream, graph_k.replay, steps, groups, world, dev, note, steps_per_call=steps)
        else:
            group_ms = timed_groups(torch, dist, stream, run_step, steps, groups, world, dev, note)
        ms = float(np.median(group_ms))

        # the gathered outputs after the timed replays are still right (slot check on the last step)
        if pg is not None:
            check_all_slots(torch, dist, rank, world, dev, ("k",), dims, xs_h, weights_h, lambda n: pg.gathered(n))

        # ---- kernel-only duration of the dominant kernel (no collectives) ----
        def kernels_only():
            for name, N, K in shapes:
                ctx.matmul(X[name], W[name], out=Y[name])

        kgraph = capture_steps(torch, stream, kernels_only, steps)
        ctx.launch_count(reset=True)
        kernels_only()
        launches_per_step = ctx.launch_count()
        kgraph.replay()
        kernel_ms = float(np.median(timed_groups(torch, dist, stream, kgraph.replay, steps, groups, world, dev, steps_per_call=steps)))

        # ---- end to end through the host-buffer entry point ---------------
        xs_pin = {n: torch.from_numpy(xs_h[n]).pin_memory() for n, _, _ in shapes}
        ys_pin = {n: torch.zeros(1, N, dtype=torch.float32).pin_memory() for n, N, _ in shapes}
        xs_np = {n: xs_pin[n].numpy() for n in xs_pin}
        ys_np = {n: ys_pin[n].numpy() for n in ys_pin}
        d2h = sum(N * 4 for _, N, _ in shapes)

        if world == 1:
            # the user-facing call: one dispatch list on host buffers (uploads, kernels, read-backs, one wait)
            batch = ctx.make_host_batch([(xs_np[n], W[n], ys_np[n], None) for n, _, _ in shapes])

            def e2e_pass():
                ctx.matmul_host_batch(batch)
            e2e_note = "one bpq4k_matmul_host_batch_f32 call per step on pinned host buffers"
        elif pg is not None and graph is not None:
            # one copy up (all activation vectors), the recorded step (matmuls storing into every rank's gather
            # buffer + flag barrier), one copy down: this rank's 1/world share of the gathered result (a
            # contiguous range of the step's half of the gather buffer, most of it produced by peers), so that
            # the whole gathered output of the job lands in host memory once per step.  The slots are
            # double-buffered, so no second barrier is needed before the next step's stores.
            x_all_pin = torch.zeros(x_total, dtype=torch.float32).pin_memory()
            for name, _, K in shapes:
                x_all_pin[x_off[name]: x_off[name] + K] = xs_pin[name].view(-1)
            share = pg.half // world
            y_share_pin = torch.zeros(share, dtype=torch.float32).pin_memory()
            r_share = (rank + 1) % world
            d2h = share * 4

            def e2e_pass():
                X_all.copy_(x_all_pin, non_blocking=True)
                graph.replay()
                pg.note_replays(1)
                base = ((pg.steps - 1) % 2) * pg.half + r_share * share
                y_share_pin.copy_(pg.buf[base: base + share], non_blocking=True)
                torch.cuda.current_stream().synchronize()
            e2e_note = ("per rank: one copy of all activation vectors up, the recorded step, one copy of this rank's "
                        "1/world share of the gathered outputs down, one wait")
        else:
            yall_pin = {n: torch.zeros(world * N, dtype=torch.float32).pin_memory() for n, N, _ in shapes}
            d2h = world * d2h

            def e2e_pass():
                for name, N, K in shapes:
                    X[name].copy_(xs_pin[name], non_blocking=True)
                    lin[name].forward(X[name], Yall[name])
                    yall_pin[name].copy_(Yall[name].view(-1), non_blocking=True)
                torch.cuda.current_stream().synchronize()
            e2e_note = "per projection: copy up, matmul, NCCL all-gather, copy of the whole gathered output down"

        for _ in range(3):
            e2e_pass()
        e2e_steps = max(1, min(steps, 200))
        e2e_s = float(np.median(wall_groups(torch, dist, e2e_pass, e2e_steps, groups, dev)))
        if world == 1:
            want = None
            from oracle import q4k_oracle as orc

            want = orc.matmul(xs_h["k"], weights_h["k"], None, 1024, 4096)
            rel = float(np.linalg.norm(ys_np["k"] - want) / np.linalg.norm(want))
            assert rel < 1e-3, f"end-to-end output differs from the CPU checker: rel_l2={rel}"
    sampler.stop()

    extras = {}
    if world == 1:
        extras["per_shape"] = measure_per_shape(ctx, torch, bp, shapes, weights_h, dev)
        extras["fused_projections"] = measure_fused_projections(ctx, torch, bp, shapes, weights_h, X, dev, stream, steps)
        extras["config0"] = measure_config0(ctx, torch, bp, weights_h["q"], dev)
        if not args.no_prefill:
            extras["prefill"] = measure_prefill(ctx, torch, shapes, W, dev, weights_h=weights_h)
        if not args.no_siblings:
            extras["small_batch"] = measure_small_batch(ctx, torch, W["lm_head"], dev)
            extras["kquant_siblings"] = measure_siblings(ctx, torch, dev)
            extras["fused_prologues"] = measure_fusions(ctx, torch, dev)
            extras["routed_experts"] = measure_routed_experts(ctx, torch, dev)
            extras["gguf_upload"] = measure_gguf_upload(ctx)
    # free the config-1 tensors before the 70B-shaped ones go up
    if pg is not None:
        pg.close()
    del W, Y, Yall, lin
    torch.cuda.empty_cache()
    if not args.no_config4:
        extras["config4"] = measure_config4(ctx, torch, dist, bp, sharded, rank, world, dev, args)

    if rank == 0:
        peak, peak_src = load_peaks()
        sb = step_bytes()
        value = world * sb * steps / (ms * 1e-3) / 1e9
        e2e_val = world * sb * e2e_steps / e2e_s / 1e9
        per_launch_bytes = sb / launches_per_step
        per_launch_s = kernel_ms * 1e-3 / (steps * launches_per_step)
        achieved = per_launch_bytes / per_launch_s / 1e9
        cpu = cpu_baseline(args.cpu_budget, shapes, weights_h, xs_h)
        h2d = sum(K * 4 for _, _, K in shapes)
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "traffic": per_launch_bytes * TRAFFIC_RATIO,
                    "traffic_note": "ncu dram read+write of a 151 MB launch, scaled to the average launch by bytes",
                    "peak_source": peak_src,
                    "kernel": "q4k matmul (M=1)", "launches_per_step": launches_per_step,
                    "avg_launch_us": per_launch_s * 1e6, "alg_bytes_per_launch": per_launch_bytes}
        fp = extras.get("fused_projections")
        if fp:
            # the same step as the reference's loader lays the weights out (Q+K+V and gate+up fused by rows): 5 launches
            roofline["fused_step"] = {"launches_per_step": 5, "achieved": fp["value"], "frac": fp["frac_of_hbm_peak"],
                                      "avg_launch_us": fp["ms_per_step"] * 1e3 / 5}
        pf = extras.get("prefill")
        if pf:
            roofline["prefill"] = {"bound": "tensor", "unit": "TFLOP/s", "peak": pf.get("bf16_tflops"),
                                   "peak_sustained": pf.get("bf16_tflops_sustained"),
                                   "modes": {k: {"achieved": v["tflops"], "frac": v["frac_of_burst_peak"],
                                                 "meets_float_tolerance": v["meets_float_tolerance"]}
                                             for k, v in pf["modes"].items()}}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "gpu_launches": int(launches_per_step * steps * groups),
            "roofline": roofline,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_s * 1e3 / e2e_steps, "what": e2e_note},
            "cpu_baseline": cpu,
            "clocks": sampler.summary(),
            "parity_before_timing": parity,
            "config": {"workload": WORKLOAD, "M": 1, "projections": [list(s) for s in shapes],
                       "bytes_per_step_per_gpu": sb, "weight_bytes_per_step_per_gpu": weight_bytes_total(),
                       "l2": "inputs larger than L2 (418 MB of weights per pass vs 126 MB L2)",
                       "timing": f"median of {groups} back-to-back groups of {steps} steps each (CUDA events, max over ranks per group); "
                                 f"a group is one replay of a CUDA graph of {steps} steps",
                       "group_ms": group_ms,
                       "replay": "cuda graph" if graph is not None else "eager launches",
                       "sharding": ("none" if world == 1 else
                                    "rows (N) per rank, every rank a full single-GPU-sized shard (weak); slices stored into "
                                    "every rank's double-buffered gather slots by the matmul epilogue (peer memory), one "
                                    "flag barrier per step" if pg is not None else
                                    "rows (N) per rank; NCCL all-gather per projection")},
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def graph_time_us(torch, stream, fn, n_in_graph, replays=5):
    """Capture `fn` (which launches n_in_graph calls) into a graph, replay it, return us per call."""
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        g.replay()
        ts = []
        for _ in range(replays):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            stream.synchronize()
            ts.append(e0.elapsed_time(e1))
    return float(np.median(ts)) * 1e3 / n_in_graph


def measure_fused_projections(ctx, torch, bp, shapes, weights_h, X, dev, stream, steps):
    """The same bytes with Q+K+V and gate+up fused by rows, as the reference's loader fuses them (fuseKQ):
    five launches instead of eight."""
    groups = [("qkv", ["q", "k", "v"]), ("o", ["o"]), ("gate_up", ["gate", "up"]), ("down", ["down"]),
              ("lm_head", ["lm_head"])]
    dims = {n: (N, K) for n, N, K in shapes}
    FW, FX, FY = {}, {}, {}
    for gname, members in groups:
        packed = None
        for mname in members:
            pk = bp.pack_q4k(weights_h[mname], *dims[mname])
            packed = pk if packed is None else bp.fuse_kq(packed, pk)
        FW[gname] = ctx.upload(packed)
        FX[gname] = X[members[0]]
        FY[gname] = torch.zeros(1, packed.N, dtype=torch.float32, device=dev)

    def fused_pass():
        for gname, _ in groups:
            ctx.matmul(FX[gname], FW[gname], out=FY[gname])

    # timed like the headline: back-to-back replays between two events (a single replay between synchronisations
    # would charge the launch of the first kernel, which the dependent launches otherwise overlap)
    with torch.cuda.stream(stream):
        fused_pass()
        stream.synchronize()
        fg = capture_steps(torch, stream, fused_pass, steps)
        fg.replay()
        us = float(np.median(timed_groups(torch, None, stream, fg.replay, steps, 5, 1, dev, steps_per_call=steps))) * 1e3 / steps
    fbytes = sum(synth.algorithmic_bytes(1, FW[g].N, FW[g].K) for g, _ in groups)
    peak, _ = load_peaks()
    return {"what": "same weights, Q+K+V and gate+up fused by rows as the reference's loader does: 5 launches",
            "ms_per_step": us * 1e-3, "value": fbytes / us / 1e3, "unit": UNIT, "frac_of_hbm_peak": fbytes / us / 1e3 / peak}


def measure_config0(ctx, torch, bp, raw_q, dev):
    """Configuration 0: the single 4096 x 4096 GEMV (9.4 MB).  HBM-cold: 32 copies of the weight walked in one graph
    (302 MB > L2); L2-warm: the same copy 32 times."""
    N = K = 4096
    packed = bp.pack_q4k(raw_q, N, K)
    Ws = [ctx.upload(packed) for _ in range(32)]
    x = torch.randn(1, K, device=dev, generator=torch.Generator(device=dev).manual_seed(3))
    y = torch.empty(1, N, device=dev)
    stream = torch.cuda.Stream(device=dev)
    cold = graph_time_us(torch, stream, lambda: [ctx.matmul(x, w, out=y) for w in Ws], 32)
    warm = graph_time_us(torch, stream, lambda: [ctx.matmul(x, Ws[0], out=y) for _ in range(32)], 32)
    b = synth.algorithmic_bytes(1, N, K)
    peak, _ = load_peaks()
    return {"workload": "single GEMV 4096 x 4096, M=1 (config 0)", "alg_bytes": b,
            "hbm_cold": {"us_per_launch": cold, "value": b / cold / 1e3, "unit": UNIT, "frac_of_hbm_peak": b / cold / 1e3 / peak},
            "l2_warm": {"us_per_launch": warm, "value": b / warm / 1e3, "unit": UNIT}}


def measure_per_shape(ctx, torch, bp, shapes, weights_h, dev):
    """Configuration 1 shape by shape: each distinct projection shape alone, M = 1, launched back to back over enough
    copies of the weight that every launch streams from HBM (>= 400 MB walked per graph replay)."""
    peak, _ = load_peaks()
    out = {"unit": UNIT, "what": "one launch per copy of the weight, >= 400 MB of copies walked per replay (HBM-cold)", "shapes": {}}
    stream = torch.cuda.Stream(device=dev)
    seen = {}
    for name, N, K in shapes:
        if (N, K) in seen:
            seen[(N, K)].append(name)
            continue
        seen[(N, K)] = [name]
        wb = synth.weight_bytes(N, K)
        nc = max(2, min(160, int(400e6 // wb) + 1))
        packed = bp.pack_q4k(weights_h[name], N, K)
        Ws = [ctx.upload(packed) for _ in range(nc)]
        x = torch.randn(1, K, device=dev, generator=torch.Generator(device=dev).manual_seed(11))
        y = torch.empty(1, N, device=dev)
        reps = max(1, 64 // nc)
        us = graph_time_us(torch, stream, lambda: [ctx.matmul(x, w, out=y) for _ in range(reps) for w in Ws], nc * reps)
        b = synth.algorithmic_bytes(1, N, K)
        out["shapes"][f"{N}x{K}"] = {"projections": seen[(N, K)], "alg_bytes": b, "us_per_launch": us, "value": b / us / 1e3,
                                    "frac_of_hbm_peak": b / us / 1e3 / peak}
        del Ws
        torch.cuda.empty_cache()
    return out


def measure_small_batch(ctx, torch, w_head, dev):
    """Decode with several activation rows (M = 2..16) on the output head 128256 x 4096: one weight pass per call,
    algorithmic GB/s in graph replay (296 MB per launch > L2)."""
    peak, _ = load_peaks()
    N, K = w_head.N, w_head.K
    stream = torch.cuda.Stream(device=dev)
    out = {"workload": f"{N} x {K}, Q4_K, M rows per call", "unit": UNIT, "rows": {}}
    for M in (2, 4, 8, 12, 16):
        x = torch.randn(M, K, device=dev, generator=torch.Generator(device=dev).manual_seed(M))
        y = torch.empty(M, N, device=dev)
        ctx.launch_count(reset=True)
        ctx.matmul(x, w_head, out=y)
        launches = ctx.launch_count()
        us = graph_time_us(torch, stream, lambda: [ctx.matmul(x, w_head, out=y) for _ in range(4)], 4)
        gbs = synth.algorithmic_bytes(M, N, K) / us / 1e3
        out["rows"][str(M)] = {"us_per_call": us, "launches_per_call": launches, "value": gbs, "frac_of_hbm_peak": gbs / peak}
    return out


def measure_config4(ctx, torch, dist, bp, sharded, rank, world, dev, args):
    """Configuration 4: the Llama-3-70B-shaped projections, M = 1 and M = 8, rows split N/G per rank (a STRONG
    split of fixed matrices over G = world GPUs; every N is divisible by 8).  Per M: the kernels alone, the step
    with the fused peer-store gather and one flag barrier, the same step with one eager NCCL all-gather per
    projection, and end to end from pinned host memory.  Aggregate algorithmic GB/s over all ranks."""
    shapes = synth.LLAMA3_70B
    peak, peak_src = load_peaks()
    steps, groups = max(min(args.steps, 50), 1), max(min(args.groups, 5), 1)
    stream = torch.cuda.Stream(device=dev)
    Wd, raws = {}, {}
    for name, N, K in shapes:
        ns = N // world
        # this rank's rows of the global matrix: the global matrix is the concatenation of the ranks' draws
        raws[name] = synth.make_q4k_weights(ns, K, synth.shape_seed("config4", name) + rank)
        Wd[name] = ctx.upload(bp.pack_q4k(raws[name], ns, K))
    out = {"workload": "llama3-70b decode projections (config 4), Q4_K, rows split N/G per rank (strong)", "G": world,
           "unit": UNIT, "peak_gbs": peak, "peak_source": peak_src, "steps": steps, "groups": groups}
    for M in (1, 8):
        xs_h = {name: synth.make_activations(M, K, synth.shape_seed("config4", name + ".x") + M) for name, _, K in shapes}
        x_off, x_total = {}, 0
        for name, _, K in shapes:
            x_off[name] = x_total
            x_total += M * K
        X_all = torch.zeros(x_total, dtype=torch.float32, device=dev)
        X = {}
        for name, _, K in shapes:
            X[name] = X_all[x_off[name]: x_off[name] + M * K].view(M, K)
            X[name].copy_(torch.from_numpy(xs_h[name]))
        Y = {name: torch.zeros(M, N // world, dtype=torch.float32, device=dev) for name, N, _ in shapes}
        total_bytes = sum(synth.algorithmic_bytes(M, N, K) for _, N, K in shapes)   # whole job, all ranks together
        row = {}

        def kernels_only():
            for name, _, _ in shapes:
                ctx.matmul(X[name], Wd[name], out=Y[name])

        with torch.cuda.stream(stream):
            kernels_only()
            stream.synchronize()
            kg = capture_steps(torch, stream, kernels_only, steps)
            kg.replay()
            kms = float(np.median(timed_groups(torch, dist, stream, kg.replay, steps, groups, world, dev, steps_per_call=steps))) / steps
        row["kernels_only"] = {"ms_per_step": kms, "value": total_bytes / kms / 1e6, "frac_of_hbm_peak": total_bytes / kms / 1e6 / (peak * world)}
        dims = {name: (N // world, K) for name, N, K in shapes}
        if world == 1:
            row["parity"] = check_all_slots(torch, None, rank, 1, dev, ("k", "lm_head"), dims, xs_h, raws, lambda n: Y[n], M)
        else:
            pg = sharded.PeerGather(ctx, world, rank, {name: (M, N // world) for name, N, _ in shapes})

            def peer_step():
                for name, _, _ in shapes:
                    pg.matmul(name, X[name], Wd[name])
                pg.barrier()

            peer_step()
            torch.cuda.synchronize()
            row["parity"] = check_all_slots(torch, dist, rank, world, dev, ("k", "lm_head"), dims, xs_h, raws,
                                            lambda n: pg.gathered(n), M)
            with torch.cuda.stream(stream):
                peer_step()
                stream.synchronize()
                before = pg.steps
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    peer_step()
                pg.steps = before
                for _ in range(3):
                    g.replay()
                pg.note_replays(3)
                before = pg.steps
                gk = capture_steps(torch, stream, peer_step, steps)
                pg.steps = before
                pms = float(np.median(timed_groups(torch, dist, stream, gk.replay, steps, groups, world, dev, pg.note_replays, steps_per_call=steps))) / steps
            check_all_slots(torch, dist, rank, world, dev, ("k",), dims, xs_h, raws, lambda n: pg.gathered(n), M)
            row["peer_gather"] = {"ms_per_step": pms, "value": total_bytes / pms / 1e6,
                                  "frac_of_hbm_peak": total_bytes / pms / 1e6 / (peak * world),
                                  "what": "matmul epilogues store the slices to every rank (double-buffered slots), one flag barrier per step, one CUDA graph"}
            # end to end: activations up, the recorded step, this rank's share of the gathered result down
            x_pin = torch.zeros(x_total, dtype=torch.float32).pin_memory()
            x_pin.copy_(X_all.cpu())
            share = pg.half // world
            y_pin = torch.zeros(share, dtype=torch.float32).pin_memory()
            r_share = (rank + 1) % world

            def e2e_pass():
                X_all.copy_(x_pin, non_blocking=True)
                g.replay()
                pg.note_replays(1)
                base = ((pg.steps - 1) % 2) * pg.half + r_share * share
                y_pin.copy_(pg.buf[base: base + share], non_blocking=True)
                torch.cuda.current_stream().synchronize()

            with torch.cuda.stream(stream):
                for _ in range(3):
                    e2e_pass()
                es = float(np.median(wall_groups(torch, dist, e2e_pass, steps, groups, dev))) / steps
            row["e2e"] = {"ms_per_step": es * 1e3, "value": total_bytes / es / 1e9, "h2d_bytes_per_step": x_total * 4,
                          "d2h_bytes_per_step": share * 4}
            pg.close()
            # NCCL baseline: one eager all-gather per projection (never captured together with the kernels)
            Yall = {name: torch.zeros((world, M, N // world), dtype=torch.float32, device=dev) for name, N, _ in shapes}
            lin = {name: sharded.ShardedQ4KLinear(N, K, world, rank, Wd[name],
                                                   lambda x, shard, out=None: ctx.matmul(x, shard, out=out))
                   for name, N, K in shapes}

            def nccl_step():
                for name, _, _ in shapes:
                    lin[name].forward(X[name], Yall[name])

            with torch.cuda.stream(stream):
                for _ in range(3):
                    nccl_step()
                stream.synchronize()
                nms = float(np.median(timed_groups(torch, dist, stream, nccl_step, steps, groups, world, dev))) / steps
            check_all_slots(torch, dist, rank, world, dev, ("k",), dims, xs_h, raws, lambda n: Yall[n], M)
            row["nccl_gather"] = {"ms_per_step": nms, "value": total_bytes / nms / 1e6,
                                  "what": "one eager NCCL all-gather per projection after its matmul"}
            del Yall, lin
        if world == 1:
            pins = [(torch.from_numpy(xs_h[n]).pin_memory(), torch.zeros(M, N, dtype=torch.float32).pin_memory()) for n, N, _ in shapes]
            batch = ctx.make_host_batch([(p[0].numpy(), Wd[n], p[1].numpy(), None) for p, (n, _, _) in zip(pins, shapes)])
            for _ in range(3):
                ctx.matmul_host_batch(batch)
            es = float(np.median(wall_groups(torch, None, lambda: ctx.matmul_host_batch(batch), steps, groups, dev))) / steps
            row["e2e"] = {"ms_per_step": es * 1e3, "value": total_bytes / es / 1e9, "h2d_bytes_per_step": x_total * 4,
                          "d2h_bytes_per_step": sum(M * N * 4 for _, N, _ in shapes)}
        out[f"M{M}"] = row
        del X, Y, X_all
    del Wd
    torch.cuda.empty_cache()
    return out


def measure_gguf_upload(ctx):
    """File -> HBM rate of the GGUF tensor loader on the output head (128256 x 4096, Q4_K, 295 MB) and on
    its Q6_K form re-spaced into the padded layout on the device.  The file is written to the temp
    directory just before, so it is read from the page cache: the figure is the pinned double-buffer
    copy path, not a disk."""
    import struct
    import tempfile

    from backpack_b200 import q4k, synth
    from backpack_b200.gguf import GGUFFile

    def s(b):
        return struct.pack("<Q", len(b)) + b

    N, K = 128256, 4096
    out = {"unit": "GB/s of file bytes", "tensors": {}}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "head.gguf")
        q4 = synth.make_q4k_weights(N, K, 41)
        q6 = synth.make_kq_weights(q4k.Q6_K, N, K, 42)
        hdr = struct.pack("<IIQQ", 0x46554747, 3, 2, 0)
        hdr += s(b"output.q4k") + struct.pack("<IQQIQ", 2, K, N, 12, 0)
        off6 = (q4.nbytes + 31) // 32 * 32
        hdr += s(b"output.q6k") + struct.pack("<IQQIQ", 2, K, N, 14, off6)
        hdr += b"\0" * ((-len(hdr)) % 32)
        with open(path, "wb") as f:
            f.write(hdr)
            f.write(q4.tobytes())
            f.write(b"\0" * (off6 - q4.nbytes))
            f.write(q6.tobytes())
        g = GGUFFile(path)
        for name, layout, nbytes in (("output.q4k", 0, q4.nbytes), ("output.q6k", q4k.Q6_K_PADDED, q6.nbytes)):
            best = 1e9
            for _ in range(3):
                t0 = time.perf_counter()
                t = g.upload(ctx, name, layout)
                best = min(best, time.perf_counter() - t0)
                t.free()
            out["tensors"][name] = {"file_bytes": int(nbytes), "seconds": best, "value": nbytes / best / 1e9}
        g.close()
    return out


def measure_fusions(ctx, torch, dev):
    """What the fused prologues cost on top of the plain single-row matmul (graph replay over enough
    weight copies to stay out of L2): Q+K+V with the RMSNorm prologue, the down projection with the
    silu*up prologue and the residual epilogue.  The reference runs each of these steps as its own
    dispatch; here each is folded into the matmul launch."""
    import backpack_b200 as bp
    from backpack_b200 import q4k, synth

    out = {"unit": "us per launch", "cases": {}}
    for name, N, K, kind, with_res in (("qkv_rmsnorm", 6144, 4096, q4k.PROLOGUE_RMSNORM, False),
                                       ("down_silu_mul_residual", 4096, 14336, q4k.PROLOGUE_SILU_MUL, True)):
        ncopies = int(400e6 // synth.weight_bytes(N, K)) + 1
        packed = bp.pack_q4k(synth.make_q4k_weights(N, K, 31), N, K)
        Ws = [ctx.upload(packed) for _ in range(ncopies)]
        g0 = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(1, K, device=dev, generator=g0)
        aux = torch.randn(K, device=dev, generator=g0)
        res = torch.randn(N, device=dev, generator=g0) if with_res else None
        y = torch.empty(1, N, device=dev)
        row = {}
        for label, fn in (("plain", lambda w: ctx.matmul(x, w, out=y)),
                          ("fused", lambda w: ctx.matmul_fused(x, w, kind, aux=aux, eps=1e-5, residual=res, out=y))):
            for w in Ws[:2]:
                fn(w)
            torch.cuda.synchronize()
            stream = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(stream):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(2 * ncopies):
                        fn(Ws[i % ncopies])
                g.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                g.replay()
                e1.record(stream)
                stream.synchronize()
            row[label] = e0.elapsed_time(e1) * 1e3 / (2 * ncopies)
        out["cases"][name] = row
        del Ws
        torch.cuda.empty_cache()
    return out


def measure_routed_experts(ctx, torch, dev):
    """Configuration 3: 128 experts with gate/up [768, 2048] and down [2048, 768] stacks (113 MB each), 8 tokens
    routed to 8 distinct experts each.  Times (a) the three expert-indexed matmuls alone and (b) the whole
    routed-expert step (gate+up in one launch, down with the silu*up prologue, weighted accumulate) -- the
    reference issues 6 dispatches per slot, 384 for this step.  Graph replay over three copies of the stacks and
    six routings, so that a replayed step finds none of its experts in L2.  Algorithmic bytes count each distinct
    expert touched once per matrix."""
    import backpack_b200 as bp
    from backpack_b200 import synth

    peak, peak_src = load_peaks()
    E, F, H, T, topk, ncopies = 128, 768, 2048, 8, 8, 3
    stacks = []
    for N, K, seed in ((E * F, H, 41), (E * F, H, 42), (E * H, F, 43)):
        packed = bp.pack_q4k(synth.make_q4k_weights(N, K, seed), N, K)
        stacks.append([ctx.upload(packed) for _ in range(ncopies)])
    n = 2 * ncopies
    routes = [synth.make_moe_routing(T, E, topk, 100 + i).reshape(-1) for i in range(n)]
    ids = [torch.from_numpy(r.astype(np.int32)).to(dev) for r in routes]
    offg = [torch.from_numpy((r * F).astype(np.int32)).to(dev) for r in routes]
    offd = [torch.from_numpy((r * H).astype(np.int32)).to(dev) for r in routes]
    gen = torch.Generator(device=dev).manual_seed(9)
    x = torch.randn(T, H, device=dev, generator=gen) * 0.05
    act = torch.randn(T * topk, F, device=dev, generator=gen)
    rw = torch.softmax(torch.randn(T, topk, device=dev, generator=gen), dim=1).reshape(-1).contiguous()
    x_rows = torch.arange(T, device=dev, dtype=torch.int32).repeat_interleave(topk)
    yg, yu = torch.empty(T * topk, F, device=dev), torch.empty(T * topk, F, device=dev)
    yd, y = torch.empty(T * topk, H, device=dev), torch.zeros(T, H, device=dev)
    work = torch.empty(T * topk * (2 * F + H), device=dev)

    def three_matmuls(i):
        c, r = i % ncopies, i % n
        ctx.matmul_moe(x, stacks[0][c], F, offg[r], x_rows=x_rows, out=yg)
        ctx.matmul_moe(x, stacks[1][c], F, offg[r], x_rows=x_rows, out=yu)
        ctx.matmul_moe(act, stacks[2][c], H, offd[r], out=yd)

    def whole_step(i):
        c = i % ncopies
        ctx.moe_ffn(x, stacks[0][c], stacks[1][c], stacks[2][c], ids[i % n], rw, y, E, work=work)

    distinct = float(np.mean([len(np.unique(r)) for r in routes]))
    weight_bytes = distinct * 3 * synth.weight_bytes(F, H)
    out = {"workload": "128 experts, gate/up 768 x 2048 and down 2048 x 768 (Q4_K), 8 tokens x 8 experts",
           "distinct_experts_per_step": distinct, "weight_bytes_per_step": weight_bytes, "peak_gbs": peak,
           "peak_source": peak_src, "reference_dispatches_per_step": 6 * T * topk}
    for name, fn in (("three_matmuls", three_matmuls), ("whole_step", whole_step)):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        ctx.launch_count(reset=True)
        fn(0)
        launches = ctx.launch_count()
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(n):
                    fn(i)
            g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(5):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (5 * n)
        gbs = weight_bytes / us / 1e3
        out[name] = {"us_per_step": us, "launches_per_step": launches, "value": gbs, "unit": UNIT, "frac_of_hbm_peak": gbs / peak}
    del stacks
    torch.cuda.empty_cache()
    return out


def measure_siblings(ctx, torch, dev, reps=8):
    """The Q5_K and Q6_K versions of the output-head projection (128256 x 4096, M = 1): real
    "Q4_K_M" files keep that tensor in Q6_K.  Algorithmic GB/s counts the file format's bytes per
    block (176 and 210); each weight is larger than L2, so back-to-back launches stream from HBM."""
    import backpack_b200 as bp
    from backpack_b200 import q4k, synth

    peak, peak_src = load_peaks()
    N, K = 128256, 4096
    x = torch.randn(1, K, device=dev, generator=torch.Generator(device=dev).manual_seed(11))
    y = torch.empty(1, N, device=dev)
    out = {"workload": "output head 128256 x 4096, M=1", "peak_gbs": peak, "peak_source": peak_src, "types": {}}
    for name, layout, ftype in (("q5_k", q4k.Q5_K, q4k.Q5_K), ("q6_k", q4k.Q6_K_PADDED, q4k.Q6_K)):
        w = ctx.upload(bp.pack_kq(layout, synth.make_kq_weights(ftype, N, K, 21), N, K))
        for _ in range(3):
            ctx.matmul(x, w, out=y)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(reps):
                    ctx.matmul(x, w, out=y)
            g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        gbs = synth.kq_algorithmic_bytes(ftype, 1, N, K) / us / 1e3
        out["types"][name] = {"us_per_launch": us, "value": gbs, "unit": UNIT, "frac_of_hbm_peak": gbs / peak,
                              "device_layout": "file format" if layout == ftype else "blocks padded to 224 bytes"}
        del w
        torch.cuda.empty_cache()
    return out


def measure_prefill(ctx, torch, shapes, W, dev, M=512, reps=5, weights_h=None):
    """Config 2: the same projections at M = 512 through the tensor-core kernel; useful TFLOP/s
    (2*M*N*K, extra passes not counted) per precision mode, summed over the eight projections."""
    from backpack_b200 import q4k

    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        peaks = {"bf16_tflops": p.get("bf16_tflops"), "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                 "peak_source": "measured"}
    except Exception:
        peaks = {"bf16_tflops": FALLBACK_PEAKS["bf16_tflops"], "bf16_tflops_sustained": None, "peak_source": "fallback"}
    xs = {K: torch.randn(M, K, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) for K in {k for _, _, k in shapes}}
    ys = {n: torch.empty(M, N, device=dev) for n, N, _ in shapes}
    flops = sum(2.0 * M * N * K for _, N, K in shapes)
    out = {"workload": "llama3-8b prefill projections, M=512, Q4_K (config 2)", "M": M, "flops_per_pass": flops, **peaks,
           "modes": {}}
    for mode, name in ((q4k.PREFILL_F16X3, "f16x3"), (q4k.PREFILL_F16, "f16"), (q4k.PREFILL_BF16, "bf16")):
        ctx.set_option(q4k.OPT_PREFILL_MODE, mode)

        def one_pass():
            for n, N, K in shapes:
                ctx.matmul(xs[K], W[n], out=ys[n])

        for _ in range(2):
            one_pass()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            one_pass()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        tf = flops / (ms * 1e-3) / 1e12
        out["modes"][name] = {"ms_per_pass": ms, "tflops": tf,
                              "frac_of_burst_peak": tf / peaks["bf16_tflops"] if peaks.get("bf16_tflops") else None,
                              "meets_float_tolerance": name == "f16x3"}
        if weights_h is not None:
            # error of this mode against the CPU checker (the reference's float dot) on the first 64 weight rows of a
            # K = 4096 and of the K = 14336 projection, all 512 activation rows
            from oracle import q4k_oracle as orc
            errs = {}
            for pname in ("gate", "down"):
                N, K = W[pname].N, W[pname].K
                rows = 64
                want = orc.matmul(xs[K].cpu().numpy(), np.ascontiguousarray(weights_h[pname][:rows]), None, rows, K, threads=4)
                got = ys[pname][:, :rows].cpu().numpy()
                errs[f"K={K}"] = {"rel_l2": float(np.linalg.norm(got - want) / np.linalg.norm(want)),
                                  "max_abs": float(np.abs(got - want).max()), "out_rms": float(np.sqrt(np.mean(want * want)))}
            out["modes"][name]["error_vs_checker"] = errs
    # the two other forms of the single-pass kernel (same bits, kept for comparison): bfloat16, the whole pass
    out["variants_bf16"] = {}
    ctx.set_option(q4k.OPT_PREFILL_MODE, q4k.PREFILL_BF16)
    for variant, name in ((q4k.PREFILL_CTA_PAIR, "cta_pair_cta_group2"), (q4k.PREFILL_TMEM_WEIGHTS, "weights_in_tmem")):
        ctx.set_option(q4k.OPT_PREFILL_VARIANT, variant)
        for n, N, K in shapes:
            ctx.matmul(xs[K], W[n], out=ys[n])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for n, N, K in shapes:
                ctx.matmul(xs[K], W[n], out=ys[n])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        out["variants_bf16"][name] = {"ms_per_pass": ms, "tflops": flops / (ms * 1e-3) / 1e12}
    ctx.set_option(q4k.OPT_PREFILL_VARIANT, q4k.PREFILL_ONE_CTA)
    ctx.set_option(q4k.OPT_PREFILL_MODE, q4k.PREFILL_F16X3)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=10.0, help="seconds of CPU work for cpu_baseline")
    ap.add_argument("--ref-budget", type=float, default=120.0, help="seconds the --impl reference run may take")
    ap.add_argument("--no-prefill", action="store_true", help="skip the M=512 (config 2) measurement")
    ap.add_argument("--no-siblings", action="store_true", help="skip the small-batch, Q5_K / Q6_K, prologue, routed-expert and loader measurements")
    ap.add_argument("--no-config4", action="store_true", help="skip the 70B-shaped strong-split measurement (config 4)")
    ap.add_argument("--groups", type=int, default=10, help="timed groups of --steps steps each; the median group is reported")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="several ranks: fused peer-store all-gather (default) or one NCCL all-gather per projection")
    ap.add_argument("--graph-multi", action="store_true", help="with several ranks, replay the step from a CUDA graph too")
    ap.add_argument("--no-pdl", action="store_true", help="launch the streaming kernel without programmatic dependent launch")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
