"""N-sharded matmul on two real GPUs over NCCL (skipped on boxes with one GPU)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import backpack_b200 as bp
    from backpack_b200 import sharded, synth
    from oracle import q4k_oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    ctx = bp.Q4KContext(rank)
    ok = True
    for (M, N, K) in [(1, 8192, 4096), (8, 1024, 8192), (1, 1000, 1024), (3, 130, 512)]:
        raw = synth.make_q4k_weights(N, K, 5)
        x = synth.make_activations(M, K, 6)
        lin = sharded.make_cuda_linear(ctx, raw, N, K, world, rank)
        y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        want = orc.matmul(x, raw, None, N, K, threads=4)
        rel = np.linalg.norm(y - want) / np.linalg.norm(want)
        ok = ok and y.shape == (M, N) and rel <= 1e-3 and np.abs(y - want).max() <= 2e-2
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_sharded_matches_checker():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, 29650 + os.getpid() % 300, ret), nprocs=2, join=True)
    assert ret[0] and ret[1]


def _peer_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import backpack_b200 as bp
    from backpack_b200 import sharded, synth
    from oracle import q4k_oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    ctx = bp.Q4KContext(rank)
    # name: (M, N, K, device layout, file type): Q4_K, Q5_K and the padded Q6_K single-row kernel
    cases = {"a": (1, 8192, 4096, 12, 12), "b": (8, 1024, 8192, 12, 12), "c": (3, 128, 512, 12, 12),
             "d": (1, 4096, 4096, 13, 13), "e": (5, 300, 1024, 13, 13), "f": (1, 6000, 2048, 0x10E, 14)}
    types = {n: c[4] for n, c in cases.items()}
    cases_full, cases = cases, {n: c[:3] for n, c in cases.items()}
    ok = True
    # double-buffered slots: one barrier per step, three steps so that both halves are written and the first
    # one is written again; single slots: a second barrier after the reads
    for double_buffer in (True, False):
        pg = sharded.PeerGather(ctx, world, rank, {n: (c[0], sharded.shard_rows(c[1], world)) for n, c in cases.items()},
                                double_buffer=double_buffer)
        for rep in range(3):
            xs, raws = {}, {}
            for n, (M, N, K) in cases.items():
                layout, ftype = cases_full[n][3], cases_full[n][4]
                raws[n] = synth.make_kq_weights(ftype, N, K, 5 + rep)
                xs[n] = synth.make_activations(M, K, 6 + rep)
                ns = sharded.shard_rows(N, world)
                w = ctx.upload(bp.pack_kq(layout, sharded.shard_raw(raws[n], N, K, world, rank, synth.KQ_BLOCK_BYTES[ftype]), ns, K))
                pg.matmul(n, torch.from_numpy(xs[n]).cuda(), w)
            pg.barrier()
            torch.cuda.synchronize()
            ok = ok and ctx.device_status() == 0
            for n, (M, N, K) in cases.items():
                g = pg.gathered(n)                                     # [world, M, Ns]
                y = g.permute(1, 0, 2).reshape(M, -1)[:, :N].cpu().numpy()
                want = orc.kq_matmul(types[n], xs[n], raws[n], None, N, K, threads=4)
                rel = np.linalg.norm(y - want) / np.linalg.norm(want)
                ok = ok and rel <= 1e-3 and np.abs(y - want).max() <= 2e-2 * max(1.0, float(np.abs(want).max()) / 100.0)
            if not double_buffer:
                pg.barrier()                                           # nobody overwrites slots others still read
                torch.cuda.synchronize()
        pg.close()
        dist.barrier()
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_fused_peer_gather():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_peer_worker, args=(2, 29950 + os.getpid() % 300, ret), nprocs=2, join=True)
    assert ret[0] and ret[1]


def test_peer_barrier_wait_is_bounded(ctx):
    """A flag nothing ever sets: the barrier kernel must give up after its limit, report
    BPQ4K_ERR_TIMEOUT through the device status word, and leave the context usable."""
    import ctypes as C
    import time

    import torch

    mine = torch.zeros(8, dtype=torch.int32, device="cuda")      # this GPU's flag array: slot 1 stays 0
    other = torch.zeros(8, dtype=torch.int32, device="cuda")     # stands in for the absent peer's array
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    t0 = time.time()
    ctx.peer_barrier(ptrs, rank=0, epoch=1, timeout_ms=200)
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    from backpack_b200 import q4k

    with pytest.raises(q4k.Q4KError) as e:
        ctx.device_status()
    assert e.value.status == 6
    assert ctx.device_status() == 0                                # cleared by the read
    assert int(other[0]) == 1 and int(mine[0]) == 1 and int(mine[1]) == 0
    # satisfied barrier: both slots already at the epoch
    mine[1] = 2
    ctx.peer_barrier(ptrs, rank=0, epoch=2, timeout_ms=200)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
