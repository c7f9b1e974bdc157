"""The N-sharded multi-GPU path, host-side logic on CPU: two gloo ranks, each owning half the
rows; the local product is stood in for by the CPU checker (this file tests partitioning,
padding and the gather/transposition, not kernels)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, cases, ret):
    sys.path.insert(0, ROOT)
    from backpack_b200 import sharded, synth
    from oracle import q4k_oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = True
    for (M, N, K) in cases:
        raw = synth.make_q4k_weights(N, K, 3)
        x = synth.make_activations(M, K, 4)
        ns = sharded.shard_rows(N, world)
        shard = sharded.shard_raw(raw, N, K, world, rank)

        def fn(xt, sh, out=None):
            y = torch.from_numpy(orc.matmul(xt.numpy(), sh, None, ns, K))
            if out is not None:
                out.copy_(y)
                return out
            return y

        lin = sharded.ShardedQ4KLinear(N, K, world, rank, shard, fn)
        y = lin.forward(torch.from_numpy(x)).numpy()
        want = orc.matmul(x, raw, None, N, K)
        ok = ok and y.shape == (M, N) and np.array_equal(y, want)
    ret[rank] = ok
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_forward_matches_unsharded(world):
    cases = [(1, 64, 512), (1, 70, 256), (4, 64, 512), (3, 37, 256)]   # divisible and ragged N, M = 1 and M > 1
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 500) + world
    mp.spawn(_worker, args=(world, port, cases, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)) and len(ret) == world


def test_shard_ranges_cover_rows_once():
    sys.path.insert(0, ROOT)
    from backpack_b200 import sharded

    for N in (1, 7, 64, 128256, 1024):
        for world in (1, 2, 3, 4, 8):
            spans = [sharded.shard_range(N, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == N
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(b - a <= sharded.shard_rows(N, world) for a, b in spans)
