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
