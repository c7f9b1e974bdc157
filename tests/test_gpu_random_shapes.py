"""Seeded random shapes through every kernel-selection branch: row counts on both sides of the slab and
tensor-core hand-overs, row-tile remainders, K from one block to lengths that change the staging plan,
all three weight types (and the padded Q6_K layout), with and without bias."""
import numpy as np
import pytest

from backpack_b200 import pack_kq, synth
from conftest import rel_l2
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu

Q6_K_PADDED = 0x10E
LAYOUTS = [(orc.Q4_K, orc.Q4_K), (orc.Q5_K, orc.Q5_K), (orc.Q6_K, orc.Q6_K), (Q6_K_PADDED, orc.Q6_K)]
IDS = ["q4k", "q5k", "q6k", "q6k_padded"]


def cases(seed, n):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        M = int(rng.choice([1, 1, 1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 16, 23, 24, 25, 26, 31, 40, 64, 70]))
        nb = int(rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 12, 16, 17, 24, 32, 33, 40, 56, 64]))
        N = int(rng.choice([1, 5, 15, 16, 17, 31, 100, 129, 250, 500, 1000, 1500, 2049]))
        if M * N * nb > 3_000_000:        # keep the CPU oracle quick
            N = max(1, 3_000_000 // (M * nb))
        out.append((M, N, nb * 256, bool(rng.integers(0, 2))))
    return out


@pytest.mark.parametrize("layout,ftype", LAYOUTS, ids=IDS)
@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_shapes(ctx, layout, ftype, seed):
    import torch

    for i, (M, N, K, with_bias) in enumerate(cases(100 * seed + ftype, 14)):
        raw = synth.make_kq_weights(ftype, N, K, 1000 * seed + i)
        x = synth.make_activations(M, K, 2000 * seed + i)
        bias = np.linspace(-1, 1, N).astype(np.float32) if with_bias else None
        w = ctx.upload(pack_kq(layout, raw, N, K))
        y = ctx.matmul(torch.from_numpy(x).cuda(), w, bias=torch.from_numpy(bias).cuda() if with_bias else None).cpu().numpy()
        want = orc.kq_matmul(ftype, x, raw, bias, N, K, threads=8)
        tag = f"M={M} N={N} K={K} bias={with_bias}"
        assert rel_l2(y, want) <= 1e-3, tag
        assert float(np.abs(y - want).max()) <= 2e-2 * max(1.0, float(np.abs(want).max()) / 100.0), tag
    assert ctx.device_status() == 0
