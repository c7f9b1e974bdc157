"""Out-of-bounds discipline of the kernels, in the way the reference's kernel tests probe it (tiny exhaustive shapes:
N in {1, 7, 8, 9}, 1..3 super-blocks per row, M in {1, 5, 9}; runtime/tests/kernel_test.cpp:1678-1748) plus a few large
ones: every device buffer of a call sits between guard zones that are checked after the call -- outputs and scratch may
not be written outside their extent, and inputs are surrounded by NaNs, so a read outside them poisons the result.  The
same calls then run on the debug build of the library, whose kernels carry index checks that report through the device
status word instead of trapping."""
import numpy as np
import pytest

from backpack_b200 import pack_kq, q4k, synth
from conftest import rel_l2
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu

GUARD = 256          # floats (or bytes for weights) on each side
CANARY = -7777.0


def guarded(torch, host: np.ndarray, fill):
    """A device copy of `host` with GUARD elements of `fill` on both sides; returns (whole buffer, view of the middle)."""
    n = host.size
    buf = torch.full((n + 2 * GUARD,), fill, dtype=torch.from_numpy(host.reshape(-1)[:1].copy()).dtype, device="cuda")
    buf[GUARD:GUARD + n] = torch.from_numpy(np.ascontiguousarray(host).reshape(-1)).cuda()
    return buf, buf[GUARD:GUARD + n].view(*host.shape)


def guards_intact(buf, fill):
    a, b = buf[:GUARD], buf[-GUARD:]
    return bool((a == fill).all()) and bool((b == fill).all())


def run_guarded_matmul(ctx, qtype, layout, M, N, K, seed, with_bias=True):
    import torch

    raw = synth.make_kq_weights(qtype, N, K, seed)
    packed = pack_kq(layout, raw, N, K)
    wbytes = packed.data.view(np.uint8)
    # weights between two zones of 0xFF bytes (as weights those decode to NaN/inf scales); 16-byte aligned middle
    wbuf = torch.full((wbytes.size + 2 * GUARD,), 0xFF, dtype=torch.uint8, device="cuda")
    wbuf[GUARD:GUARD + wbytes.size] = torch.from_numpy(wbytes).cuda()
    w = q4k.Q4KWeight(wbuf[GUARD:GUARD + wbytes.size], N, K, packed.rowStrideWords, layout)
    x = synth.make_activations(M, K, seed + 1)
    xbuf, xd = guarded(torch, x, float("nan"))
    bias = np.linspace(-2, 2, N).astype(np.float32) if with_bias else None
    bbuf, bd = guarded(torch, bias, float("nan")) if with_bias else (None, None)
    ybuf, yd = guarded(torch, np.zeros((M, N), np.float32), CANARY)
    ctx.matmul(xd, w, bias=bd, out=yd)
    torch.cuda.synchronize()
    assert guards_intact(ybuf, CANARY), "the kernel wrote outside Y"
    y = yd.cpu().numpy()
    assert np.isfinite(y).all(), "a read outside X, W or bias reached the result"
    want = orc.kq_matmul(qtype, x, raw, bias, N, K)
    assert rel_l2(y, want) <= 1e-3 and float(np.abs(y - want).max()) <= 2e-2 * max(1.0, float(np.abs(want).max()) / 100.0)
    assert ctx.device_status() == 0


SMALL = [(M, N, nb * 256) for M in (1, 5, 9) for N in (1, 7, 8, 9) for nb in (1, 2, 3)]
# (the last three: cluster-shared staging of a long row; uneven tile counts per CTA on a 148-SM device, ragged and whole)
LARGE = [(1, 4096, 4096), (8, 1000, 8192), (3, 130, 14336), (16, 257, 2048), (40, 300, 1024),
         (1, 1030, 14336), (1, 16 * 148 * 4 + 9, 4096), (1, 28672, 4096)]


@pytest.mark.parametrize("M,N,K", SMALL + LARGE)
def test_q4k_matmul_stays_inside_its_buffers(ctx, M, N, K):
    run_guarded_matmul(ctx, orc.Q4_K, q4k.Q4_K, M, N, K, 500 + N)


@pytest.mark.parametrize("qtype,layout", [(orc.Q5_K, q4k.Q5_K), (orc.Q6_K, q4k.Q6_K), (orc.Q6_K, q4k.Q6_K_PADDED)])
@pytest.mark.parametrize("M,N,K", [(1, 7, 256), (5, 9, 512), (9, 8, 768), (1, 1000, 4096), (4, 300, 2048)])
def test_sibling_types_stay_inside_their_buffers(ctx, qtype, layout, M, N, K):
    run_guarded_matmul(ctx, qtype, layout, M, N, K, 600 + N)


def test_expert_indexed_form_stays_inside_its_buffers(ctx):
    import torch

    E, N, K, slots = 5, 40, 768, 9
    raw = synth.make_q4k_weights(E * N, K, 31)
    packed = pack_kq(q4k.Q4_K, raw, E * N, K)
    wbytes = packed.data.view(np.uint8)
    wbuf = torch.full((wbytes.size + 2 * GUARD,), 0xFF, dtype=torch.uint8, device="cuda")
    wbuf[GUARD:GUARD + wbytes.size] = torch.from_numpy(wbytes).cuda()
    w = q4k.Q4KWeight(wbuf[GUARD:GUARD + wbytes.size], E * N, K, packed.rowStrideWords, q4k.Q4_K)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, E, slots)
    offsets = (ids * N).astype(np.int32)
    x = synth.make_activations(slots, K, 32)
    xbuf, xd = guarded(torch, x, float("nan"))
    obuf, od = guarded(torch, offsets, 2 ** 30)               # a huge row offset on both sides of the table
    ybuf, yd = guarded(torch, np.zeros((slots, N), np.float32), CANARY)
    ctx.matmul_moe(xd, w, N, od, out=yd)
    torch.cuda.synchronize()
    assert guards_intact(ybuf, CANARY)
    y = yd.cpu().numpy()
    want = orc.matmul_moe(x, raw, None, N, K, offsets.astype(np.uint32)).reshape(slots, N)
    assert np.isfinite(y).all() and rel_l2(y, want) <= 1e-3
    assert ctx.device_status() == 0


@pytest.fixture(scope="module")
def debug_ctx():
    import backpack_b200 as bp

    c = bp.Q4KContext(0, debug=True)
    yield c
    c.close()


@pytest.mark.parametrize("M,N,K", SMALL[::3] + LARGE)
def test_debug_build_reports_no_failed_index_check(debug_ctx, M, N, K):
    """The debug build's kernels check the coordinates of every weight copy, the indices of every digit they stage and
    every output index; a failed check would surface as status 9 here."""
    run_guarded_matmul(debug_ctx, orc.Q4_K, q4k.Q4_K, M, N, K, 700 + N)
    assert debug_ctx.device_status() == 0


def test_debug_build_fused_and_experts(debug_ctx):
    import torch

    N, K = 333, 1024
    raw = synth.make_q4k_weights(N, K, 9)
    w = debug_ctx.upload(pack_kq(q4k.Q4_K, raw, N, K))
    x = synth.make_activations(1, K, 10)[0]
    aux = (synth.make_activations(1, K, 11)[0] * 0.5 + 1.0).astype(np.float32)
    y = debug_ctx.matmul_fused(torch.from_numpy(x).cuda(), w, q4k.PROLOGUE_SILU_MUL, aux=torch.from_numpy(aux).cuda()).cpu().numpy()[0]
    want = orc.kq_matmul(orc.Q4_K, orc.prologue(3, x, aux), raw, None, N, K)[0]
    assert rel_l2(y, want) <= 1e-3
    E, Ne, slots = 16, 96, 300                                    # more slots than SMs: the unit-list form
    rawe = synth.make_q4k_weights(E * Ne, 512, 12)
    we = debug_ctx.upload(pack_kq(q4k.Q4_K, rawe, E * Ne, 512))
    ids = np.random.default_rng(4).integers(0, E, slots)
    xs = synth.make_activations(slots, 512, 13)
    ye = debug_ctx.matmul_moe(torch.from_numpy(xs).cuda(), we, Ne, torch.from_numpy((ids * Ne).astype(np.int32)).cuda()).cpu().numpy()
    wante = orc.matmul_moe(xs[:32], rawe, None, Ne, 512, (ids[:32] * Ne).astype(np.uint32)).reshape(32, Ne)
    assert rel_l2(ye[:32], wante) <= 1e-3
    assert debug_ctx.device_status() == 0
