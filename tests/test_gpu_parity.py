"""GPU parity: the CUDA path through the C ABI against the CPU checker and the
reference-generated golden vectors.  Dequantised weights must be bit-exact;
matmul outputs must be within 1e-3 relative L2 and 2e-2 max absolute error of
the reference computation (and within the reference's own test tolerance,
atol = rtol = 2e-4, on its own fixtures)."""
import numpy as np
import pytest

from backpack_b200 import pack_q4k, q4k, synth
from conftest import GOLDEN_CASES, assert_close_ref, rel_l2
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3     # stated tolerance of the path
MAX_ABS_TOL = 2e-2

VARIANTS = [q4k.GEMV_FP32, q4k.GEMV_STREAM, q4k.GEMV_AUTO]
VARIANT_IDS = ["fp32", "stream", "auto"]


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def dev(t, a):
    return t.from_numpy(np.ascontiguousarray(a)).cuda()


def run_matmul(ctx, x, raw, bias, N, K, variant=q4k.GEMV_AUTO):
    import torch

    ctx.set_option(q4k.OPT_GEMV_VARIANT, variant)
    try:
        w = ctx.upload(pack_q4k(raw, N, K))
        y = ctx.matmul(dev(torch, x.reshape(-1, K)), w, dev(torch, bias) if bias is not None else None)
        torch.cuda.synchronize()
        return y.cpu().numpy()
    finally:
        ctx.set_option(q4k.OPT_GEMV_VARIANT, q4k.GEMV_AUTO)


def check(y, want):
    assert y.shape == want.shape
    assert np.isfinite(y).all()
    assert rel_l2(y, want) <= REL_L2_TOL
    assert float(np.abs(y - want).max()) <= MAX_ABS_TOL


# ---------------------------------------------------------------- dequant

@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_dequant_bit_exact_on_golden(ctx, golden, case):
    import torch

    M, N, K = (int(v) for v in golden[f"{case}.shape"])
    w = ctx.upload(pack_q4k(golden[f"{case}.raw"], N, K))
    out = ctx.dequant(w)
    torch.cuda.synchronize()
    assert np.array_equal(bits(out.cpu().numpy()), bits(golden[f"{case}.deq"]))


@pytest.mark.parametrize("N,K,seed", [(1, 256, 1), (3, 768, 2), (257, 1024, 3), (4096, 4096, 0)])
def test_dequant_bit_exact_on_synthetic(ctx, N, K, seed):
    import torch

    raw = synth.make_q4k_weights(N, K, seed)
    out = ctx.dequant(ctx.upload(pack_q4k(raw, N, K)))
    torch.cuda.synchronize()
    assert np.array_equal(bits(out.cpu().numpy()), bits(orc.dequant(raw, N, K)))


def test_dequant_random_bytes_every_field_value(ctx):
    """Arbitrary bytes: every scale/min/code value and many half patterns (finite ones compared)."""
    import torch

    N, K = 512, 512
    raw = np.random.default_rng(11).integers(0, 256, (N, 2 * 144), dtype=np.uint8)
    out = ctx.dequant(ctx.upload(pack_q4k(raw, N, K))).cpu().numpy()
    torch.cuda.synchronize()
    want = orc.dequant(raw, N, K)
    ok = np.isfinite(want)
    assert np.array_equal(bits(out[ok]), bits(want[ok]))
    assert np.array_equal(np.isnan(out), np.isnan(want))


def test_dequant_padded_row_stride(ctx):
    import torch

    N, K = 5, 512
    raw = synth.make_q4k_weights(N, K, 4)
    stride_words = 2 * 36 + 8
    padded = np.full((N, stride_words * 4), 0xEE, np.uint8)
    padded[:, : 2 * 144] = raw
    w = q4k.Q4KWeight(dev(torch, padded.reshape(-1)), N, K, stride_words)
    out = ctx.dequant(w).cpu().numpy()
    assert np.array_equal(bits(out), bits(orc.dequant(raw, N, K)))


# ---------------------------------------------------------------- matmul

@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_matmul_golden(ctx, golden, case, variant):
    M, N, K = (int(v) for v in golden[f"{case}.shape"])
    y = run_matmul(ctx, golden[f"{case}.x"], golden[f"{case}.raw"], golden[f"{case}.bias"], N, K, variant)
    want = golden[f"{case}.y"]
    assert rel_l2(y, want) <= REL_L2_TOL
    if case != "synthetic":
        # the reference's own bar on its fixtures; the hand-made corner blocks reach 3.6e5 in
        # magnitude (d = 65504), where only a relative bound is meaningful
        assert_close_ref(y, want, 2e-4, 2e-4)
    if case != "corner":
        check(y, want)


@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 9, 16, 17, 33])
@pytest.mark.parametrize("N,K", [(1, 256), (7, 512), (8, 256), (9, 768), (17, 1024), (130, 2048)])
def test_matmul_small_shapes(ctx, M, N, K, variant):
    raw = synth.make_q4k_weights(N, K, 100 + N)
    x = synth.make_activations(M, K, 200 + M)
    bias = (np.arange(N) * 0.01).astype(np.float32)
    y = run_matmul(ctx, x, raw, bias, N, K, variant)
    check(y, orc.matmul(x, raw, bias, N, K))


@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
@pytest.mark.parametrize("M", [1, 8])
@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 4096), (4096, 14336), (3000, 8192)])
def test_matmul_projection_shapes(ctx, M, N, K, variant):
    raw = synth.make_q4k_weights(N, K, 0)
    x = synth.make_activations(M, K, 1)
    y = run_matmul(ctx, x, raw, None, N, K, variant)
    check(y, orc.matmul(x, raw, None, N, K, threads=8))


@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
def test_matmul_y_offset_and_canaries(ctx, variant):
    """yOffset as q4k_matmul_128 uses it; nothing outside [yOffset, yOffset+M*N) may be written."""
    import torch

    N, K, M, yo = 20, 512, 1, 12
    raw = synth.make_q4k_weights(N, K, 1)
    x = synth.make_activations(M, K, 2)
    ctx.set_option(q4k.OPT_GEMV_VARIANT, variant)
    w = ctx.upload(pack_q4k(raw, N, K))
    out = torch.full((64,), -777.0, dtype=torch.float32, device="cuda")
    ctx.matmul(dev(torch, x), w, None, out=out, y_offset=yo)
    ctx.set_option(q4k.OPT_GEMV_VARIANT, q4k.GEMV_AUTO)
    got = out.cpu().numpy()
    check(got[yo:yo + N].reshape(1, N), orc.matmul(x, raw, None, N, K))
    assert (got[:yo] == -777.0).all() and (got[yo + N:] == -777.0).all()


@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
def test_matmul_extreme_activations(ctx, variant):
    """Large, tiny and mixed-magnitude activations (the split-precision path must rescale)."""
    N, K = 64, 1024
    raw = synth.make_q4k_weights(N, K, 8)
    base = synth.make_activations(4, K, 9)
    x = base.copy()
    x[0] *= 1e5
    x[1] *= 1e-6
    x[2, ::7] *= 3e4
    x[3] = 0.0
    y = run_matmul(ctx, x, raw, None, N, K, variant)
    want = orc.matmul_f64(x, raw, None, N, K)
    for m in range(4):
        scale = max(float(np.abs(want[m]).max()), 1e-30)
        assert float(np.abs(y[m] - want[m]).max()) / scale <= 2e-5 or float(np.abs(want[m]).max()) == 0.0
    assert (y[3] == 0).all()


@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
def test_matmul_linearity_full_size(ctx, variant):
    """Size-independent property at a full benchmark shape: f(a*x1 + x2) == a*f(x1) + f(x2)."""
    import torch

    N, K = 14336, 4096
    raw = synth.make_q4k_weights(N, K, 3)
    ctx.set_option(q4k.OPT_GEMV_VARIANT, variant)
    w = ctx.upload(pack_q4k(raw, N, K))
    x1 = dev(torch, synth.make_activations(1, K, 4))
    x2 = dev(torch, synth.make_activations(1, K, 5))
    y1, y2 = ctx.matmul(x1, w).double(), ctx.matmul(x2, w).double()
    y12 = ctx.matmul(0.5 * x1 + x2, w).double()
    ctx.set_option(q4k.OPT_GEMV_VARIANT, q4k.GEMV_AUTO)
    err = (y12 - (0.5 * y1 + y2)).abs().max().item()
    # three evaluations, each within a few 1e-4 of exact at |y| ~ 250: a quarter of the 2e-2 bound
    assert err <= 5e-3, err
    # and the output equals X . dequant(W)^T computed from the library's own bit-exact dequant
    deq = ctx.dequant(w).double()
    ref = x1.double() @ deq.T
    assert ((y1 - ref).abs().max().item()) <= MAX_ABS_TOL
    assert ((y1 - ref).norm() / ref.norm()).item() <= REL_L2_TOL


# ---------------------------------------------------------------- prefill (tensor-core kernel)

PREFILL_MODES = [(q4k.PREFILL_F16X3, "f16x3"), (q4k.PREFILL_F16, "f16"), (q4k.PREFILL_BF16, "bf16")]


@pytest.mark.parametrize("mode,name", PREFILL_MODES, ids=[m[1] for m in PREFILL_MODES])
@pytest.mark.parametrize("M,N,K", [(25, 130, 512), (40, 300, 1024), (64, 256, 256), (100, 130, 512), (256, 300, 1024), (300, 1024, 2048),
                                   (512, 4096, 4096), (512, 1000, 14336)])
def test_prefill_tensor_core(ctx, M, N, K, mode, name):
    """Large M goes to the tcgen05 kernel.  The three-pass half split must meet the float tolerance
    of the path; the single-pass modes round weights and activations to 16 bits and are held to the
    error that rounding implies (half: 2^-11 per operand, bfloat16: 2^-8)."""
    import torch

    raw = synth.make_q4k_weights(N, K, 60)
    x = synth.make_activations(M, K, 61)
    bias = np.linspace(-1, 1, N).astype(np.float32)
    ctx.set_option(q4k.OPT_PREFILL_MODE, mode)
    try:
        w = ctx.upload(pack_q4k(raw, N, K))
        ctx.launch_count(reset=True)
        y = ctx.matmul(dev(torch, x), w, dev(torch, bias))
        torch.cuda.synchronize()
        assert ctx.launch_count() in (2, 3)     # activation cast + tensor-core kernel (+ split-K reduction)
        assert ctx.device_status() == 0
    finally:
        ctx.set_option(q4k.OPT_PREFILL_MODE, q4k.PREFILL_F16X3)
    y = y.cpu().numpy()
    want = orc.matmul(x, raw, bias, N, K, threads=8)
    assert np.isfinite(y).all()
    if mode == q4k.PREFILL_F16X3:
        check(y, want)
    else:
        tol = 1e-3 if mode == q4k.PREFILL_F16 else 8e-3
        assert rel_l2(y, want) <= tol


@pytest.mark.parametrize("variant", [q4k.PREFILL_CTA_PAIR, q4k.PREFILL_TMEM_WEIGHTS], ids=["cta_pair", "weights_in_tmem"])
@pytest.mark.parametrize("M,N,K", [(257, 256, 256), (512, 1000, 1024), (300, 2100, 2048), (700, 777, 4096), (64, 300, 512)])
def test_prefill_variants_give_the_bits_of_the_default_kernel(ctx, variant, M, N, K):
    """BPQ4K_OPT_PREFILL_VARIANT: CTA pairs sharing tcgen05.mma.cta_group::2, and dequantised weights as a tensor-memory
    operand.  Each output element is the same sum of the same 16-bit products in the same k order, so with one K slice
    (K <= 1024 here) the outputs must equal the default kernel's bit for bit; always within the mode's tolerance of the
    checker."""
    import torch

    raw = synth.make_q4k_weights(N, K, 80)
    x = synth.make_activations(M, K, 81)
    bias = np.linspace(-2, 2, N).astype(np.float32)
    w = ctx.upload(pack_q4k(raw, N, K))
    want = orc.matmul(x, raw, bias, N, K)
    for mode, tol in ((q4k.PREFILL_F16, 1e-3), (q4k.PREFILL_BF16, 8e-3)):
        ctx.set_option(q4k.OPT_PREFILL_MODE, mode)
        try:
            ctx.set_option(q4k.OPT_PREFILL_VARIANT, q4k.PREFILL_ONE_CTA)
            y0 = ctx.matmul(dev(torch, x), w, bias=dev(torch, bias)).cpu().numpy()
            ctx.set_option(q4k.OPT_PREFILL_VARIANT, variant)
            y1 = ctx.matmul(dev(torch, x), w, bias=dev(torch, bias)).cpu().numpy()
            assert ctx.device_status() == 0
        finally:
            ctx.set_option(q4k.OPT_PREFILL_VARIANT, q4k.PREFILL_ONE_CTA)
            ctx.set_option(q4k.OPT_PREFILL_MODE, q4k.PREFILL_F16X3)
        assert rel_l2(y1, want) <= tol
        # the K slices per problem follow the tile count, which differs between the forms: compare bits where both use one slice
        if K <= 1024:
            assert np.array_equal(y0, y1)
        else:
            assert rel_l2(y1, y0) <= 1e-5


def test_prefill_threshold_option(ctx):
    """BPQ4K_OPT_PREFILL_MIN_M moves the hand-over point between the streaming and the tensor-core kernel."""
    import torch

    N, K, M = 128, 512, 64
    raw = synth.make_q4k_weights(N, K, 62)
    x = synth.make_activations(M, K, 63)
    w = ctx.upload(pack_q4k(raw, N, K))
    want = orc.matmul(x, raw, None, N, K)
    default_min_m = ctx.get_option(q4k.OPT_PREFILL_MIN_M)
    ctx.set_option(q4k.OPT_PREFILL_MIN_M, 65)
    ctx.launch_count(reset=True)
    y_stream = ctx.matmul(dev(torch, x), w).cpu().numpy()
    n_stream = ctx.launch_count(reset=True)
    ctx.set_option(q4k.OPT_PREFILL_MIN_M, 64)
    y_tc = ctx.matmul(dev(torch, x), w).cpu().numpy()
    n_tc = ctx.launch_count()
    ctx.set_option(q4k.OPT_PREFILL_MIN_M, default_min_m)
    # slabs of 8 or 16 rows (one launch each; two where the activations are quantised by a kernel of their own)
    # vs. cast + tensor-core launch (+ reduction)
    assert n_stream in (4, 8, 16) and n_tc in (2, 3)
    check(y_stream, want)
    check(y_tc, want)


@pytest.mark.parametrize("N,K", [(16, 256), (100, 1024), (4099, 4096), (1024, 14336), (777, 28672)])
def test_cluster_staging_gives_identical_bits(ctx, N, K):
    """BPQ4K_OPT_STREAM_CLUSTER: the CTAs of a cluster quantise a share of the activation row each and write it into
    every member's shared memory.  The staged bytes are the same whoever computes them, so the outputs must be
    bit-identical for cluster sizes 1, 2 and 4 (and within tolerance of the checker)."""
    import torch

    raw = synth.make_q4k_weights(N, K, 70)
    x = synth.make_activations(1, K, 71)
    w = ctx.upload(pack_q4k(raw, N, K))
    want = orc.matmul(x, raw, None, N, K)
    default = ctx.get_option(q4k.OPT_STREAM_CLUSTER)
    ys = []
    try:
        for cs in (1, 2, 4):
            ctx.set_option(q4k.OPT_STREAM_CLUSTER, cs)
            ys.append(ctx.matmul(dev(torch, x), w).cpu().numpy())
            assert ctx.device_status() == 0
    finally:
        ctx.set_option(q4k.OPT_STREAM_CLUSTER, default)
    check(ys[0], want)
    assert np.array_equal(ys[0], ys[1]) and np.array_equal(ys[0], ys[2])


def test_stream_time_stamps(ctx):
    """BPQ4K_OPT_STREAM_STAMPS (libbpq4k_stamps.so: the product library with the streaming kernel compiled again with
    the stamps): thread 0 of every CTA of a single-row launch leaves six ordered time stamps and its SM id; the result
    equals the product library's bit for bit; the product library refuses the option."""
    import torch

    import backpack_b200 as bp

    N, K = 4096, 4096
    raw = synth.make_q4k_weights(N, K, 90)
    x = synth.make_activations(1, K, 91)
    y0 = ctx.matmul(dev(torch, x), ctx.upload(pack_q4k(raw, N, K))).cpu().numpy()
    with pytest.raises(q4k.Q4KError):
        ctx.set_option(q4k.OPT_STREAM_STAMPS, 4)
    sctx = bp.Q4KContext(0, stamps=True)
    try:
        w = sctx.upload(pack_q4k(raw, N, K))
        with pytest.raises(q4k.Q4KError):
            sctx.stream_stamps(4)                       # not switched on yet
        sctx.set_option(q4k.OPT_STREAM_STAMPS, 4)
        y1 = sctx.matmul(dev(torch, x), w).cpu().numpy()
        ts, n = sctx.stream_stamps(4)
        sctx.set_option(q4k.OPT_STREAM_STAMPS, 0)
    finally:
        sctx.close()
    assert n == 1 and np.array_equal(y0, y1)
    grid = int(ts[0, 0, 7] >> np.uint64(32))
    assert 1 <= grid <= 160
    t = ts[0, :grid, :6].astype(np.int64)
    assert (t > 0).all() and (np.diff(t, axis=1) >= 0).all()
    assert (t[:, 5] - t[:, 0]).max() < 1_000_000       # a launch of 9 MB ends within a millisecond
    assert not ts[1:].any()


# ---------------------------------------------------------------- MoE indirect form

@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
def test_moe_indirect(ctx, variant):
    import torch

    E, N, K, T, topk = 16, 96, 512, 4, 3
    raw = synth.make_q4k_weights(E * N, K, 21)
    x = synth.make_activations(T, K, 22)
    ids = synth.make_moe_routing(T, E, topk, 23)                  # [T, topk]
    offsets = (ids.reshape(-1) * N).astype(np.int32)               # slot s = (token, k)
    x_rows = np.repeat(np.arange(T), topk).astype(np.int32)
    ctx.set_option(q4k.OPT_GEMV_VARIANT, variant)
    w = ctx.upload(pack_q4k(raw, E * N, K))
    y = ctx.matmul_moe(dev(torch, x), w, N, dev(torch, offsets), dev(torch, x_rows))
    # per-slot activations (the "down" direction): row s of X belongs to slot s
    xs = synth.make_activations(T * topk, K, 24)
    y2 = ctx.matmul_moe(dev(torch, xs), w, N, dev(torch, offsets))
    ctx.set_option(q4k.OPT_GEMV_VARIANT, q4k.GEMV_AUTO)
    want = orc.matmul_moe(x[x_rows], raw, None, N, K, offsets.astype(np.uint32))
    check(y.cpu().numpy(), want.reshape(T * topk, N))
    want2 = orc.matmul_moe(xs, raw, None, N, K, offsets.astype(np.uint32))
    check(y2.cpu().numpy(), want2.reshape(T * topk, N))


@pytest.mark.parametrize("E,N,K,slots", [(32, 16, 256, 700),      # one tile per expert, many slots: one grid row per slot
                                         (5, 40, 768, 9),         # ragged last tile of every slot
                                         (3, 16, 256, 1), (7, 48, 512, 2),
                                         (16, 768, 2048, 64),     # the gate/up shape of benchmark configuration 3
                                         (16, 2048, 768, 64),     # its down shape
                                         (4, 4096, 1024, 5), (9, 272, 4096, 37), (64, 32, 512, 300),
                                         (16, 768, 2048, 256),    # more slots than SMs: served as one unit list
                                         (8, 512, 256, 200)])
def test_moe_unit_list_shapes(ctx, E, N, K, slots):
    """Slots are served as one list of (slot, tile) units when each CTA's share spans few slots, else as one grid row
    per slot: both against the per-slot oracle, with repeated experts and a shuffled activation-row map."""
    import torch

    rng = np.random.default_rng(E * 1000 + slots)
    raw = synth.make_q4k_weights(E * N, K, 31)
    w = ctx.upload(pack_q4k(raw, E * N, K))
    ids = rng.integers(0, E, slots)
    offsets = (ids * N).astype(np.int32)
    n_x = max(1, slots // 3)
    x = synth.make_activations(n_x, K, 32)
    x_rows = rng.integers(0, n_x, slots).astype(np.int32)
    y = ctx.matmul_moe(dev(torch, x), w, N, dev(torch, offsets), dev(torch, x_rows)).cpu().numpy()
    sample = np.arange(slots) if slots <= 64 else rng.choice(slots, 64, replace=False)
    want = orc.matmul_moe(x[x_rows[sample]], raw, None, N, K, offsets[sample].astype(np.uint32)).reshape(len(sample), N)
    check(y[sample], want)
    assert ctx.device_status() == 0
    # the other form of the launch walks the same tiles with the same arithmetic: identical bits
    ctx.set_option(q4k.OPT_STREAM_NO_UNIT_LIST, 1)
    try:
        y_rows = ctx.matmul_moe(dev(torch, x), w, N, dev(torch, offsets), dev(torch, x_rows)).cpu().numpy()
    finally:
        ctx.set_option(q4k.OPT_STREAM_NO_UNIT_LIST, 0)
    assert np.array_equal(y.view(np.uint32), y_rows.view(np.uint32))


# ---------------------------------------------------------------- host entry point

def test_matmul_host_buffers(ctx):
    N, K, M = 300, 1024, 2
    raw = synth.make_q4k_weights(N, K, 31)
    x = synth.make_activations(M, K, 32)
    w = ctx.upload(pack_q4k(raw, N, K))
    y = np.zeros((M, N), np.float32)
    ctx.matmul_host(x, w, y)
    check(y, orc.matmul(x, raw, None, N, K))
    # a second, larger call re-sizes the staging buffers
    M2 = 700
    x2 = synth.make_activations(M2, K, 33)
    y2 = np.zeros((M2, N), np.float32)
    ctx.matmul_host(x2, w, y2)
    check(y2, orc.matmul(x2, raw, None, N, K, threads=8))


def test_matmul_host_batch(ctx):
    """A dispatch list of independent matmuls on host buffers, one call."""
    shapes = [(1, 300, 1024), (2, 64, 512), (1, 1024, 4096), (0, 8, 256)]
    items, wants = [], []
    for i, (M, N, K) in enumerate(shapes):
        raw = synth.make_q4k_weights(N, K, 40 + i)
        x = synth.make_activations(M, K, 50 + i)
        y = np.full((M, N), np.nan, np.float32)
        items.append((x, ctx.upload(pack_q4k(raw, N, K)), y, None))
        wants.append(orc.matmul(x, raw, None, N, K))
    batch = ctx.make_host_batch(items)
    for _ in range(2):          # the second call reuses the staging buffers
        ctx.matmul_host_batch(batch)
        for (x, w, y, b), want in zip(items, wants):
            if want.size:
                check(y, want)


def test_matmul_host_batch_pinned_buffers_replay(ctx):
    """Pinned host buffers: inputs move with one kernel, the streaming kernel stores its outputs straight into
    the host buffers, the tensor-core item's output is staged and scattered; from the third call on the same
    dispatch list is replayed from a CUDA graph.  New input values in the same buffers give new results; a
    different list falls back to recording again."""
    import torch

    shapes = [(1, 300, 1024), (1, 1024, 4096), (3, 64, 512), (1, 2000, 2048), (40, 130, 512)]
    items, raws = [], []
    for i, (M, N, K) in enumerate(shapes):
        raw = synth.make_q4k_weights(N, K, 140 + i)
        x = torch.zeros((M, K), dtype=torch.float32).pin_memory()
        y = torch.full((M, N), float("nan"), dtype=torch.float32).pin_memory()
        items.append((x.numpy(), ctx.upload(pack_q4k(raw, N, K)), y.numpy(), None))
        raws.append((raw, x, y))
    batch = ctx.make_host_batch(items)
    for rep in range(5):
        for i, (M, N, K) in enumerate(shapes):
            items[i][0][...] = synth.make_activations(M, K, 150 + 10 * rep + i)
            items[i][2][...] = np.nan
        ctx.launch_count(reset=True)
        ctx.matmul_host_batch(batch)
        # gather, four streaming matmuls, the 40-row item (cast + tensor-core kernel, + reduction), scatter of that
        # item's output -- also when replayed
        assert ctx.launch_count() in (1 + 4 + 2 + 1, 1 + 4 + 3 + 1)
        for (xh, w, yh, _), (raw, _, _), (M, N, K) in zip(items, raws, shapes):
            check(yh, orc.matmul(xh, raw, None, N, K))
    # another list (the first two items only) after the graph exists
    batch2 = ctx.make_host_batch(items[:2])
    for rep in range(3):
        for i in range(2):
            items[i][0][...] = synth.make_activations(shapes[i][0], shapes[i][2], 300 + rep + i)
        ctx.matmul_host_batch(batch2)
        for (xh, w, yh, _), (raw, _, _), (M, N, K) in zip(items[:2], raws[:2], shapes[:2]):
            check(yh, orc.matmul(xh, raw, None, N, K))
    assert ctx.device_status() == 0


def test_host_batch_replay_graph_is_rerecorded_after_a_buffer_grows():
    """The replay graph of a dispatch list holds the addresses of the handle's staging and scratch buffers.  A larger
    call through another entry point makes those buffers grow; the list must then be recorded again (never replayed
    against the outgrown blocks), and results stay right throughout."""
    import torch

    import backpack_b200 as bp

    c = bp.Q4KContext(0)
    try:
        shapes = [(1, 300, 1024), (4, 64, 8192), (1, 1024, 4096)]
        items, raws = [], []
        for i, (M, N, K) in enumerate(shapes):
            raw = synth.make_q4k_weights(N, K, 240 + i)
            x = torch.from_numpy(synth.make_activations(M, K, 250 + i)).pin_memory()
            y = torch.full((M, N), float("nan"), dtype=torch.float32).pin_memory()
            items.append((x.numpy(), c.upload(pack_q4k(raw, N, K)), y.numpy(), None))
            raws.append((raw, x, y))
        batch = c.make_host_batch(items)

        def run_and_check():
            for it in items:
                it[2][...] = np.nan
            c.matmul_host_batch(batch)
            for (xh, w, yh, _), (raw, _, _), (M, N, K) in zip(items, raws, shapes):
                check(yh, orc.matmul(xh, raw, None, N, K))

        for _ in range(3):
            run_and_check()
        assert c.get_option(q4k.OPT_BATCH_RECORDS) == 1
        # a call whose activations (32 MB) and outputs outgrow the staging buffers
        N2, K2, M2 = 64, 4096, 2048
        raw2 = synth.make_q4k_weights(N2, K2, 260)
        x2 = synth.make_activations(M2, K2, 261)
        y2 = np.zeros((M2, N2), np.float32)
        c.matmul_host(x2, c.upload(pack_q4k(raw2, N2, K2)), y2)
        check(y2, orc.matmul(x2, raw2, None, N2, K2, threads=8))
        for _ in range(3):
            run_and_check()
        assert c.get_option(q4k.OPT_BATCH_RECORDS) == 2
        assert c.device_status() == 0
    finally:
        c.close()


def test_four_rows_of_long_k_quantise_once_and_copy_in(ctx):
    """2..4 rows with 32K or more staged values: one quantising launch, then the matmul copies the digits in."""
    import torch

    N, K, M = 1000, 8192, 4
    raw = synth.make_q4k_weights(N, K, 270)
    x = synth.make_activations(M, K, 271)
    w = ctx.upload(pack_q4k(raw, N, K))
    ctx.launch_count(reset=True)
    y = ctx.matmul(dev(torch, x), w).cpu().numpy()
    assert ctx.launch_count() == 2
    check(y, orc.matmul(x, raw, None, N, K, threads=4))


# ---------------------------------------------------------------- error behaviour

def test_errors_are_statuses_not_faults(ctx):
    import torch

    N, K = 8, 512
    w = ctx.upload(pack_q4k(synth.make_q4k_weights(N, K, 1), N, K))
    x = torch.zeros(1, K, device="cuda")
    with pytest.raises(q4k.Q4KError) as e:     # K not a multiple of 256
        ctx.matmul(torch.zeros(1, 300, device="cuda"), q4k.Q4KWeight(w.buf, N, 300, 72))
    assert e.value.status == 2 and "256" in str(e.value)
    with pytest.raises(q4k.Q4KError) as e:     # stride shorter than a row
        ctx.matmul(x, q4k.Q4KWeight(w.buf, N, K, 36))
    assert e.value.status == 1
    with pytest.raises(q4k.Q4KError) as e:     # stride not a multiple of 16 bytes
        ctx.matmul(x, q4k.Q4KWeight(w.buf, N, K, 73))
    assert e.value.status == 3
    with pytest.raises(q4k.Q4KError) as e:     # misaligned activations
        ctx.matmul(torch.zeros(K + 1, device="cuda")[1:].reshape(1, K), w)
    assert e.value.status == 3
    with pytest.raises(q4k.Q4KError) as e:     # misaligned weights
        ctx.matmul(x, q4k.Q4KWeight(torch.zeros(w.buf.numel() + 4, dtype=torch.uint8, device="cuda")[4:], N, K, 72))
    assert e.value.status == 3
    with pytest.raises(q4k.Q4KError):
        ctx.set_option(q4k.OPT_GEMV_VARIANT, 17)
    # empty problems are no-ops
    assert ctx.matmul(torch.zeros(0, K, device="cuda"), w).shape == (0, N)
    # the context is still healthy
    y = ctx.matmul(x, w)
    torch.cuda.synchronize()
    assert (y == 0).all()


def test_launch_counter_counts_kernels(ctx):
    import torch

    N, K = 64, 512
    w = ctx.upload(pack_q4k(synth.make_q4k_weights(N, K, 1), N, K))
    ctx.launch_count(reset=True)
    ctx.matmul(torch.zeros(1, K, device="cuda"), w)
    ctx.dequant(w)
    assert ctx.launch_count() >= 2


# ---------------------------------------------------------------- benchmark configurations 3 and 4

def test_moe_config3_shapes(ctx):
    """128 experts, hidden 2048, expert FFN 768, 8 rows x 8 routed experts: gate/up share the row's
    activations, down takes one activation row per (row, expert) pair."""
    import torch

    E, H, F, T, topk = 128, 2048, 768, 8, 8
    ids = synth.make_moe_routing(T, E, topk, 5).reshape(-1)
    x_rows = np.repeat(np.arange(T), topk).astype(np.int32)
    # gate / up direction: [E*F, H]
    raw_gate = synth.make_q4k_weights(E * F, H, 70)
    wg = ctx.upload(pack_q4k(raw_gate, E * F, H))
    x = synth.make_activations(T, H, 71)
    off_g = (ids * F).astype(np.int32)
    y = ctx.matmul_moe(dev(torch, x), wg, F, dev(torch, off_g), dev(torch, x_rows)).cpu().numpy()
    want = orc.matmul_moe(x[x_rows], raw_gate, None, F, H, off_g.astype(np.uint32)).reshape(T * topk, F)
    check(y, want)
    # down direction: [E*H, F], K = 768 (three super-blocks per row)
    raw_down = synth.make_q4k_weights(E * H, F, 72)
    wd = ctx.upload(pack_q4k(raw_down, E * H, F))
    xs = synth.make_activations(T * topk, F, 73)
    off_d = (ids * H).astype(np.int32)
    y = ctx.matmul_moe(dev(torch, xs), wd, H, dev(torch, off_d)).cpu().numpy()
    want = orc.matmul_moe(xs, raw_down, None, H, F, off_d.astype(np.uint32)).reshape(T * topk, H)
    check(y, want)


@pytest.mark.parametrize("M", [1, 8])
@pytest.mark.parametrize("N,K", [(8192, 8192), (1024, 8192), (3584, 8192), (1024, 28672)])
def test_llama70b_shard_shapes(ctx, M, N, K):
    """Config 4 shapes as one rank of an 8-way row split sees them (28672/8 = 3584 rows of gate/up,
    8192/8 = 1024 rows of down with K = 28672), plus the unsplit q/k."""
    raw = synth.make_q4k_weights(N, K, 80)
    x = synth.make_activations(M, K, 81)
    y = run_matmul(ctx, x, raw, None, N, K)
    check(y, orc.matmul(x, raw, None, N, K, threads=8))


@pytest.mark.parametrize("M", [2, 3, 4, 5, 7, 8])
@pytest.mark.parametrize("N,K", [(600, 14336), (300, 28672), (1000, 8192), (33, 14336), (2500, 8192)])
def test_several_rows_with_long_k_walk_k_in_phases(ctx, M, N, K):
    """Rows whose digits do not fit in shared memory together: the kernel copies them in K range by K
    range (tile counts that are odd, below a group, and spread unevenly over the warps of a CTA)."""
    raw = synth.make_q4k_weights(N, K, 90 + M)
    x = synth.make_activations(M, K, 91)
    bias = np.linspace(-3, 3, N).astype(np.float32)
    y = run_matmul(ctx, x, raw, bias, N, K)
    check(y, orc.matmul(x, raw, bias, N, K, threads=8))
    assert ctx.device_status() == 0
