"""GPU parity of the Q5_K / Q6_K siblings through the C ABI: bit-exact dequantisation and gather,
matmul against the oracle on the reference's fixtures, on corner blocks and on seeded shapes."""
import numpy as np
import pytest

from backpack_b200 import pack_kq, synth
from conftest import KQ_GOLDEN_GATHER, KQ_GOLDEN_MATMUL, assert_close_ref, rel_l2
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu

Q6_K_PADDED = 0x10E     # device layout of the fast single-row Q6_K kernel; same weights as Q6_K
TYPES = [orc.Q5_K, orc.Q6_K, Q6_K_PADDED]


def file_type(qtype):
    """The file format (what the oracle decodes) behind a device layout."""
    return orc.Q6_K if qtype == Q6_K_PADDED else qtype


def layouts(qtype):
    return [orc.Q6_K, Q6_K_PADDED] if qtype == orc.Q6_K else [qtype]


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check(y, want):
    """The float tolerance of the path: rel-L2 <= 1e-3 and max-abs <= 2e-2 (scaled to the output's size)."""
    assert rel_l2(y, want) <= 1e-3
    scale = max(1.0, float(np.abs(want).max()) / 100.0)
    assert float(np.abs(y - want).max()) <= 2e-2 * scale


@pytest.mark.parametrize("case", KQ_GOLDEN_MATMUL + KQ_GOLDEN_GATHER)
def test_dequant_bit_exact_on_golden(ctx, kq_golden, case):
    qtype = int(kq_golden[f"{case}.type"][0])
    _, N, K = (int(v) for v in kq_golden[f"{case}.shape"])
    for lay in layouts(qtype):
        w = ctx.upload(pack_kq(lay, kq_golden[f"{case}.raw"], N, K))
        got = ctx.dequant(w).cpu().numpy()
        assert np.array_equal(bits(got), bits(kq_golden[f"{case}.deq"]))


@pytest.mark.parametrize("case", KQ_GOLDEN_GATHER)
def test_gather_matches_reference_fixture(ctx, kq_golden, case):
    """q6k_gather_reference / q6k_gather_batched_reference: rows of the dequantised table, bit-exact."""
    import torch

    qtype = int(kq_golden[f"{case}.type"][0])
    _, N, K = (int(v) for v in kq_golden[f"{case}.shape"])
    tokens = kq_golden[f"{case}.tokens"].astype(np.int32)
    for lay in layouts(qtype):
        w = ctx.upload(pack_kq(lay, kq_golden[f"{case}.raw"], N, K))
        got = ctx.gather(w, dev(torch, tokens)).cpu().numpy()
        assert np.array_equal(bits(got), bits(kq_golden[f"{case}.deq"][tokens]))


@pytest.mark.parametrize("qtype", TYPES)
def test_gather_out_of_range_token_gives_zeros(ctx, qtype):
    import torch

    N, K = 6, 512
    raw = synth.make_kq_weights(file_type(qtype), N, K, 31)
    w = ctx.upload(pack_kq(qtype, raw, N, K))
    tokens = np.array([5, 6, 0, 4000000000 & 0x7FFFFFFF], np.int32)
    got = ctx.gather(w, dev(torch, tokens)).cpu().numpy()
    deq = orc.kq_dequant(file_type(qtype), raw, N, K)
    assert np.array_equal(bits(got[0]), bits(deq[5])) and np.array_equal(bits(got[2]), bits(deq[0]))
    assert not got[1].any() and not got[3].any()


@pytest.mark.parametrize("case", KQ_GOLDEN_MATMUL)
def test_matmul_on_golden(ctx, kq_golden, case):
    import torch

    qtype = int(kq_golden[f"{case}.type"][0])
    M, N, K = (int(v) for v in kq_golden[f"{case}.shape"])
    want = kq_golden[f"{case}.y"]
    for lay in layouts(qtype):
        w = ctx.upload(pack_kq(lay, kq_golden[f"{case}.raw"], N, K))
        y = ctx.matmul(dev(torch, kq_golden[f"{case}.x"]), w, bias=dev(torch, kq_golden[f"{case}.bias"])).cpu().numpy()
        if case.startswith("synthetic"):
            check(y, want)
        else:  # the reference's own assertClose(atol = rtol = 2e-4) on its fixtures and on the corner blocks
            assert_close_ref(y, want)


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 256), (1, 333, 1024), (1, 2048, 4096), (2, 100, 768), (3, 17, 512),
                                   (4, 256, 2048), (5, 9, 768), (8, 512, 4096), (13, 40, 1280), (40, 64, 512),
                                   (1, 4096, 14336), (1, 9000, 2048), (1, 1030, 28672), (3, 700, 8192)])
def test_matmul_seeded_shapes(ctx, qtype, M, N, K):
    import torch

    raw = synth.make_kq_weights(file_type(qtype), N, K, 100 + N)
    x = synth.make_activations(M, K, 200 + M)
    bias = np.linspace(-2, 2, N).astype(np.float32)
    w = ctx.upload(pack_kq(qtype, raw, N, K))
    y = ctx.matmul(dev(torch, x), w, bias=dev(torch, bias)).cpu().numpy()
    check(y, orc.kq_matmul(file_type(qtype), x, raw, bias, N, K, threads=4))


def test_q6k_streaming_kernel_is_the_one_that_runs(ctx):
    """Padded Q6_K with one activation row takes the tensor-core streaming kernel (one launch), the
    file-format layout the plain kernel; both agree with the oracle; extreme activations keep their
    precision because every 16-value group has its own scale."""
    import torch

    N, K = 1000, 4096
    raw = synth.make_kq_weights(orc.Q6_K, N, K, 17)
    x = synth.make_activations(1, K, 18)
    x[0, 5] = 3.0e4
    x[0, 1000:1016] = 1.0e-6
    x[0, 2048:2064] = 0.0
    want = orc.kq_matmul(orc.Q6_K, x, raw, None, N, K, threads=4)
    ys = []
    for lay in (Q6_K_PADDED, orc.Q6_K):
        w = ctx.upload(pack_kq(lay, raw, N, K))
        ctx.launch_count(reset=True)
        ys.append(ctx.matmul(dev(torch, x), w).cpu().numpy())
        assert ctx.launch_count() == 1
        check(ys[-1], want)
    assert ctx.device_status() == 0
    assert rel_l2(ys[0], ys[1]) < 1e-5


@pytest.mark.parametrize("qtype", TYPES)
def test_y_offset_and_no_bias(ctx, qtype):
    import torch

    N, K = 48, 512
    raw = synth.make_kq_weights(file_type(qtype), N, K, 7)
    x = synth.make_activations(1, K, 8)
    w = ctx.upload(pack_kq(qtype, raw, N, K))
    out = torch.full((3 * N,), -7.0, device="cuda")
    ctx.matmul(dev(torch, x), w, out=out, y_offset=N)
    got = out.cpu().numpy()
    check(got[N:2 * N], orc.kq_matmul(file_type(qtype), x, raw, None, N, K)[0])
    assert (got[:N] == -7.0).all() and (got[2 * N:] == -7.0).all()


def test_kq_errors_are_statuses(ctx):
    import torch

    from backpack_b200 import Q4KError

    lib = ctx.lib
    x = torch.zeros(256, device="cuda")
    wbuf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    y = torch.zeros(8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert lib.bpq4k_kq_matmul_f32(ctx.h, 7, x.data_ptr(), wbuf.data_ptr(), None, y.data_ptr(), 1, 8, 256, 53, 0, s) == 2
    assert lib.bpq4k_kq_matmul_f32(ctx.h, 14, x.data_ptr(), wbuf.data_ptr(), None, y.data_ptr(), 1, 8, 300, 53, 0, s) == 2
    assert lib.bpq4k_kq_matmul_f32(ctx.h, 14, x.data_ptr(), wbuf.data_ptr(), None, y.data_ptr(), 1, 8, 256, 52, 0, s) == 1
    assert lib.bpq4k_kq_matmul_f32(ctx.h, 13, x.data_ptr(), wbuf.data_ptr() + 4, None, y.data_ptr(), 1, 8, 256, 44, 0, s) == 3
    assert lib.bpq4k_kq_gather_f32(ctx.h, 12, wbuf.data_ptr(), 8, 256, 36, x.data_ptr(), 1, y.data_ptr(), s) == 2
    assert lib.bpq4k_kq_dequant_f32(ctx.h, 14, None, 8, 256, 53, y.data_ptr(), s) == 1
    assert isinstance(Q4KError(2, "x"), RuntimeError)


def argmax_oracle(v):
    """The reference's argmax.wgsl / argmax_reduce.wgsl where the maximum is unique: strict > against a
    start of -1e30, index 0 when nothing wins; lowest index on ties."""
    v = np.asarray(v, np.float32)
    ok = v > np.float32(-1e30)          # False for NaN too
    if not ok.any():
        return 0
    m = v[ok].max()
    return int(np.flatnonzero(ok & (v == m))[0])


@pytest.mark.parametrize("n", [1, 7, 256, 1000, 32000, 128256, 400000])
def test_argmax_matches_reference_rule(ctx, n):
    import torch

    rng = np.random.default_rng(n)
    cases = [rng.standard_normal(n).astype(np.float32) * 10]
    t = cases[0].copy(); t[n // 2] = t.max() + 1; t[n - 1] = t[n // 2]; cases.append(t)       # a tie: lowest index wins
    t = cases[0].copy(); t[: max(1, n // 3)] = np.nan; cases.append(t)                           # NaNs never win
    cases.append(np.full(n, -2e30, np.float32))                                                   # nothing above the start value
    t = np.full(n, -np.inf, np.float32); t[n - 1] = -5.0; cases.append(t)                         # maximum at the very end
    cases.append(-np.abs(cases[0]) - 1)                                                           # all negative
    for v in cases:
        got = int(ctx.argmax(dev(torch, v)).cpu()[0])
        assert got == argmax_oracle(v)
    # back to back on one stream: the scratch words are left clean
    a = dev(torch, cases[0]); b = dev(torch, cases[5])
    r1, r2 = ctx.argmax(a), ctx.argmax(b)
    assert (int(r1.cpu()[0]), int(r2.cpu()[0])) == (argmax_oracle(cases[0]), argmax_oracle(cases[5]))


@pytest.mark.parametrize("layout,ftype", [(orc.Q5_K, orc.Q5_K), (Q6_K_PADDED, orc.Q6_K)], ids=["q5k", "q6k_padded"])
@pytest.mark.parametrize("mode,tol", [(0, 1e-3), (1, 1e-3), (2, 8e-3)], ids=["f16x3", "f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(25, 130, 512), (64, 256, 256), (100, 300, 1024), (512, 1024, 4096), (300, 1000, 14336)])
def test_siblings_many_rows_run_the_tensor_core_kernel(ctx, M, N, K, mode, tol, layout, ftype):
    """Q5_K and padded Q6_K from M = 25 on: tcgen05 kernel with the codes assembled before dequantisation.
    The three-pass mode keeps the float tolerance; the single-pass modes are held to their rounding."""
    import torch

    from backpack_b200 import q4k

    raw = synth.make_kq_weights(ftype, N, K, 500 + N)
    x = synth.make_activations(M, K, 501)
    bias = np.linspace(-2, 2, N).astype(np.float32)
    w = ctx.upload(pack_kq(layout, raw, N, K))
    want = orc.kq_matmul(ftype, x, raw, bias, N, K, threads=8)
    ctx.set_option(q4k.OPT_PREFILL_MODE, mode)
    try:
        ctx.launch_count(reset=True)
        y = ctx.matmul(dev(torch, x), w, bias=dev(torch, bias)).cpu().numpy()
        assert ctx.launch_count() in (2, 3)      # cast + tensor-core kernel (+ split-K reduction)
    finally:
        ctx.set_option(q4k.OPT_PREFILL_MODE, q4k.PREFILL_F16X3)
    if mode == 0:
        check(y, want)
    else:
        assert rel_l2(y, want) <= tol
    assert ctx.device_status() == 0


@pytest.mark.parametrize("qtype", [orc.Q5_K, Q6_K_PADDED])
@pytest.mark.parametrize("E,N,K,S", [(6, 48, 1024, 9), (3, 40, 256, 1), (16, 768, 2048, 64), (12, 16, 512, 200)])
def test_expert_indexed_form_of_the_siblings(ctx, qtype, E, N, K, S):
    """The indirect (expert-stacked) form on Q5_K and padded Q6_K weights: every slot multiplies its own activation
    row with the rows of its expert, one launch for all slots."""
    import torch

    ftype = file_type(qtype)
    raw = synth.make_kq_weights(ftype, E * N, K, 61)
    x = synth.make_activations(4, K, 62)
    rng = np.random.default_rng(63)
    experts = rng.integers(0, E, S).astype(np.uint32)
    x_rows = rng.integers(0, 4, S).astype(np.uint32)
    bias = np.linspace(-1, 1, N).astype(np.float32)
    w = ctx.upload(pack_kq(qtype, raw, E * N, K))
    ctx.launch_count(reset=True)
    y = ctx.matmul_moe(dev(torch, x), w, N, dev(torch, (experts * N).astype(np.int32)), x_rows=dev(torch, x_rows.astype(np.int32)),
                       bias=dev(torch, bias)).cpu().numpy()
    assert ctx.launch_count() == 1
    rawr = raw.reshape(E, N, -1)
    for s in range(min(S, 48)):
        want = orc.kq_matmul(ftype, x[x_rows[s]:x_rows[s] + 1], rawr[experts[s]], bias, N, K)[0]
        check(y[s], want)
    assert ctx.device_status() == 0


def test_expert_indexed_form_rejects_unpadded_q6k(ctx):
    import torch
    from backpack_b200 import Q4KError

    raw = synth.make_kq_weights(orc.Q6_K, 32, 256, 1)
    w = ctx.upload(pack_kq(orc.Q6_K, raw, 32, 256))
    with pytest.raises(Q4KError):
        ctx.matmul_moe(dev(torch, synth.make_activations(1, 256, 2)), w, 16, dev(torch, np.zeros(1, np.int32)))


@pytest.mark.parametrize("layout", [orc.Q6_K, Q6_K_PADDED])
@pytest.mark.parametrize("N,K", [(1, 256), (37, 768), (512, 4096)])
def test_respace_on_device_equals_host_pack(ctx, layout, N, K):
    """bpq4k_kq_respace_device writes the same bytes as bpq4k_kq_pack_host, gaps zeroed."""
    import torch
    from backpack_b200 import Q4KError
    raw = synth.make_kq_weights(orc.Q6_K, N, K, 5)
    want = pack_kq(layout, raw, N, K)
    w = ctx.respace_q6k(dev(torch, raw.reshape(-1)), N, K, layout)
    assert w.rowStrideWords == want.rowStrideWords and w.qtype == layout
    got = w.buf[: want.data.size * 4].cpu().numpy()
    assert np.array_equal(got, want.data.view(np.uint8))
    with pytest.raises(Q4KError):    # only Q6_K needs re-spacing
        ctx._check(ctx.lib.bpq4k_kq_respace_device(ctx.h, orc.Q5_K, w.buf.data_ptr(), N, K, w.buf.data_ptr(), 0))
