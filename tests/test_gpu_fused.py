"""The single-row matmul with a fused prologue (RMSNorm, gelu*up, silu*up) and residual epilogue,
through the C ABI, against the oracle's restatement of the reference's fused decode shaders followed
by its expected-value matmul."""
import numpy as np
import pytest

from backpack_b200 import pack_kq, q4k, synth
from conftest import rel_l2
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check(y, want):
    assert rel_l2(y, want) <= 1e-3
    assert float(np.abs(y - want).max()) <= 2e-2 * max(1.0, float(np.abs(want).max()) / 100.0)


@pytest.mark.parametrize("qtype", [orc.Q4_K, orc.Q5_K, orc.Q6_K])
@pytest.mark.parametrize("kind", [q4k.PROLOGUE_RMSNORM, q4k.PROLOGUE_GELU_MUL, q4k.PROLOGUE_SILU_MUL])
@pytest.mark.parametrize("N,K", [(64, 256), (333, 1024), (4096, 4096), (1000, 14336)])
def test_fused_prologue_matches_oracle(ctx, qtype, kind, N, K):
    import torch

    layout = q4k.Q6_K_PADDED if qtype == orc.Q6_K else qtype     # Q6_K: the padded device layout of the fast kernel
    raw = synth.make_kq_weights(qtype, N, K, 300 + N)
    x = synth.make_activations(1, K, 301)[0] * (3.0 if kind == q4k.PROLOGUE_RMSNORM else 1.0)
    aux = (synth.make_activations(1, K, 302)[0] * 0.5 + 1.0).astype(np.float32)
    bias = np.linspace(-1, 1, N).astype(np.float32)
    res = synth.make_activations(1, N, 303)[0]
    eps = 1e-5
    xp = orc.prologue(kind, x, aux, eps)
    want = orc.kq_matmul(qtype, xp, raw, bias, N, K, threads=4)[0] + res
    w = ctx.upload(pack_kq(layout, raw, N, K))
    ctx.launch_count(reset=True)
    y = ctx.matmul_fused(dev(torch, x), w, kind, aux=dev(torch, aux), eps=eps, bias=dev(torch, bias),
                         residual=dev(torch, res)).cpu().numpy()[0]
    assert ctx.launch_count() == 1          # one kernel: nothing runs ahead of or behind the matmul
    check(y, want)
    # the unfused sequence through the plain entry point gives the same numbers
    y2 = ctx.matmul(dev(torch, xp[None, :]), w, bias=dev(torch, bias)).cpu().numpy()[0] + res
    assert rel_l2(y, y2) < 1e-5


def test_fused_none_with_residual_and_offset(ctx):
    import torch

    N, K = 200, 512
    raw = synth.make_q4k_weights(N, K, 5)
    x = synth.make_activations(1, K, 6)
    res = synth.make_activations(1, N, 7)[0]
    w = ctx.upload(pack_kq(orc.Q4_K, raw, N, K))
    out = torch.full((3 * N,), 9.0, device="cuda")
    ctx.matmul_fused(dev(torch, x), w, residual=dev(torch, res), out=out, y_offset=N)
    got = out.cpu().numpy()
    check(got[N:2 * N], orc.matmul(x, raw, None, N, K)[0] + res)
    assert (got[:N] == 9.0).all() and (got[2 * N:] == 9.0).all()


def test_fused_errors(ctx):
    import torch

    lib = ctx.lib
    x = torch.zeros(256, device="cuda")
    wbuf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    y = torch.zeros(8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(), None, 0.0, wbuf.data_ptr(), None, None, y.data_ptr(), 8, 256, 36, 0, s)
    assert lib.bpq4k_matmul_fused_f32(ctx.h, 14, 0, *args) == 2          # file-format Q6_K has no fused form (the padded layout has)
    assert lib.bpq4k_matmul_fused_f32(ctx.h, 12, 7, *args) == 1          # unknown prologue
    assert lib.bpq4k_matmul_fused_f32(ctx.h, 12, 1, *args) == 1          # RMSNorm without its weight
    assert lib.bpq4k_matmul_fused_f32(ctx.h, 12, 0, *args) == 0
