"""The routed-expert feed-forward step through the C ABI (bpq4k_moe_ffn_f32) against the oracle's
restatement of the reference's per-slot loop: gate, up, silu*up, down, weighted accumulate."""
import numpy as np
import pytest

from backpack_b200 import Q4KError, pack_kq, synth
from conftest import rel_l2
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_layer(ctx, qtype, E, H, F, seed):
    from backpack_b200 import q4k

    layout = q4k.Q6_K_PADDED if qtype == orc.Q6_K else qtype     # Q6_K stacks live in the padded device layout
    raws = [synth.make_kq_weights(qtype, E * F, H, seed), synth.make_kq_weights(qtype, E * F, H, seed + 1),
            synth.make_kq_weights(qtype, E * H, F, seed + 2)]
    ws = [ctx.upload(pack_kq(layout, raws[0], E * F, H)), ctx.upload(pack_kq(layout, raws[1], E * F, H)),
          ctx.upload(pack_kq(layout, raws[2], E * H, F))]
    return raws, ws


def routing_weights(T, topk, seed):
    rng = np.random.default_rng(seed)
    w = rng.random((T, topk)).astype(np.float32) + 0.05
    return (w / w.sum(axis=1, keepdims=True)).astype(np.float32)


@pytest.mark.parametrize("qtype", [orc.Q4_K, orc.Q5_K, orc.Q6_K])
@pytest.mark.parametrize("E,H,F,T,topk", [(4, 256, 256, 1, 1), (8, 512, 256, 3, 2), (16, 2048, 768, 8, 8), (6, 768, 1024, 5, 3),
                                          (16, 512, 256, 32, 8)])    # 256 slots: the down matmul runs as a unit list too
def test_moe_ffn_matches_reference_loop(ctx, qtype, E, H, F, T, topk):
    import torch

    raws, ws = make_layer(ctx, qtype, E, H, F, 40)
    # activations scaled so that gate/up outputs stay O(1) and the silu is exercised around zero
    x = (synth.make_activations(T, H, 43) * 0.05).astype(np.float32)
    ids = synth.make_moe_routing(T, E, topk, 44)
    rw = routing_weights(T, topk, 45)
    y0 = synth.make_activations(T, H, 46)
    y = dev(torch, y0.copy())
    ctx.moe_ffn(dev(torch, x), ws[0], ws[1], ws[2], dev(torch, ids.astype(np.int32)), dev(torch, rw), y, E)
    got = y.cpu().numpy()
    want = orc.moe_ffn(qtype, x, raws[0], raws[1], raws[2], ids, rw, y0, F, H)
    assert rel_l2(got, want) <= 1e-3
    assert rel_l2(got - y0, want - y0) <= 1e-3          # the added part alone, not hidden behind the residual
    scale = max(1.0, float(np.abs(want).max()) / 100.0)
    assert float(np.abs(got - want).max()) <= 2e-2 * scale
    assert ctx.device_status() == 0


def test_moe_ffn_equals_the_separate_calls(ctx):
    """Same numbers as the expert-indexed matmuls, the fused silu*up prologue and a float accumulate done by hand."""
    import torch

    qtype, E, H, F, T, topk = orc.Q4_K, 8, 1024, 512, 4, 4
    _, ws = make_layer(ctx, qtype, E, H, F, 50)
    x = dev(torch, (synth.make_activations(T, H, 53) * 0.05).astype(np.float32))
    ids = synth.make_moe_routing(T, E, topk, 54).reshape(-1)
    rw = routing_weights(T, topk, 55)
    y = torch.zeros(T, H, device="cuda")
    ctx.launch_count(reset=True)
    ctx.moe_ffn(x, ws[0], ws[1], ws[2], dev(torch, ids.astype(np.int32)), dev(torch, rw), y, E)
    assert ctx.launch_count() == 3                       # gate+up, down (with its prologue), accumulate
    x_rows = dev(torch, np.repeat(np.arange(T), topk).astype(np.int32))
    g = ctx.matmul_moe(x, ws[0], F, dev(torch, (ids * F).astype(np.int32)), x_rows=x_rows)
    u = ctx.matmul_moe(x, ws[1], F, dev(torch, (ids * F).astype(np.int32)), x_rows=x_rows)
    act = torch.nn.functional.silu(g) * u
    o = ctx.matmul_moe(act, ws[2], H, dev(torch, (ids * H).astype(np.int32))).reshape(T, topk, H)
    want = torch.zeros(T, H, device="cuda")
    for k in range(topk):
        want = want + dev(torch, rw[:, k:k + 1]) * o[:, k]
    assert rel_l2(y.cpu().numpy(), want.cpu().numpy()) <= 2e-6


def test_moe_ffn_expert_id_out_of_range_reads_zeros(ctx):
    import torch

    qtype, E, H, F, T, topk = orc.Q4_K, 4, 256, 256, 2, 2
    _, ws = make_layer(ctx, qtype, E, H, F, 60)
    x = dev(torch, synth.make_activations(T, H, 61))
    y0 = synth.make_activations(T, H, 62)
    y = dev(torch, y0.copy())
    ids = np.full((T, topk), E + 3, np.int32)            # no such expert: contributes nothing
    ctx.moe_ffn(x, ws[0], ws[1], ws[2], dev(torch, ids), dev(torch, routing_weights(T, topk, 1)), y, E)
    assert np.array_equal(y.cpu().numpy(), y0)
    assert ctx.device_status() == 0


def test_moe_ffn_errors(ctx):
    import torch

    qtype, E, H, F, T, topk = orc.Q4_K, 4, 256, 256, 2, 2
    _, ws = make_layer(ctx, qtype, E, H, F, 70)
    x = dev(torch, synth.make_activations(T, H, 71))
    y = torch.zeros(T, H, device="cuda")
    ids = dev(torch, np.zeros((T, topk), np.int32))
    rw = dev(torch, routing_weights(T, topk, 2))
    lib, h = ctx.lib, ctx.h
    need = lib.bpq4k_moe_ffn_work_floats(T, topk, H, F)
    assert need == T * topk * (2 * F + H)
    work = torch.empty(need, device="cuda")

    def call(qt=qtype, xp=x.data_ptr(), wk=work.data_ptr(), wn=need, Hh=H, Ff=F, t=T):
        return lib.bpq4k_moe_ffn_f32(h, qt, xp, ws[0].buf.data_ptr(), ws[1].buf.data_ptr(), ws[2].buf.data_ptr(),
                                     ids.data_ptr(), rw.data_ptr(), y.data_ptr(), t, topk, E, Hh, Ff, wk, wn, 0)

    assert call() == 0
    assert call(t=0) == 0                                  # nothing to do
    assert call(qt=orc.Q6_K) != 0                          # file-format Q6_K: no expert-indexed kernel (the padded layout has one)
    assert call(wn=need - 1) != 0 and "work holds" in lib.bpq4k_last_error_string(h).decode()
    assert call(xp=None) != 0
    assert call(wk=work.data_ptr() + 4) != 0               # misaligned scratch
    assert call(Hh=300) != 0                               # not a multiple of 256
    with pytest.raises(Q4KError):
        ctx._check(call(Ff=100))
