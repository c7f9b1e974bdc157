"""The CPU checker for the Q5_K / Q6_K siblings: restatement vs. the reference-generated golden
vectors, vs. an independent numpy restatement, and vs. the compiled reference when present."""
import numpy as np
import pytest

from backpack_b200 import synth
from oracle import q4k_oracle as orc
from conftest import KQ_GOLDEN_GATHER, KQ_GOLDEN_MATMUL

TYPES = [orc.Q4_K, orc.Q5_K, orc.Q6_K]


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("case", KQ_GOLDEN_MATMUL + KQ_GOLDEN_GATHER)
def test_dequant_matches_reference_golden_bit_exact(kq_golden, case):
    qtype = int(kq_golden[f"{case}.type"][0])
    _, N, K = (int(v) for v in kq_golden[f"{case}.shape"])
    got = orc.kq_dequant(qtype, kq_golden[f"{case}.raw"], N, K)
    assert np.array_equal(bits(got), bits(kq_golden[f"{case}.deq"]))
    assert np.array_equal(bits(orc.kq_dequant_numpy(qtype, kq_golden[f"{case}.raw"], N, K)), bits(kq_golden[f"{case}.deq"]))


@pytest.mark.parametrize("case", KQ_GOLDEN_MATMUL)
def test_matmul_matches_reference_golden_bit_exact(kq_golden, case):
    qtype = int(kq_golden[f"{case}.type"][0])
    _, N, K = (int(v) for v in kq_golden[f"{case}.shape"])
    got = orc.kq_matmul(qtype, kq_golden[f"{case}.x"], kq_golden[f"{case}.raw"], kq_golden[f"{case}.bias"], N, K)
    assert np.array_equal(bits(got), bits(kq_golden[f"{case}.y"]))


@pytest.mark.parametrize("qtype", TYPES)
def test_threaded_equals_serial_and_q4k_front(qtype):
    N, K, M = 37, 768, 3
    w = synth.make_kq_weights(qtype, N, K, 5)
    x = synth.make_activations(M, K, 6)
    bias = np.linspace(-1, 1, N).astype(np.float32)
    a = orc.kq_matmul(qtype, x, w, bias, N, K)
    assert np.array_equal(bits(a), bits(orc.kq_matmul(qtype, x, w, bias, N, K, threads=4)))
    if qtype == orc.Q4_K:   # the type-dispatching front agrees with the Q4_K entry points
        assert np.array_equal(bits(a), bits(orc.matmul(x, w, bias, N, K)))
        assert np.array_equal(bits(orc.kq_dequant(qtype, w, N, K)), bits(orc.dequant(w, N, K)))


@pytest.mark.parametrize("qtype,K,stride", [(orc.Q4_K, 1024, 144), (orc.Q5_K, 1024, 176), (orc.Q6_K, 1024, 210),
                                            (orc.Q6_K, 768, 158), (orc.Q6_K, 256, 53)])
def test_pack_pads_rows_to_words(qtype, K, stride):
    """Q6_K rows (210 bytes per block) are padded with zeros to a whole number of words."""
    N = 5
    w = synth.make_kq_weights(qtype, N, K, 3)
    words, rs, nb = orc.kq_pack(qtype, w, N, K)
    assert (rs, nb) == (stride, K // 256)
    rows = words.view(np.uint8).reshape(N, rs * 4)
    rb = nb * orc.KQ_BLOCK_BYTES[qtype]
    assert np.array_equal(rows[:, :rb], w)
    assert not rows[:, rb:].any()


@pytest.mark.skipif(not orc.ref_available(), reason="compiled reference not present")
@pytest.mark.parametrize("qtype", TYPES)
def test_against_compiled_reference(qtype):
    rng = np.random.default_rng(11)
    N, K, M = 9, 1280, 2
    bb = orc.KQ_BLOCK_BYTES[qtype]
    raw = rng.integers(0, 256, N * (K // 256) * bb, dtype=np.uint8)          # arbitrary bytes, NaN/inf factors included
    assert np.array_equal(bits(orc.kq_dequant(qtype, raw, N, K)), bits(orc.kq_dequant(qtype, raw, N, K, use_ref=True)))
    w = synth.make_kq_weights(qtype, N, K, 12)
    x = synth.make_activations(M, K, 13)
    assert np.array_equal(bits(orc.kq_matmul(qtype, x, w, None, N, K)), bits(orc.kq_matmul(qtype, x, w, None, N, K, use_ref=True)))
    a, b = orc.kq_pack(qtype, w, N, K), orc.kq_pack(qtype, w, N, K, use_ref=True)
    assert np.array_equal(a[0], b[0]) and a[1:] == b[1:]


def test_moe_ffn_loop_equals_its_parts():
    """The routed-expert restatement is the composition of the pinned pieces: matmuls on expert slices,
    the silu*up step, and a float32 accumulate in slot order."""
    E, H, F, T, topk = 3, 512, 256, 2, 2
    for qtype in (orc.Q4_K, orc.Q5_K):
        bb = orc.KQ_BLOCK_BYTES[qtype]
        rg, ru = synth.make_kq_weights(qtype, E * F, H, 1), synth.make_kq_weights(qtype, E * F, H, 2)
        rd = synth.make_kq_weights(qtype, E * H, F, 3)
        x = (synth.make_activations(T, H, 4) * 0.05).astype(np.float32)
        ids = np.array([[2, 0], [1, 2]])
        w = np.array([[0.25, 0.75], [0.6, 0.4]], np.float32)
        y0 = synth.make_activations(T, H, 5)
        got = orc.moe_ffn(qtype, x, rg, ru, rd, ids, w, y0, F, H)
        want = y0.copy()
        deq = [orc.kq_dequant(qtype, r, n, k) for r, n, k in ((rg, E * F, H), (ru, E * F, H), (rd, E * H, F))]
        for t in range(T):
            for k in range(topk):
                e = ids[t, k]
                g = deq[0][e * F:(e + 1) * F].astype(np.float64) @ x[t]
                u = deq[1][e * F:(e + 1) * F].astype(np.float64) @ x[t]
                act = g / (1 + np.exp(-g)) * u
                want[t] = want[t] + w[t, k] * (deq[2][e * H:(e + 1) * H].astype(np.float64) @ act).astype(np.float32)
        assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-5
        assert np.linalg.norm((got - y0) - (want - y0)) / np.linalg.norm(want - y0) < 1e-5
        assert bb in (144, 176)
