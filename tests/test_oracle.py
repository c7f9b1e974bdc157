"""The CPU checker itself: restatement vs. the reference-generated golden vectors,
vs. an independent numpy restatement, and vs. the compiled reference when present."""
import numpy as np
import pytest

from backpack_b200 import synth
from oracle import q4k_oracle as orc
from conftest import GOLDEN_CASES


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_dequant_matches_reference_golden_bit_exact(golden, case):
    M, N, K = golden[f"{case}.shape"]
    got = orc.dequant(golden[f"{case}.raw"], int(N), int(K))
    assert np.array_equal(bits(got), bits(golden[f"{case}.deq"]))


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_matmul_matches_reference_golden_bit_exact(golden, case):
    M, N, K = (int(v) for v in golden[f"{case}.shape"])
    got = orc.matmul(golden[f"{case}.x"], golden[f"{case}.raw"], golden[f"{case}.bias"], N, K)
    # same float operations in the same order as the reference's test code
    assert np.array_equal(bits(got), bits(golden[f"{case}.y"]))


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_numpy_restatement_agrees(golden, case):
    M, N, K = (int(v) for v in golden[f"{case}.shape"])
    assert np.array_equal(bits(orc.dequant_numpy(golden[f"{case}.raw"], N, K)), bits(golden[f"{case}.deq"]))


def test_fp16_widening_every_bit_pattern():
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    L = orc.lib()
    got = np.array([L.oracle_fp16_to_f32(int(v)) for v in h], np.float32)
    finite = np.isfinite(want)
    assert np.array_equal(bits(got[finite]), bits(want[finite]))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[np.isinf(want)], want[np.isinf(want)])


def test_threaded_equals_serial():
    N, K, M = 37, 768, 3
    w = synth.make_q4k_weights(N, K, 5)
    x = synth.make_activations(M, K, 6)
    bias = np.linspace(-1, 1, N).astype(np.float32)
    a = orc.matmul(x, w, bias, N, K)
    b = orc.matmul(x, w, bias, N, K, threads=4)
    assert np.array_equal(bits(a), bits(b))


def test_pack_is_identity_relayout():
    N, K = 5, 1024
    w = synth.make_q4k_weights(N, K, 3)
    words, rs, nb = orc.pack(w, N, K)
    assert (rs, nb) == (4 * 36, 4)
    assert np.array_equal(words.view(np.uint8), w.reshape(-1))


def test_moe_slots_equal_direct_on_expert_slices():
    E, N, K = 4, 16, 512
    w = synth.make_q4k_weights(E * N, K, 9)
    x = synth.make_activations(3, K, 10)
    ids = np.array([2, 0, 3], np.uint32)
    y = orc.matmul_moe(x, w, None, N, K, ids * N)
    for s, e in enumerate(ids):
        want = orc.matmul(x[s:s + 1], w[e * N:(e + 1) * N], None, N, K)
        assert np.array_equal(bits(y[s]), bits(want))


def test_empty_inputs():
    assert orc.dequant(np.zeros(0, np.uint8), 0, 256).shape == (0, 256)
    assert orc.matmul(np.zeros((0, 256), np.float32), np.zeros(144, np.uint8), None, 1, 256).shape == (0, 1)


def test_synthetic_distribution_has_subnormal_dmin():
    # the U(0, 1e-2) draw of dmin reaches below the smallest normal half (6.1e-5)
    w = synth.make_q4k_weights(64, 4096, 0).reshape(-1, 144)
    dmin = w[:, 2:4].copy().view(np.float16).astype(np.float32).ravel()
    assert (dmin < 6.1e-5).any() and (dmin >= 0).all()


@pytest.mark.skipif(not orc.ref_available(), reason="compiled reference not present")
def test_restatement_equals_compiled_reference_on_random_blocks():
    N, K = 128, 2048
    w = synth.make_q4k_weights(N, K, 123)
    assert np.array_equal(bits(orc.dequant(w, N, K)), bits(orc.dequant(w, N, K, use_ref=True)))
    x = synth.make_activations(2, K, 4)
    assert np.array_equal(bits(orc.matmul(x, w, None, N, K)), bits(orc.matmul(x, w, None, N, K, use_ref=True)))
    wa, rsa, nba = orc.pack(w, N, K)
    wb, rsb, nbb = orc.pack(w, N, K, use_ref=True)
    assert (rsa, nba) == (rsb, nbb) and np.array_equal(wa, wb)
    # arbitrary bytes (every half bit pattern class appears): decode must still agree where finite
    rnd = np.random.default_rng(1).integers(0, 256, (64, 144 * 2), dtype=np.uint8)
    a, b = orc.dequant(rnd, 64, 512), orc.dequant(rnd, 64, 512, use_ref=True)
    ok = np.isfinite(b)
    assert np.array_equal(bits(a[ok]), bits(b[ok])) and np.array_equal(np.isnan(a), np.isnan(b))
