"""Generate the committed golden vectors for the Q5_K and Q6_K siblings of the Q4_K path.

Run in a container where the reference tree is mounted and
``oracle/_ref/libq4k_ref.so`` has been built from it (``make -C oracle ref``):

    python tests/golden/make_golden_kq.py

Inputs follow the formula-defined fixtures of the reference's
runtime/tests/kernel_test.cpp: ``q5k_matmul_reference`` (:1669-1676),
``q6k_matmul_reference`` (:1691-1698), ``q6k_gather_reference``,
``q6k_matmul_wide_reference``, ``q6k_gather_batched_reference``,
``q5k_matmul_batched4_reference`` and ``q6k_matmul_batched4_reference``
(:1700-1742), with the generator and the truncating half conversion of
make_golden.py.  The expected numbers come from the reference's own
``dequant_kquant`` and the tests' float dot product, compiled from its sources.
The gather fixtures store the token ids; their expected output is rows of ``deq``.

Two fixtures per type use the same reference code on inputs of our own:
``corner_*`` (extreme scales and super-block factors) and ``synthetic_*`` (a
slice of the seeded distribution the benchmark uses).

Output: tests/golden/kq_golden.npz
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from oracle import q4k_oracle as orc  # noqa: E402
from backpack_b200 import synth  # noqa: E402
from make_golden import Rng, f32_to_f16_trunc, put_half  # noqa: E402

f32 = np.float32
Q5_K, Q6_K = 13, 14


def u8(v: int) -> int:
    return v & 255


def q5k_blocks(N, NB, byte_fn, d_fn, dm_fn):
    raw = np.zeros((N, NB, 176), np.uint8)
    for n in range(N):
        for b in range(NB):
            put_half(raw[n, b], 0, f32_to_f16_trunc(d_fn(n, b)))
            put_half(raw[n, b], 2, f32_to_f16_trunc(dm_fn(n, b)))
            for i in range(4, 176):
                raw[n, b, i] = u8(byte_fn(n, b, i))
    return raw.reshape(N, NB * 176)


def q6k_blocks(N, NB, byte_fn, d_fn):
    raw = np.zeros((N, NB, 210), np.uint8)
    for n in range(N):
        for b in range(NB):
            for i in range(208):
                raw[n, b, i] = u8(byte_fn(n, b, i))
            put_half(raw[n, b], 208, f32_to_f16_trunc(d_fn(n, b)))
    return raw.reshape(N, NB * 210)


def lin(*terms):
    """c0 + c1*v1 + c2*v2 ... evaluated left to right in float32, as the C expressions are."""
    acc = f32(terms[0])
    for c, v in terms[1:]:
        acc = f32(acc + f32(f32(c) * f32(v)))
    return acc


def corner_q5k() -> np.ndarray:
    rows = []
    ramp = (np.arange(128) * 37 + 11) & 255

    def blk(d_bits, m_bits, scale_bytes, qh_fill, code_fill):
        b = np.zeros(176, np.uint8)
        put_half(b, 0, d_bits)
        put_half(b, 2, m_bits)
        b[4:16] = scale_bytes
        b[16:48] = qh_fill
        b[48:] = code_fill
        rows.append(b)

    blk(0x2000, 0x1C00, 0xFF, 0xFF, 0xFF)                  # every code 31, scales and mins 63
    blk(0x2000, 0x1C00, 0x00, 0x00, 0x00)                  # all zero but d, dmin
    blk(0x0001, 0x0001, 0xFF, 0xAA, ramp)                  # smallest subnormal factors
    blk(0x0000, 0x2100, 0xA5, 0x55, ramp)                  # d == 0
    blk(0x2400, 0x0000, 0x5A, 0x0F, ramp)                  # dmin == 0
    blk(0xA400, 0x2100, (np.arange(12) * 13 + 7) & 255, 0xF0, ramp)     # negative d
    blk(0x2400, 0xA100, (np.arange(12) * 29 + 3) & 255, (np.arange(32) * 9 + 1) & 255, ramp)  # negative dmin
    blk(0x3C00, 0x3C00, 0x3F, 0x01, 0x0F)                  # d = dmin = 1, fifth bit only in sub-block 0
    blk(0x7BFF, 0x0000, 0x01, 0x80, 0x11)                  # largest finite half, fifth bit only in sub-block 7
    return np.stack(rows)


def corner_q6k() -> np.ndarray:
    rows = []
    ramp = (np.arange(192) * 37 + 11) & 255

    def blk(codes, scales, d_bits):
        b = np.zeros(210, np.uint8)
        b[0:192] = codes
        b[192:208] = scales
        put_half(b, 208, d_bits)
        rows.append(b)

    blk(0xFF, 0x7F, 0x2000)                                # every code 63 (q = 31), scales +127
    blk(0x00, 0x80, 0x2000)                                # every code 0 (q = -32), scales -128
    blk(ramp, 0x00, 0x2400)                                # zero scales
    blk(ramp, (np.arange(16) * 17 + 3) & 255, 0x0001)      # smallest subnormal d
    blk(ramp, (np.arange(16) * 31 + 129) & 255, 0xA400)    # negative d, mixed-sign scales
    blk(ramp, 0x01, 0x7BFF)                                # largest finite half
    blk(ramp, 0xFF, 0x8000)                                # d = -0, scales -1
    blk(np.concatenate([np.full(128, 0x20), np.full(64, 0xAA)]), 0x40, 0x1C00)   # q = 0 everywhere (code 32)
    return np.stack(rows)


def main() -> None:
    if not orc.ref_available():
        raise SystemExit("oracle/_ref/libq4k_ref.so missing: run `make -C oracle ref` with the reference mounted")
    out = {}

    def add(name, qtype, x, raw, bias, N, K, tokens=None):
        out[f"{name}.type"] = np.array([qtype], np.int64)
        out[f"{name}.raw"] = raw.reshape(N, -1)
        out[f"{name}.deq"] = orc.kq_dequant(qtype, raw, N, K, use_ref=True)
        if x is not None:
            out[f"{name}.x"] = x.reshape(-1, K)
            out[f"{name}.bias"] = bias if bias is not None else np.zeros(N, f32)
            out[f"{name}.y"] = orc.kq_matmul(qtype, x, raw, bias, N, K, use_ref=True)
        if tokens is not None:
            out[f"{name}.tokens"] = np.array(tokens, np.uint32)
        out[f"{name}.shape"] = np.array([0 if x is None else x.size // K, N, K], np.int64)

    def bias_of(N):
        return np.array([f32(.01) * f32(n) for n in range(N)], f32)

    # q5k_matmul_reference
    N, K = 8, 256
    add("kt_q5k_matmul", Q5_K, Rng(4242).randn_vec(K),
        q5k_blocks(N, 1, lambda n, b, i: n * 37 + i * 13 + 7, lambda n, b: lin(.02, (.001, n)), lambda n, b: lin(.01, (.0005, n))),
        None, N, K)
    # q6k_matmul_reference
    N, K = 8, 768
    add("kt_q6k_matmul", Q6_K, Rng(4646).randn_vec(K),
        q6k_blocks(N, 3, lambda n, q, i: n * 29 + q * 23 + i * 19 + 5, lambda n, q: lin(.02, (.001, n), (.0003, q))), None, N, K)
    # q6k_gather_reference (token 2 of 3 rows)
    N, K = 3, 768
    add("kt_q6k_gather", Q6_K, None,
        q6k_blocks(N, 3, lambda n, b, i: n * 41 + b * 23 + i * 11 + 9, lambda n, b: lin(.015, (.001, n), (.0002, b))), None, N, K,
        tokens=[2])
    # q6k_matmul_wide_reference
    N, K = 19, 768
    add("kt_q6k_matmul_wide", Q6_K, Rng(4747).randn_vec(K),
        q6k_blocks(N, 3, lambda n, b, i: n * 37 + b * 17 + i * 13 + 11, lambda n, b: lin(.018, (.0007, n), (.0002, b))),
        bias_of(N), N, K)
    # q6k_gather_batched_reference
    N, K = 4, 768
    add("kt_q6k_gather_batched", Q6_K, None,
        q6k_blocks(N, 3, lambda n, b, i: n * 43 + b * 19 + i * 7 + 3, lambda n, b: lin(.014, (.001, n))), None, N, K,
        tokens=[3, 0, 2])
    # q5k_matmul_batched4_reference
    M, N, K = 5, 9, 512
    add("kt_q5k_matmul_batched4", Q5_K, Rng(4949).randn_vec(M * K),
        q5k_blocks(N, 2, lambda n, b, i: n * 29 + b * 11 + i * 19, lambda n, b: lin(.02, (.001, n)), lambda n, b: lin(.01, (.0002, b))),
        bias_of(N), N, K)
    # q6k_matmul_batched4_reference
    M, N, K = 5, 9, 768
    add("kt_q6k_matmul_batched4", Q6_K, Rng(5050).randn_vec(M * K),
        q6k_blocks(N, 3, lambda n, b, i: n * 23 + b * 17 + i * 13, lambda n, b: lin(.018, (.0007, n), (.0002, b))),
        bias_of(N), N, K)
    # corner cases
    raw = corner_q5k()
    add("corner_q5k", Q5_K, synth.make_activations(3, 256, 78), raw, None, raw.shape[0], 256)
    raw = corner_q6k()
    add("corner_q6k", Q6_K, synth.make_activations(3, 256, 79), raw, None, raw.shape[0], 256)
    # slices of the synthetic benchmark distribution
    N, K, M = 48, 1024, 4
    add("synthetic_q5k", Q5_K, synth.make_activations(M, K, 1), synth.make_kq_weights(Q5_K, N, K, 0), None, N, K)
    add("synthetic_q6k", Q6_K, synth.make_activations(M, K, 1), synth.make_kq_weights(Q6_K, N, K, 0), None, N, K)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kq_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
