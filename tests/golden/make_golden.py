"""Generate the committed golden vectors for the Q4_K path.

Run in a container where the reference tree is mounted and
``oracle/_ref/libq4k_ref.so`` has been built from it (``make -C oracle ref``):

    python tests/golden/make_golden.py

Inputs follow the four formula-defined Q4_K fixtures of the reference's
runtime/tests/kernel_test.cpp (``q4k_matmul_reference`` :1678-1685,
``q4k_matmul_128_reference`` :1687-1689, ``q4k_matmul_batched4_reference``
:1726-1730, ``q4k_matmul_batched8_reference`` :1744-1748): the same block-byte
formulas, the same xoshiro128+ generator with Box-Muller normals (:62-99) and
the same truncating float->half conversion (:103-112).  The reference stores
no expected numbers; its tests compute them with ``dequant_kquant`` plus a
float dot product.  Here those expected numbers are produced by that same
reference code (compiled from its sources) and written next to the inputs, so
they can be checked on machines where the reference tree is absent.

Two further fixtures use the same reference code on inputs of our own:
``corner`` (hand-made blocks: subnormal/zero/negative d and dmin, saturated
and empty scale bytes, extreme code bytes) and ``synthetic`` (a small slice of
the seeded synthetic distribution the benchmarks use).

Output: tests/golden/q4k_golden.npz
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import q4k_oracle as orc  # noqa: E402
from backpack_b200 import synth  # noqa: E402

U32 = 0xFFFFFFFF
f32 = np.float32


class Rng:
    """xoshiro128+ with the seeding, warm-up and float mapping of kernel_test.cpp:62-99."""

    def __init__(self, seed: int):
        self.s = [seed & U32, (seed ^ 0x9E3779B9) & U32, (seed ^ 0x6A09E667) & U32, (seed ^ 0xBB67AE85) & U32]
        for _ in range(8):
            self.next()

    def next(self) -> int:
        s = self.s
        t = (s[1] << 9) & U32
        result = (s[0] + s[3]) & U32
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = ((s[3] << 11) | (s[3] >> 21)) & U32
        return result

    def uniform(self, lo, hi) -> np.float32:
        u = f32(self.next() >> 8) / f32(1 << 24)
        return f32(f32(lo) + u * f32(f32(hi) - f32(lo)))

    def randn(self) -> np.float32:
        u1 = self.uniform(1e-6, 1.0)
        u2 = self.uniform(0.0, 6.2831853)
        return f32(np.sqrt(f32(-2.0) * np.log(u1), dtype=f32) * np.cos(u2, dtype=f32))

    def randn_vec(self, n: int) -> np.ndarray:
        return np.array([self.randn() for _ in range(n)], f32)


def f32_to_f16_trunc(v) -> int:
    """Truncating float->half of kernel_test.cpp:103-112 (flushes subnormals to zero)."""
    u = int(np.array([v], f32).view(np.uint32)[0])
    sign = (u >> 16) & 0x8000
    e = ((u >> 23) & 0xFF) - 127 + 15
    frac = (u >> 13) & 0x3FF
    if e <= 0:
        return sign
    if e >= 31:
        return sign | 0x7C00
    return sign | (e << 10) | frac


def put_half(dst: np.ndarray, off: int, h: int) -> None:
    dst[off] = h & 255
    dst[off + 1] = h >> 8


def blocks_single(N: int) -> np.ndarray:
    """kernel_test.cpp:1680 -- K=256, one block per row."""
    raw = np.zeros((N, 144), np.uint8)
    for n in range(N):
        put_half(raw[n], 0, f32_to_f16_trunc(f32(.02) + f32(.001) * f32(n)))
        put_half(raw[n], 2, f32_to_f16_trunc(f32(.01) + f32(.0005) * f32(n)))
        for i in range(4, 144):
            raw[n, i] = (n * 31 + i * 17 + 3) & 255
    return raw


def blocks_multi(N: int, NB: int) -> np.ndarray:
    """kernel_test.cpp:1688, 1727, 1745 -- NB blocks per row."""
    raw = np.zeros((N, NB, 144), np.uint8)
    for n in range(N):
        for b in range(NB):
            put_half(raw[n, b], 0, f32_to_f16_trunc(f32(.02) + f32(.001) * f32(n)))
            put_half(raw[n, b], 2, f32_to_f16_trunc(f32(.01) + f32(.0002) * f32(b)))
            for j in range(4, 144):
                raw[n, b, j] = (n * 31 + b * 13 + j * 17) & 255
    return raw.reshape(N, NB * 144)


def corner_blocks() -> np.ndarray:
    """Hand-made super-blocks that hit the decode's edge cases (K=256, one block per row)."""
    rows = []

    def blk(d_bits, m_bits, scale_bytes, code_fill):
        b = np.zeros(144, np.uint8)
        put_half(b, 0, d_bits)
        put_half(b, 2, m_bits)
        b[4:16] = scale_bytes
        b[16:] = code_fill
        rows.append(b)

    ramp = (np.arange(128) * 37 + 11) & 255
    blk(0x2000, 0x1C00, 0xFF, 0xFF)                 # all scales/mins 63, all codes 15
    blk(0x2000, 0x1C00, 0x00, 0x00)                 # everything zero but d, dmin
    blk(0x0001, 0x0001, 0xFF, ramp)                 # smallest subnormal d and dmin
    blk(0x03FF, 0x0200, np.arange(12) * 21 & 255, ramp)   # largest subnormal d, mid subnormal dmin
    blk(0x0000, 0x2100, 0xA5, ramp)                 # d == 0
    blk(0x2400, 0x0000, 0x5A, ramp)                 # dmin == 0
    blk(0xA400, 0x2100, np.arange(12) * 13 + 7 & 255, ramp)   # negative d
    blk(0x2400, 0xA100, np.arange(12) * 29 + 3 & 255, ramp)   # negative dmin
    blk(0x8000, 0x8000, 0xFF, 0xF0)                 # negative zeros, codes hi=15 lo=0
    blk(0x3C00, 0x3C00, 0x3F, 0x0F)                 # d = dmin = 1, codes hi=0 lo=15
    blk(0x7BFF, 0x0000, 0x01, 0x11)                 # largest finite half as d
    blk(0x1234, 0x0456, np.array([0x40, 0x80, 0xC0, 0xFF, 0x3F, 0x7F, 0xBF, 0x00, 0xF0, 0x0F, 0xAA, 0x55]), ramp)
    return np.stack(rows)


def expected(x, raw, bias, N, K):
    """deq and y from the REFERENCE's code (dequant_kquant + the tests' float dot)."""
    deq = orc.dequant(raw, N, K, use_ref=True)
    y = orc.matmul(x, raw, bias, N, K, use_ref=True)
    return deq, y


def main() -> None:
    if not orc.ref_available():
        raise SystemExit("oracle/_ref/libq4k_ref.so missing: run `make -C oracle ref` with the reference mounted")
    out = {}

    def add(name, x, raw, bias, N, K):
        deq, y = expected(x, raw, bias, N, K)
        out[f"{name}.x"] = x.reshape(-1, K)
        out[f"{name}.raw"] = raw.reshape(N, -1)
        out[f"{name}.bias"] = bias if bias is not None else np.zeros(N, f32)
        out[f"{name}.deq"] = deq
        out[f"{name}.y"] = y
        out[f"{name}.shape"] = np.array([x.size // K, N, K], np.int64)

    # q4k_matmul_reference
    N, K = 8, 256
    add("kt_q4k_matmul", Rng(4343).randn_vec(K), blocks_single(N), None, N, K)
    # q4k_matmul_128_reference
    N, K = 7, 512
    add("kt_q4k_matmul_128", Rng(5555).randn_vec(K), blocks_multi(N, 2),
        np.array([f32(.01) * f32(n) for n in range(N)], f32), N, K)
    # q4k_matmul_batched4_reference
    M, N, K = 5, 9, 512
    add("kt_q4k_matmul_batched4", Rng(4848).randn_vec(M * K), blocks_multi(N, 2),
        np.array([f32(.01) * f32(n) for n in range(N)], f32), N, K)
    # q4k_matmul_batched8_reference
    M, N, K = 9, 9, 512
    add("kt_q4k_matmul_batched8", Rng(5151).randn_vec(M * K), blocks_multi(N, 2),
        np.array([f32(.01) * f32(n) for n in range(N)], f32), N, K)
    # corner cases
    raw = corner_blocks()
    add("corner", synth.make_activations(3, 256, 77), raw, None, raw.shape[0], 256)
    # slice of the synthetic benchmark distribution (config-0 recipe, smaller)
    N, K, M = 96, 1024, 4
    add("synthetic", synth.make_activations(M, K, 1), synth.make_q4k_weights(N, K, 0),
        None, N, K)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "q4k_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
