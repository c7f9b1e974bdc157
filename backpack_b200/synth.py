"""Seeded synthetic Q4_K tensors and activations.

The reference measures whole models from a private model zoo; here every
tensor is synthetic with the value distributions the benchmark configurations
state: per 144-byte super-block an fp16 ``d`` ~ U(1e-3, 2e-2), an fp16
``dmin`` ~ U(0, 1e-2), twelve packed scale/min bytes uniform 0..255 (which
makes each decoded 6-bit scale and min uniform 0..63) and 128 code bytes
uniform 0..255 (nibbles uniform 0..15).  Activations are float32 N(0, 1).

Generator: ``numpy.random.default_rng(seed)`` (PCG64), fixed draw order
``d, dmin, scales, codes`` for weights; activations use their own seed.
The byte layout is the raw GGUF one the reference uploads unchanged
(runtime/gguf_loader.cpp:359-379): row-major [N][K/256] blocks, no padding.
"""
from __future__ import annotations

import zlib

import numpy as np

BLOCK_BYTES = 144
QK_K = 256


def row_bytes(K: int) -> int:
    if K % QK_K:
        raise ValueError(f"K={K} is not a multiple of {QK_K}")
    return (K // QK_K) * BLOCK_BYTES


def make_q4k_weights(N: int, K: int, seed: int = 0) -> np.ndarray:
    """uint8 [N, K/256*144] raw Q4_K super-blocks."""
    nb = K // QK_K
    if K % QK_K:
        raise ValueError(f"K={K} is not a multiple of {QK_K}")
    rng = np.random.default_rng(seed)
    nblk = N * nb
    d = rng.uniform(1e-3, 2e-2, nblk).astype(np.float16)
    dmin = rng.uniform(0.0, 1e-2, nblk).astype(np.float16)
    scales = rng.integers(0, 256, (nblk, 12), dtype=np.uint8)
    codes = rng.integers(0, 256, (nblk, 128), dtype=np.uint8)
    blk = np.empty((nblk, BLOCK_BYTES), np.uint8)
    blk[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
    blk[:, 2:4] = dmin.view(np.uint8).reshape(nblk, 2)
    blk[:, 4:16] = scales
    blk[:, 16:] = codes
    return blk.reshape(N, nb * BLOCK_BYTES)


# Sibling K-quant formats (reference GGUFType numbers, runtime/gguf_loader.h:27-30).
Q4_K, Q5_K, Q6_K = 12, 13, 14
KQ_BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210}


def make_kq_weights(qtype: int, N: int, K: int, seed: int = 0) -> np.ndarray:
    """uint8 [N, K/256*block_bytes] raw super-blocks of a K-quant type, GGUF layout, no padding.

    Q5_K: d, dmin and scale bytes as for Q4_K, 32 fifth-bit bytes and 128 nibble bytes uniform.
    Q6_K: 128 + 64 code bytes uniform (6-bit codes uniform 0..63), 16 signed scales uniform
    -128..127, fp16 d ~ U(1e-4, 2e-3) (so that weights have a spread of order 1).
    """
    if qtype == Q4_K:
        return make_q4k_weights(N, K, seed)
    if K % QK_K:
        raise ValueError(f"K={K} is not a multiple of {QK_K}")
    nb = K // QK_K
    rng = np.random.default_rng(seed)
    nblk = N * nb
    bb = KQ_BLOCK_BYTES[qtype]
    blk = np.empty((nblk, bb), np.uint8)
    if qtype == Q5_K:
        d = rng.uniform(1e-3, 2e-2, nblk).astype(np.float16)
        dmin = rng.uniform(0.0, 1e-2, nblk).astype(np.float16)
        blk[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
        blk[:, 2:4] = dmin.view(np.uint8).reshape(nblk, 2)
        blk[:, 4:16] = rng.integers(0, 256, (nblk, 12), dtype=np.uint8)
        blk[:, 16:48] = rng.integers(0, 256, (nblk, 32), dtype=np.uint8)
        blk[:, 48:] = rng.integers(0, 256, (nblk, 128), dtype=np.uint8)
    elif qtype == Q6_K:
        d = rng.uniform(1e-4, 2e-3, nblk).astype(np.float16)
        blk[:, 0:192] = rng.integers(0, 256, (nblk, 192), dtype=np.uint8)
        blk[:, 192:208] = rng.integers(0, 256, (nblk, 16), dtype=np.uint8)
        blk[:, 208:210] = d.view(np.uint8).reshape(nblk, 2)
    else:
        raise ValueError(f"unknown K-quant type {qtype}")
    return blk.reshape(N, nb * bb)


def kq_weight_bytes(qtype: int, N: int, K: int) -> int:
    return N * (K // QK_K) * KQ_BLOCK_BYTES[qtype]


def kq_algorithmic_bytes(qtype: int, M: int, N: int, K: int, bias: bool = False) -> int:
    """As algorithmic_bytes, with the file-format block size of the type (no padding counted)."""
    return kq_weight_bytes(qtype, N, K) + M * K * 4 + M * N * 4 + (N * 4 if bias else 0)


def make_activations(M: int, K: int, seed: int = 0) -> np.ndarray:
    """float32 [M, K] ~ N(0, 1)."""
    return np.random.default_rng(seed).standard_normal((M, K), dtype=np.float32)


def shape_seed(config: str, name: str) -> int:
    """Stable per-(config, projection) seed so every shape has its own stream."""
    return zlib.crc32(f"{config}/{name}".encode()) & 0x7FFFFFFF


# Projection shapes (name, N, K) of the benchmark configurations.
LLAMA3_8B = [
    ("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
    ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336),
    ("lm_head", 128256, 4096),
]
LLAMA3_70B = [
    ("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
    ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672),
    ("lm_head", 128256, 8192),
]
QWEN3_MOE = {"experts": 128, "hidden": 2048, "ffn": 768, "tokens": 8, "topk": 8}


def weight_bytes(N: int, K: int) -> int:
    return N * row_bytes(K)


def algorithmic_bytes(M: int, N: int, K: int, bias: bool = False) -> int:
    """Bytes one matmul call must move: weights once, activations once, outputs once."""
    return weight_bytes(N, K) + M * K * 4 + M * N * 4 + (N * 4 if bias else 0)


def make_moe_routing(tokens: int, experts: int, topk: int, seed: int = 0) -> np.ndarray:
    """int32 [tokens, topk] expert ids, per token uniform without replacement."""
    rng = np.random.default_rng(seed)
    return np.stack([rng.choice(experts, topk, replace=False) for _ in range(tokens)]).astype(np.int32)
