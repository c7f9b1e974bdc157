"""Python doorway to the CPU checker for the Q4_K path and its Q5_K / Q6_K siblings.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg; never by the shipped package.

Three things live here:

* ``lib()`` / ``ref_lib()`` -- ctypes handles on the C restatement
  (``_build/libq4k_oracle.so``) and, when it was built, on the reference's own
  ``gguf_loader.cpp`` (``_ref/libq4k_ref.so``).
* ``dequant`` / ``matmul`` / ``matmul_moe`` -- numpy-in, numpy-out wrappers.
* ``dequant_numpy`` -- an independent vectorised numpy restatement of the same
  decode (runtime/gguf_loader.cpp:455-496), used to cross-check the C one.

Parity status: pinned (see q4k_oracle.c).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BLOCK_BYTES = 144
QK_K = 256

_lib = None
_ref = None

_u32 = C.c_uint32
_fp = C.POINTER(C.c_float)


def build(ref_root: str | None = None) -> None:
    """Compile the restatement, and the reference shim when the reference tree can be found: `ref_root`,
    else the BPQ4K_REFERENCE_ROOT environment variable, else a directory `reference` beside this repository."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)
    ref_root = ref_root or os.environ.get("BPQ4K_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    if os.path.isfile(os.path.join(ref_root, "runtime", "gguf_loader.cpp")):
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={ref_root}"], check=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "_build", "libq4k_oracle.so")
        if not os.path.isfile(path):
            build()
        L = C.CDLL(path)
        L.oracle_fp16_to_f32.restype = C.c_float
        L.oracle_fp16_to_f32.argtypes = [C.c_uint16]
        L.oracle_q4k_dequant.argtypes = [C.c_void_p, _fp, _u32, _u32]
        L.oracle_pack_q4k.argtypes = [C.c_void_p, _u32, _u32, C.c_void_p, C.POINTER(_u32), C.POINTER(_u32)]
        L.oracle_q4k_matmul.argtypes = [_fp, C.c_void_p, _fp, _fp, _u32, _u32, _u32]
        L.oracle_q4k_matmul_mt.argtypes = [_fp, C.c_void_p, _fp, _fp, _u32, _u32, _u32, _u32]
        L.oracle_q4k_matmul_moe_slot.argtypes = [_fp, C.c_void_p, _fp, _fp, _u32, _u32, _u32,
                                                 C.POINTER(_u32), _u32, _u32]
        L.oracle_q4k_matmul_f64.argtypes = [_fp, C.c_void_p, _fp, C.POINTER(C.c_double), _u32, _u32, _u32]
        L.oracle_kq_block_bytes.restype = _u32
        L.oracle_kq_block_bytes.argtypes = [_u32]
        L.oracle_kq_dequant.argtypes = [_u32, C.c_void_p, _fp, _u32, _u32]
        L.oracle_kq_pack.argtypes = [_u32, C.c_void_p, _u32, _u32, C.c_void_p, C.POINTER(_u32), C.POINTER(_u32)]
        L.oracle_kq_matmul.argtypes = [_u32, _fp, C.c_void_p, _fp, _fp, _u32, _u32, _u32, _u32]
        L.oracle_prologue.argtypes = [_u32, _fp, _fp, C.c_float, _u32, _fp]
        _lib = L
    return _lib


def ref_available() -> bool:
    return os.path.isfile(os.path.join(HERE, "_ref", "libq4k_ref.so"))


def ref_lib() -> C.CDLL:
    """The reference's own code (built from its sources); raises if it was never built."""
    global _ref
    if _ref is None:
        L = C.CDLL(os.path.join(HERE, "_ref", "libq4k_ref.so"))
        L.ref_q4k_dequant.argtypes = [C.c_void_p, _fp, _u32, _u32]
        L.ref_pack_q4k.argtypes = [C.c_void_p, _u32, _u32, C.c_void_p, C.POINTER(_u32), C.POINTER(_u32)]
        L.ref_q4k_matmul.argtypes = [_fp, C.c_void_p, _fp, _fp, _u32, _u32, _u32, _u32]
        L.ref_kq_dequant.argtypes = [_u32, C.c_void_p, _fp, _u32, _u32]
        L.ref_kq_pack.argtypes = [_u32, C.c_void_p, _u32, _u32, C.c_void_p, C.POINTER(_u32), C.POINTER(_u32)]
        L.ref_kq_matmul.argtypes = [_u32, _fp, C.c_void_p, _fp, _fp, _u32, _u32, _u32, _u32]
        _ref = L
    return _ref


def _f(a: np.ndarray):
    return a.ctypes.data_as(_fp)


def _raw(raw: np.ndarray) -> np.ndarray:
    raw = np.ascontiguousarray(raw)
    if raw.dtype != np.uint8:
        raw = raw.view(np.uint8)
    return raw.reshape(-1)


def dequant(raw: np.ndarray, N: int, K: int, use_ref: bool = False) -> np.ndarray:
    """float32 [N, K] weights from N rows of K/256 raw 144-byte super-blocks."""
    raw = _raw(raw)
    assert raw.size >= N * (K // QK_K) * BLOCK_BYTES
    out = np.zeros((N, K), np.float32)
    if N and K:
        fn = ref_lib().ref_q4k_dequant if use_ref else lib().oracle_q4k_dequant
        fn(raw.ctypes.data, _f(out), N, K)
    return out


def matmul(x: np.ndarray, raw: np.ndarray, bias: np.ndarray | None, N: int, K: int,
           threads: int = 1, use_ref: bool = False) -> np.ndarray:
    """Y[M, N] = bias + X[M, K] . deq(W)[N, K]^T, float32, k ascending."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    raw = _raw(raw)
    y = np.zeros((M, N), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    bp = _f(b) if b is not None else None
    if M == 0 or N == 0:
        return y
    if use_ref:
        ref_lib().ref_q4k_matmul(_f(x), raw.ctypes.data, bp, _f(y), M, N, K, threads)
    elif threads > 1:
        lib().oracle_q4k_matmul_mt(_f(x), raw.ctypes.data, bp, _f(y), M, N, K, threads)
    else:
        lib().oracle_q4k_matmul(_f(x), raw.ctypes.data, bp, _f(y), M, N, K)
    return y


def matmul_f64(x: np.ndarray, raw: np.ndarray, bias: np.ndarray | None, N: int, K: int) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    raw = _raw(raw)
    y = np.zeros((M, N), np.float64)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().oracle_q4k_matmul_f64(_f(x), raw.ctypes.data, _f(b) if b is not None else None,
                                y.ctypes.data_as(C.POINTER(C.c_double)), M, N, K)
    return y


def matmul_moe(x: np.ndarray, raw: np.ndarray, bias: np.ndarray | None, N: int, K: int,
               offsets: np.ndarray, x_rows_per_slot: int = 1) -> np.ndarray:
    """Indirect expert form, one reference-style dispatch per slot.

    ``raw`` stacks every expert's [N, K] matrix row-wise; ``offsets[s]`` is the
    first weight row of slot s's expert.  Slot s multiplies activation rows
    ``x[s*x_rows_per_slot : (s+1)*x_rows_per_slot]`` and writes
    ``y[s]`` (shape [x_rows_per_slot, N]) -- i.e. yOffset = s*rows*N, the way a
    caller lays routed outputs side by side.
    """
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    offsets = np.ascontiguousarray(offsets, np.uint32)
    S = offsets.size
    R = x_rows_per_slot
    assert x.shape[0] == S * R
    raw = _raw(raw)
    y = np.zeros((S, R, N), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    op = offsets.ctypes.data_as(C.POINTER(_u32))
    for s in range(S):
        xs = np.ascontiguousarray(x[s * R:(s + 1) * R])
        lib().oracle_q4k_matmul_moe_slot(_f(xs), raw.ctypes.data, _f(b) if b is not None else None,
                                         _f(y), R, N, K, op, s, s * R * N)
    return y


def pack(raw: np.ndarray, N: int, K: int, use_ref: bool = False):
    """(words u32[N*rowStrideWords], rowStrideWords, nBlocks) as pack_q4k returns them."""
    raw = _raw(raw)
    rs, nb = _u32(0), _u32(0)
    fn = ref_lib().ref_pack_q4k if use_ref else lib().oracle_pack_q4k
    fn(raw.ctypes.data, N, K, None, C.byref(rs), C.byref(nb))
    words = np.zeros(N * rs.value, np.uint32)
    if words.size:
        fn(raw.ctypes.data, N, K, words.ctypes.data, C.byref(rs), C.byref(nb))
    return words, rs.value, nb.value


# --------------------------------------------------------------------------
# The K-quant family by type number (reference GGUFType: Q4_K 12, Q5_K 13, Q6_K 14)
# --------------------------------------------------------------------------

Q4_K, Q5_K, Q6_K = 12, 13, 14
KQ_BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210}


def kq_dequant(qtype: int, raw: np.ndarray, N: int, K: int, use_ref: bool = False) -> np.ndarray:
    """float32 [N, K] weights from N rows of K/256 raw super-blocks of the given type."""
    raw = _raw(raw)
    assert raw.size >= N * (K // QK_K) * KQ_BLOCK_BYTES[qtype]
    out = np.zeros((N, K), np.float32)
    if N and K:
        fn = ref_lib().ref_kq_dequant if use_ref else lib().oracle_kq_dequant
        fn(qtype, raw.ctypes.data, _f(out), N, K)
    return out


def kq_matmul(qtype: int, x: np.ndarray, raw: np.ndarray, bias: np.ndarray | None, N: int, K: int,
              threads: int = 1, use_ref: bool = False) -> np.ndarray:
    """Y[M, N] = bias + X[M, K] . deq(W)[N, K]^T, float32, k ascending, for any K-quant type."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    raw = _raw(raw)
    y = np.zeros((M, N), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    if M == 0 or N == 0:
        return y
    fn = ref_lib().ref_kq_matmul if use_ref else lib().oracle_kq_matmul
    fn(qtype, _f(x), raw.ctypes.data, _f(b) if b is not None else None, _f(y), M, N, K, threads)
    return y


def kq_pack(qtype: int, raw: np.ndarray, N: int, K: int, use_ref: bool = False):
    """(words u32[N*rowStrideWords], rowStrideWords, nBlocks) as pack_q4k/q5k/q6k return them."""
    raw = _raw(raw)
    rs, nb = _u32(0), _u32(0)
    fn = ref_lib().ref_kq_pack if use_ref else lib().oracle_kq_pack
    fn(qtype, raw.ctypes.data, N, K, None, C.byref(rs), C.byref(nb))
    words = np.zeros(N * rs.value, np.uint32)
    if words.size:
        fn(qtype, raw.ctypes.data, N, K, words.ctypes.data, C.byref(rs), C.byref(nb))
    return words, rs.value, nb.value


def prologue(kind: int, x: np.ndarray, aux: np.ndarray | None, eps: float = 0.0) -> np.ndarray:
    """The fused decode shaders' element-wise step on one activation row (1 RMSNorm, 2 gelu*up, 3 silu*up)."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    a = np.ascontiguousarray(aux if aux is not None else np.zeros_like(x), np.float32).reshape(-1)
    out = np.zeros_like(x)
    lib().oracle_prologue(kind, _f(x), _f(a), float(eps), x.size, _f(out))
    return out


def moe_ffn(qtype: int, x: np.ndarray, raw_gate: np.ndarray, raw_up: np.ndarray, raw_down: np.ndarray,
            expert_ids: np.ndarray, route_w: np.ndarray, y0: np.ndarray, F: int, H: int) -> np.ndarray:
    """The reference's routed-expert loop for T tokens (runtime/model_runner.cpp:3584-3651): per token and slot
    k ascending -- gate and up projections of expert e, silu(gate)*up, down projection, then
    y[t] = y[t] + w[t,k] * out in float32 (runtime/kernels/moe/weighted_accumulate_decode.wgsl)."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, H)
    T = x.shape[0]
    ids = np.ascontiguousarray(expert_ids).reshape(T, -1)
    w = np.ascontiguousarray(route_w, np.float32).reshape(T, -1)
    y = np.array(y0, np.float32).reshape(T, H).copy()
    bg, bd = KQ_BLOCK_BYTES[qtype] * (H // QK_K), KQ_BLOCK_BYTES[qtype] * (F // QK_K)   # bytes per weight row
    rg, ru, rd = _raw(raw_gate), _raw(raw_up), _raw(raw_down)
    for t in range(T):
        for k in range(ids.shape[1]):
            e = int(ids[t, k])
            g = kq_matmul(qtype, x[t], rg[e * F * bg:(e + 1) * F * bg], None, F, H).reshape(-1)
            u = kq_matmul(qtype, x[t], ru[e * F * bg:(e + 1) * F * bg], None, F, H).reshape(-1)
            act = prologue(3, g, u)
            o = kq_matmul(qtype, act, rd[e * H * bd:(e + 1) * H * bd], None, H, F).reshape(-1)
            y[t] = y[t] + w[t, k] * o
    return y


def kq_dequant_numpy(qtype: int, raw: np.ndarray, N: int, K: int) -> np.ndarray:
    """Independent vectorised restatement of the Q5_K / Q6_K branches of dequant_kquant
    (runtime/gguf_loader.cpp:497-573); Q4_K goes to dequant_numpy."""
    if qtype == Q4_K:
        return dequant_numpy(raw, N, K)
    nb = K // QK_K
    bb = KQ_BLOCK_BYTES[qtype]
    blk = _raw(raw)[: N * nb * bb].reshape(N * nb, bb)
    out = np.zeros((N, K), np.float32)
    if qtype == Q5_K:
        d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)
        dmin = blk[:, 2:4].copy().view(np.float16).astype(np.float32)
        p = blk[:, 4:16].astype(np.uint32)
        sc = np.empty((N * nb, 8), np.uint32)
        mn = np.empty((N * nb, 8), np.uint32)
        sc[:, :4] = p[:, 0:4] & 63
        mn[:, :4] = p[:, 4:8] & 63
        sc[:, 4:] = (p[:, 8:12] & 15) | ((p[:, 0:4] >> 2) & 0x30)
        mn[:, 4:] = (p[:, 8:12] >> 4) | ((p[:, 4:8] >> 2) & 0x30)
        qh = blk[:, 16:48].astype(np.uint32)                               # [B, 32]
        codes = blk[:, 48:].reshape(N * nb, 4, 32).astype(np.uint32)
        q = np.empty((N * nb, 8, 32), np.uint32)
        q[:, 0::2] = codes & 15
        q[:, 1::2] = codes >> 4
        for sb in range(8):
            q[:, sb] |= ((qh >> sb) & 1) << 4
        s = (d * sc.astype(np.float32)).astype(np.float32)
        m = (dmin * mn.astype(np.float32)).astype(np.float32)
        w = (s[:, :, None] * q.astype(np.float32)).astype(np.float32) - m[:, :, None]
        out[:, : nb * QK_K] = w.astype(np.float32).reshape(N, nb * QK_K)
        return out
    # Q6_K
    d = blk[:, 208:210].copy().view(np.float16).astype(np.float32)         # [B, 1]
    sc = blk[:, 192:208].copy().view(np.int8).astype(np.float32)           # [B, 16]
    ql = blk[:, 0:128].reshape(N * nb, 2, 2, 32).astype(np.int32)          # [B, half, byte group (l, l+32), l]
    qh = blk[:, 128:192].reshape(N * nb, 2, 32).astype(np.int32)           # [B, half, l]
    q = np.empty((N * nb, 2, 4, 32), np.int32)                             # [B, half, group of 32, l]
    q[:, :, 0] = (ql[:, :, 0] & 15) | (((qh >> 0) & 3) << 4)
    q[:, :, 1] = (ql[:, :, 1] & 15) | (((qh >> 2) & 3) << 4)
    q[:, :, 2] = (ql[:, :, 0] >> 4) | (((qh >> 4) & 3) << 4)
    q[:, :, 3] = (ql[:, :, 1] >> 4) | (((qh >> 6) & 3) << 4)
    q -= 32
    ds = (d * sc).astype(np.float32).reshape(N * nb, 2, 4, 2)              # scale index = half*8 + group*2 + l//16
    w = (np.repeat(ds, 16, axis=3) * q.astype(np.float32)).astype(np.float32)
    out[:, : nb * QK_K] = w.reshape(N, nb * QK_K)
    return out


# --------------------------------------------------------------------------
# Independent numpy restatement (cross-check of the C one)
# --------------------------------------------------------------------------

def dequant_numpy(raw: np.ndarray, N: int, K: int) -> np.ndarray:
    """Vectorised restatement of runtime/gguf_loader.cpp:455-496 (Q4_K branch)."""
    nb = K // QK_K
    blk = _raw(raw)[: N * nb * BLOCK_BYTES].reshape(N * nb, BLOCK_BYTES)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)        # exact widening
    dmin = blk[:, 2:4].copy().view(np.float16).astype(np.float32)
    p = blk[:, 4:16].astype(np.uint32)
    sc = np.empty((N * nb, 8), np.uint32)
    mn = np.empty((N * nb, 8), np.uint32)
    sc[:, :4] = p[:, 0:4] & 63
    mn[:, :4] = p[:, 4:8] & 63
    sc[:, 4:] = (p[:, 8:12] & 15) | ((p[:, 0:4] >> 2) & 0x30)
    mn[:, 4:] = (p[:, 8:12] >> 4) | ((p[:, 4:8] >> 2) & 0x30)
    codes = blk[:, 16:].reshape(N * nb, 4, 32)
    q = np.empty((N * nb, 8, 32), np.float32)
    q[:, 0::2] = (codes & 15).astype(np.float32)
    q[:, 1::2] = (codes >> 4).astype(np.float32)
    s = (d * sc.astype(np.float32)).astype(np.float32)                # d*sc rounded
    m = (dmin * mn.astype(np.float32)).astype(np.float32)             # dmin*mn rounded
    w = (s[:, :, None] * q).astype(np.float32) - m[:, :, None]        # product rounded, then difference
    out = np.zeros((N, K), np.float32)
    out[:, : nb * QK_K] = w.astype(np.float32).reshape(N, nb * QK_K)
    return out
