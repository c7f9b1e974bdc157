"""Host-side mirror of the reference's Q4_K operator interface, on top of the C ABI.

Names follow the reference: ``KQuantPacked`` / ``pack_q4k``
(runtime/gguf_loader.h:108-117, gguf_loader.cpp:359-379), ``upload`` for
``uploadKQWeight`` (runtime/model_runner.cpp:958-963), ``matmul`` for the
``q4k_matmul*`` dispatches with their five bindings X, W, Bias, Y, params
(runtime/kernels/quant_kq/q4k_matmul.wgsl:1-5), ``matmul_moe`` for the indirect
expert form (runtime/kernels/quant_kq/iq4xs_matmul_moe.wgsl:5-10) and
``dequant`` for ``dequant_kquant`` (gguf_loader.cpp:455-496).

PyTorch is used only to own device memory and streams; all arithmetic happens
in libbpq4k.so.  Nothing here computes on the CPU and nothing falls back.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib

QK_K = 256
BLOCK_BYTES = 144
BLOCK_WORDS = 36
# the reference's GGUFType numbers (runtime/gguf_loader.h:27-30)
Q4_K, Q5_K, Q6_K = 12, 13, 14
# Q6_K with every block padded to 224 bytes: the layout of the fast single-row Q6_K kernel (no reference counterpart)
Q6_K_PADDED = 0x10E

OPT_GEMV_VARIANT = 1
OPT_PREFILL_MODE = 2
OPT_PREFILL_MIN_M = 3
OPT_STREAM_WARPS, OPT_STREAM_KSPLIT, OPT_STREAM_STAGE_BLOCKS = 10, 11, 12
OPT_STREAM_STAGES, OPT_STREAM_CTAS_PER_SM, OPT_STREAM_FORCE_SCRATCH = 13, 14, 15
OPT_STREAM_NO_PDL = 16
OPT_STREAM_NO_UNIT_LIST = 17
OPT_STREAM_PREWAIT_STAGES = 18
OPT_STREAM_CLUSTER = 20
OPT_STREAM_STAGING_WARPS = 21
OPT_PREFILL_VARIANT = 23
OPT_STREAM_STAMPS = 24
PREFILL_ONE_CTA, PREFILL_CTA_PAIR, PREFILL_TMEM_WEIGHTS = 0, 1, 2
OPT_STREAM_UNIT_ROWS = 19
OPT_BATCH_RECORDS = 30   # read-only: replay graphs recorded by matmul_host_batch
GEMV_AUTO, GEMV_FP32, GEMV_STREAM = 0, 1, 2
PROLOGUE_NONE, PROLOGUE_RMSNORM, PROLOGUE_GELU_MUL, PROLOGUE_SILU_MUL = 0, 1, 2, 3
PREFILL_F16X3, PREFILL_F16, PREFILL_BF16 = 0, 1, 2


class Q4KError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"bpq4k status {status} ({_lib.load().bpq4k_status_string(status).decode()}): {message}")
        self.status = status


@dataclass
class KQuantPacked:
    """pack_q4k's result: raw block words plus the derived strides."""
    data: np.ndarray          # uint32 [N * rowStrideWords]
    N: int
    K: int
    rowStrideWords: int
    nBlocks: int
    qtype: int = Q4_K


def pack_kq(qtype: int, raw, N: int, K: int) -> KQuantPacked:
    """pack_q4k / pack_q5k / pack_q6k (runtime/gguf_loader.cpp:359-424): rows of raw blocks copied
    into u32 words; Q6_K rows (210-byte blocks) are padded with zeros to a whole word."""
    lib = _lib.load()
    bb = lib.bpq4k_kq_block_bytes(qtype)
    if not bb:
        raise ValueError(f"unknown K-quant type {qtype}")
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    nb = lib.bpq4k_n_blocks(K)
    rs = lib.bpq4k_kq_row_stride_words(qtype, K)
    file_bb = 210 if qtype == Q6_K_PADDED else bb   # the input is always the file format
    if raw.size < N * nb * file_bb:
        raise ValueError(f"raw has {raw.size} bytes, need {N * nb * file_bb}")
    words = np.zeros(N * rs, np.uint32)
    st = lib.bpq4k_kq_pack_host(qtype, raw.ctypes.data, N, K, words.ctypes.data)
    if st:
        raise Q4KError(st, "pack_kq")
    return KQuantPacked(words, N, K, rs, nb, qtype)


def pack_q5k(raw, N: int, K: int) -> KQuantPacked:
    return pack_kq(Q5_K, raw, N, K)


def pack_q6k(raw, N: int, K: int) -> KQuantPacked:
    return pack_kq(Q6_K, raw, N, K)


def pack_q4k(raw, N: int, K: int) -> KQuantPacked:
    """Row-wise copy of raw 144-byte blocks into u32 words (identity re-layout)."""
    lib = _lib.load()
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    nb = lib.bpq4k_n_blocks(K)
    rs = lib.bpq4k_row_stride_words(K)
    if raw.size < N * nb * BLOCK_BYTES:
        raise ValueError(f"raw has {raw.size} bytes, need {N * nb * BLOCK_BYTES}")
    words = np.zeros(N * rs, np.uint32)
    st = lib.bpq4k_pack_q4k_host(raw.ctypes.data, N, K, words.ctypes.data)
    if st:
        raise Q4KError(st, "pack_q4k")
    return KQuantPacked(words, N, K, rs, nb)


def fuse_kq(a: KQuantPacked, b: KQuantPacked) -> KQuantPacked:
    """Vertical fusion of two packed tensors (rows of `b` after rows of `a`), as the reference's
    loader fuses Q+K+V and gate+up so that one dispatch covers them
    (`fuseKQ`, runtime/model_runner.cpp:1002-1012)."""
    if a.K != b.K or a.rowStrideWords != b.rowStrideWords or a.qtype != b.qtype:
        raise ValueError("fuse_kq needs equal K, row stride and type")
    return KQuantPacked(np.concatenate([a.data, b.data]), a.N + b.N, a.K, a.rowStrideWords, a.nBlocks, a.qtype)


@dataclass
class Q4KWeight:
    """A packed weight resident on the device (a torch uint8 tensor owns the bytes)."""
    buf: "torch.Tensor"       # uint8 [N * rowStrideWords * 4]
    N: int
    K: int
    rowStrideWords: int
    qtype: int = Q4_K

    @property
    def nbytes(self) -> int:
        return self.N * self.rowStrideWords * 4

    def rows(self, n0: int, n1: int) -> "Q4KWeight":
        """A contiguous row range [n0, n1) as a view: rows are contiguous byte ranges."""
        rb = self.rowStrideWords * 4
        return Q4KWeight(self.buf[n0 * rb:n1 * rb], n1 - n0, self.K, self.rowStrideWords, self.qtype)


class Q4KContext:
    """One handle on one device; not thread-safe (like the reference's GPUContext)."""

    def __init__(self, device: int = 0, debug: bool = False, stamps: bool = False):
        import torch

        self._torch = torch
        self.lib = _lib.load_debug() if debug else _lib.load_stamps() if stamps else _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this library has no CPU path")
        self.device = int(device)
        h = C.c_void_p()
        st = self.lib.bpq4k_create(self.device, C.byref(h))
        if st:
            raise Q4KError(st, "bpq4k_create")
        self.h = h

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.bpq4k_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers ---------------------------------------------------------
    def _check(self, st: int) -> None:
        if st:
            raise Q4KError(st, self.lib.bpq4k_last_error_string(self.h).decode())

    def _stream(self) -> int:
        return self._torch.cuda.current_stream(self.device).cuda_stream

    def set_option(self, option: int, value: int) -> None:
        self._check(self.lib.bpq4k_set_option(self.h, option, value))

    def get_option(self, option: int) -> int:
        v = C.c_int()
        self._check(self.lib.bpq4k_get_option(self.h, option, C.byref(v)))
        return v.value

    def stream_stamps(self, slots: int):
        """Time stamps of the single-row streaming kernel (BPQ4K_OPT_STREAM_STAMPS must be on): a uint64 array
        [slots, 160, 8] of GPU-timer nanoseconds and the number of launches stamped so far."""
        import numpy as np

        buf = np.zeros((slots, 160, 8), np.uint64)
        n = C.c_uint32()
        self._check(self.lib.bpq4k_read_stream_stamps(self.h, buf.ctypes.data, buf.size, C.byref(n)))
        return buf, n.value

    def device_status(self) -> int:
        """Status word set by kernels whose bounded waits ran out (0 = none); synchronises."""
        v = C.c_int()
        self._check(self.lib.bpq4k_device_status(self.h, self._stream(), C.byref(v)))
        return v.value

    def launch_count(self, reset: bool = False) -> int:
        return int(self.lib.bpq4k_launch_count(self.h, 1 if reset else 0))

    # -- weights ---------------------------------------------------------
    def upload(self, packed: KQuantPacked) -> Q4KWeight:
        """uploadKQWeight: device buffer + copy of the packed words."""
        torch = self._torch
        host = torch.from_numpy(packed.data.view(np.uint8))
        buf = torch.empty(max(host.numel(), 16), dtype=torch.uint8, device=f"cuda:{self.device}")
        buf[: host.numel()].copy_(host)
        return Q4KWeight(buf, packed.N, packed.K, packed.rowStrideWords, packed.qtype)

    def respace_q6k(self, raw_dev, N: int, K: int, layout: int = Q6_K_PADDED) -> Q4KWeight:
        """File-format Q6_K blocks already on the device (uint8, N*K/256*210 bytes) -> a weight in `layout`."""
        torch = self._torch
        if raw_dev.dtype != torch.uint8 or not raw_dev.is_contiguous() or raw_dev.numel() < N * (K // 256) * 210:
            raise ValueError("raw_dev: contiguous uint8 tensor of N*K/256*210 bytes")
        rs = self.lib.bpq4k_kq_row_stride_words(layout, K)
        buf = torch.empty(max(N * rs * 4, 16), dtype=torch.uint8, device=raw_dev.device)
        self._check(self.lib.bpq4k_kq_respace_device(self.h, layout, raw_dev.data_ptr(), N, K, buf.data_ptr(), self._stream()))
        return Q4KWeight(buf, N, K, rs, layout)

    # -- operators -------------------------------------------------------
    def dequant(self, w: Q4KWeight, out=None):
        torch = self._torch
        if out is None:
            out = torch.empty((w.N, w.K), dtype=torch.float32, device=w.buf.device)
        if w.qtype == Q4_K:
            self._check(self.lib.bpq4k_dequant_f32(self.h, w.buf.data_ptr(), w.N, w.K, w.rowStrideWords,
                                                   out.data_ptr(), self._stream()))
        else:
            self._check(self.lib.bpq4k_kq_dequant_f32(self.h, w.qtype, w.buf.data_ptr(), w.N, w.K, w.rowStrideWords,
                                                      out.data_ptr(), self._stream()))
        return out

    def gather(self, w: Q4KWeight, tokens, out=None):
        """Embedding lookup (q6k_gather / q6k_gather_batched): out[t] = deq(W)[tokens[t]]; tokens int32/uint32 on the device."""
        torch = self._torch
        assert tokens.is_cuda and tokens.dtype in (torch.int32, torch.uint32) and tokens.is_contiguous()
        T = tokens.numel()
        if out is None:
            out = torch.empty((T, w.K), dtype=torch.float32, device=w.buf.device)
        self._check(self.lib.bpq4k_kq_gather_f32(self.h, w.qtype, w.buf.data_ptr(), w.N, w.K, w.rowStrideWords,
                                                 tokens.data_ptr(), T, out.data_ptr(), self._stream()))
        return out

    def matmul(self, x, w: Q4KWeight, bias=None, out=None, y_offset: int = 0):
        """Y[yOffset + m*N + n] = sum_k X[m,k] * deq(W)[n,k] + bias[n]; X float32 [..., K]."""
        torch = self._torch
        assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous()
        K = x.shape[-1]
        if K != w.K:
            raise ValueError(f"X has K={K}, weight has K={w.K}")
        M = x.numel() // K if K else 0
        if out is None:
            out = torch.empty(tuple(x.shape[:-1]) + (w.N,), dtype=torch.float32, device=x.device)
        if w.qtype == Q4_K:
            self._check(self.lib.bpq4k_matmul_f32(
                self.h, x.data_ptr(), w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
                out.data_ptr(), M, w.N, K, w.rowStrideWords, y_offset, self._stream()))
        else:
            self._check(self.lib.bpq4k_kq_matmul_f32(
                self.h, w.qtype, x.data_ptr(), w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
                out.data_ptr(), M, w.N, K, w.rowStrideWords, y_offset, self._stream()))
        return out

    def matmul_fused(self, x, w: Q4KWeight, prologue: int = PROLOGUE_NONE, aux=None, eps: float = 0.0, bias=None,
                     residual=None, out=None, y_offset: int = 0):
        """Single-row matmul with a fused prologue on x (RMSNorm with weight `aux`, or gelu/silu(x) * aux)
        and an optional residual added to the output (bpq4k_matmul_fused_f32)."""
        torch = self._torch
        assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous() and x.numel() == w.K
        if out is None:
            out = torch.empty((1, w.N), dtype=torch.float32, device=x.device)
        self._check(self.lib.bpq4k_matmul_fused_f32(
            self.h, w.qtype, prologue, x.data_ptr(), aux.data_ptr() if aux is not None else None, float(eps),
            w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
            residual.data_ptr() if residual is not None else None, out.data_ptr(), w.N, w.K, w.rowStrideWords,
            y_offset, self._stream()))
        return out

    def argmax(self, logits, out=None):
        """Index of the largest logit (int32 device tensor of one element); see bpq4k_argmax_f32."""
        torch = self._torch
        assert logits.dtype == torch.float32 and logits.is_cuda and logits.is_contiguous()
        if out is None:
            out = torch.empty(1, dtype=torch.int32, device=logits.device)
        self._check(self.lib.bpq4k_argmax_f32(self.h, logits.data_ptr(), logits.numel(), out.data_ptr(), self._stream()))
        return out

    def matmul_moe(self, x, w: Q4KWeight, n_rows_per_expert: int, offsets, x_rows=None, bias=None, out=None):
        """Indirect form: slot s uses weight rows offsets[s] .. offsets[s]+N of the expert stack."""
        torch = self._torch
        assert x.dtype == torch.float32 and x.is_contiguous()
        assert offsets.dtype == torch.int32 or offsets.dtype == torch.uint32
        S = offsets.numel()
        N = n_rows_per_expert
        if out is None:
            out = torch.empty((S, N), dtype=torch.float32, device=x.device)
        self._check(self.lib.bpq4k_kq_matmul_moe_f32(
            self.h, w.qtype, x.data_ptr(), w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
            out.data_ptr(), offsets.data_ptr(), x_rows.data_ptr() if x_rows is not None else None,
            S, N, w.K, w.rowStrideWords, w.N, self._stream()))
        return out

    def moe_ffn(self, x, w_gate: Q4KWeight, w_up: Q4KWeight, w_down: Q4KWeight, expert_ids, route_w, y, n_experts: int,
                work=None):
        """One routed-expert feed-forward step: y[t] += sum_k route_w[t,k] * down_e(silu(gate_e(x[t])) * up_e(x[t])),
        e = expert_ids[t,k]; the stacks hold n_experts matrices ([F,H] gate/up, [H,F] down).  y is updated in place."""
        torch = self._torch
        T, H = x.shape
        topk = expert_ids.numel() // T
        F = w_gate.N // n_experts
        assert x.dtype == torch.float32 and x.is_contiguous() and y.dtype == torch.float32 and y.is_contiguous()
        assert y.shape == x.shape and route_w.dtype == torch.float32 and route_w.numel() == T * topk
        assert expert_ids.dtype in (torch.int32, torch.uint32) and expert_ids.is_contiguous() and route_w.is_contiguous()
        assert w_gate.qtype == w_up.qtype == w_down.qtype and w_gate.K == w_up.K == H and w_down.K == F
        assert w_up.N == n_experts * F and w_down.N == n_experts * H
        need = self.lib.bpq4k_moe_ffn_work_floats(T, topk, H, F)
        if work is None:
            work = torch.empty(max(need, 4), dtype=torch.float32, device=x.device)
        self._check(self.lib.bpq4k_moe_ffn_f32(
            self.h, w_gate.qtype, x.data_ptr(), w_gate.buf.data_ptr(), w_up.buf.data_ptr(), w_down.buf.data_ptr(),
            expert_ids.data_ptr(), route_w.data_ptr(), y.data_ptr(), T, topk, n_experts, H, F, work.data_ptr(),
            work.numel(), self._stream()))
        return y

    def matmul_host(self, x_host: np.ndarray, w: Q4KWeight, y_host: np.ndarray, bias=None) -> np.ndarray:
        """Host activations in, host outputs out; copies and the wait are inside the call."""
        assert x_host.dtype == np.float32 and y_host.dtype == np.float32
        assert x_host.flags.c_contiguous and y_host.flags.c_contiguous
        M = x_host.size // w.K
        self._check(self.lib.bpq4k_matmul_host_f32(
            self.h, x_host.ctypes.data, w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
            y_host.ctypes.data, M, w.N, w.K, w.rowStrideWords, self._stream()))
        return y_host

    def make_host_batch(self, items):
        """Pre-build the dispatch list for matmul_host_batch: items = [(x_host, weight, y_host, bias|None)]."""
        arr = (_lib.HostMatmul * len(items))()
        for i, (x, w, y, bias) in enumerate(items):
            assert x.dtype == np.float32 and y.dtype == np.float32 and x.flags.c_contiguous and y.flags.c_contiguous
            arr[i] = _lib.HostMatmul(x.ctypes.data, w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
                                     y.ctypes.data, x.size // w.K, w.N, w.K, w.rowStrideWords)
        return arr, list(items)   # keep the arrays alive alongside the descriptors

    def matmul_host_batch(self, batch) -> None:
        """One call: upload every X, run every matmul, read every Y back, wait once."""
        arr, _keep = batch
        self._check(self.lib.bpq4k_matmul_host_batch_f32(self.h, arr, len(arr), self._stream()))

    # -- several GPUs (one process per GPU) ---------------------------------
    def matmul_allgather(self, x, w: Q4KWeight, slot_ptrs, bias=None) -> None:
        """Local product of this rank's row shard, stored straight into every rank's gather buffer.
        slot_ptrs: ctypes array of device addresses, own slot first (see bpq4k_matmul_allgather_f32)."""
        K = x.shape[-1]
        M = x.numel() // K
        if w.qtype == Q4_K:
            self._check(self.lib.bpq4k_matmul_allgather_f32(
                self.h, x.data_ptr(), w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
                slot_ptrs, len(slot_ptrs), M, w.N, K, w.rowStrideWords, self._stream()))
        else:
            self._check(self.lib.bpq4k_kq_matmul_allgather_f32(
                self.h, w.qtype, x.data_ptr(), w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
                slot_ptrs, len(slot_ptrs), M, w.N, K, w.rowStrideWords, self._stream()))

    def peer_double_buffer(self, step_word_ptr: int, stride_floats: int) -> None:
        """Fused all-gather calls that follow store to the half (step & 1) of double-buffered slots (0: off)."""
        self._check(self.lib.bpq4k_peer_double_buffer(self.h, step_word_ptr or None, stride_floats))

    def peer_barrier(self, flag_ptrs, rank: int, epoch: int, timeout_ms: int = 1000) -> None:
        """Bounded cross-GPU barrier on this stream (bpq4k_peer_barrier)."""
        self._check(self.lib.bpq4k_peer_barrier(self.h, flag_ptrs, len(flag_ptrs), rank, epoch, timeout_ms,
                                                self._stream()))
