"""GGUF files: metadata, tensor directory and the tensor -> device step, on top of the C ABI.

Mirrors the reference's ``GGUFFile`` (runtime/gguf_loader.h:46-91): ``open``, ``getString`` /
``getU32`` / ``getFloat`` / ``getBool`` / ``hasKey``, ``tensors`` with name, shape, type and offset,
``data_offset``.  Parsing needs no GPU.  ``upload`` is the K-quant half of the reference's weight
loading (pack_q*k + uploadKQWeight): file bytes straight into device memory.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from .q4k import Q4KContext, Q4KError


@dataclass
class GGUFTensorInfo:
    name: str
    shape: tuple          # shape[0] is the contiguous dimension (K of a weight matrix)
    type: int             # GGML type number (12 Q4_K, 13 Q5_K, 14 Q6_K, 0 F32, ...)
    offset: int           # from the start of the tensor data
    n_bytes: int          # 0 for a type the reader cannot size


class DeviceTensor:
    """A K-quant tensor resident on the device (owned by the library; freed on close/del)."""

    def __init__(self, ctx: Q4KContext, ptr: int, qtype: int, N: int, K: int, rowStrideWords: int):
        self._ctx, self.ptr, self.qtype, self.N, self.K, self.rowStrideWords = ctx, ptr, qtype, N, K, rowStrideWords

    @property
    def nbytes(self) -> int:
        return self.N * self.rowStrideWords * 4

    def as_weight(self):
        """A Q4KWeight view (torch uint8 tensor over the same memory) for Q4KContext.matmul and friends."""
        import torch

        from .q4k import Q4KWeight

        n = max(self.nbytes, 16)
        arr = (C.c_uint8 * n).from_address(self.ptr)  # address only; never dereferenced on the host

        class _Holder:  # __cuda_array_interface__ carrier that keeps this DeviceTensor alive
            def __init__(h, owner):
                h.owner = owner
                h.__cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (owner.ptr, False), "version": 2}

        del arr
        buf = torch.as_tensor(_Holder(self), device=f"cuda:{self._ctx.device}")
        return Q4KWeight(buf, self.N, self.K, self.rowStrideWords, self.qtype)

    def free(self) -> None:
        if self.ptr:
            self._ctx.lib.bpq4k_free_device(self._ctx.h, self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GGUFFile:
    def __init__(self, path: str):
        self.lib = _lib.load()
        h = C.c_void_p()
        st = self.lib.bpq4k_gguf_open(str(path).encode(), C.byref(h))
        if st:
            raise Q4KError(st, f"cannot open {path} as a GGUF file")
        self.h = h
        self.version = int(self.lib.bpq4k_gguf_version(h))
        self.n_tensors = int(self.lib.bpq4k_gguf_n_tensors(h))
        self.data_offset = int(self.lib.bpq4k_gguf_data_offset(h))
        self.tensors = [self._info(i) for i in range(self.n_tensors)]
        self.tensor_index = {t.name: i for i, t in enumerate(self.tensors)}

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.bpq4k_gguf_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _info(self, i: int) -> GGUFTensorInfo:
        name, nd, shape, typ, off, nb = C.c_char_p(), C.c_uint32(), (C.c_uint64 * 4)(), C.c_uint32(), C.c_uint64(), C.c_uint64()
        st = self.lib.bpq4k_gguf_tensor_info(self.h, i, C.byref(name), C.byref(nd), C.byref(shape), C.byref(typ), C.byref(off),
                                             C.byref(nb))
        if st:
            raise Q4KError(st, f"tensor {i}")
        return GGUFTensorInfo(name.value.decode(), tuple(int(shape[d]) for d in range(nd.value)), int(typ.value),
                              int(off.value), int(nb.value))

    # -- metadata (names follow the reference) -------------------------------
    def hasKey(self, key: str) -> bool:
        return bool(self.lib.bpq4k_gguf_has_key(self.h, key.encode()))

    def getU32(self, key: str, default: int = 0) -> int:
        return int(self.lib.bpq4k_gguf_get_u32(self.h, key.encode(), default))

    def getFloat(self, key: str, default: float = 0.0) -> float:
        return float(self.lib.bpq4k_gguf_get_f32(self.h, key.encode(), default))

    def getBool(self, key: str, default: bool = False) -> bool:
        return bool(self.lib.bpq4k_gguf_get_bool(self.h, key.encode(), 1 if default else 0))

    def _string(self, key: str, index: int):
        n = self.lib.bpq4k_gguf_get_string(self.h, key.encode(), index, None, 0)
        if n < 0:
            return None
        buf = C.create_string_buffer(n + 1)
        self.lib.bpq4k_gguf_get_string(self.h, key.encode(), index, buf, n + 1)
        return buf.raw[:n].decode("utf-8", "replace")

    def getString(self, key: str, default: str = "") -> str:
        s = self._string(key, -1)
        return default if s is None else s

    def getStringArray(self, key: str):
        n = self.lib.bpq4k_gguf_array_length(self.h, key.encode())
        if n < 0 or (n > 0 and self._string(key, 0) is None):
            return None
        return [self._string(key, i) for i in range(n)]

    def getI32Array(self, key: str):
        n = self.lib.bpq4k_gguf_array_length(self.h, key.encode())
        if n < 0:
            return None
        out = np.zeros(n, np.int32)
        if self.lib.bpq4k_gguf_get_i32_array(self.h, key.encode(), 0, n, out.ctypes.data):
            return None
        return out

    # -- tensor data ----------------------------------------------------------
    def read(self, name: str) -> np.ndarray:
        """Raw bytes of a tensor (host)."""
        i = self.tensor_index[name]
        t = self.tensors[i]
        out = np.zeros(t.n_bytes, np.uint8)
        st = self.lib.bpq4k_gguf_read_tensor(self.h, i, 0, t.n_bytes, out.ctypes.data)
        if st:
            raise Q4KError(st, self.lib.bpq4k_gguf_last_error(self.h).decode())
        return out

    def upload(self, ctx: Q4KContext, name: str, layout: int = 0) -> DeviceTensor:
        """File -> device for a Q4_K / Q5_K / Q6_K tensor (layout: 0 = packed layout of its type,
        Q6_K_PADDED for the fast Q6_K kernel)."""
        i = self.tensor_index[name]
        ptr, qt, N, K, rs = C.c_void_p(), C.c_int(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        st = self.lib.bpq4k_gguf_upload_tensor(ctx.h, self.h, i, layout, C.byref(ptr), C.byref(qt), C.byref(N), C.byref(K),
                                               C.byref(rs))
        if st:
            raise Q4KError(st, self.lib.bpq4k_gguf_last_error(self.h).decode())
        return DeviceTensor(ctx, ptr.value, qt.value, N.value, K.value, rs.value)

    def upload_fused(self, ctx: Q4KContext, names, layout: int = 0) -> DeviceTensor:
        """Several tensors of one K-quant type and one K, concatenated by rows into one device tensor
        (the reference's fuseKQ + uploadKQWeight, runtime/model_runner.cpp:1002-1012)."""
        idx = (C.c_uint64 * len(names))(*[self.tensor_index[n] for n in names])
        ptr, qt, N, K, rs = C.c_void_p(), C.c_int(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        st = self.lib.bpq4k_gguf_upload_fused(ctx.h, self.h, idx, len(names), layout, C.byref(ptr), C.byref(qt), C.byref(N),
                                              C.byref(K), C.byref(rs))
        if st:
            raise Q4KError(st, self.lib.bpq4k_gguf_last_error(self.h).decode())
        return DeviceTensor(ctx, ptr.value, qt.value, N.value, K.value, rs.value)

    # -- model level (extractModelConfig and the loader's per-layer rules) -----------------
    def model_config(self) -> dict:
        """The reference's ModelConfig (extractModelConfig, runtime/gguf_loader.cpp:184-317) as a dict; the
        per-layer attention types (0 global, 1 sliding window) under 'layerAttnTypes'."""
        cfg = _lib.ModelConfig()
        types = (C.c_uint8 * 4096)()
        st = self.lib.bpq4k_gguf_model_config(self.h, C.byref(cfg), types, 4096)
        if st:
            raise Q4KError(st, "model_config")
        out = {}
        for name, _ in _lib.ModelConfig._fields_:
            v = getattr(cfg, name)
            out[name] = v.decode() if name == "arch" else list(v) if name == "ropeSections" else v
        out["layerAttnTypes"] = [int(types[i]) for i in range(min(cfg.nLayerAttnTypes, 4096))]
        return out

    def weight_format(self):
        """(GGML type of the first primary weight tensor, whether layer 0's attn_q / ffn_gate / ffn_down all carry
        that one K-quant type): the loader's probe at runtime/model_runner.cpp:1014-1049."""
        qt, uni = C.c_int(), C.c_int()
        st = self.lib.bpq4k_gguf_weight_format(self.h, C.byref(qt), C.byref(uni))
        if st:
            raise Q4KError(st, "weight_format")
        return qt.value, bool(uni.value)

    def load_layer(self, ctx: Q4KContext, layer: int, q6_layout: int = 0) -> dict:
        """One layer's projection weights on the device with the loader's fusion rules
        (runtime/model_runner.cpp:1223-1370).  Returns {'qkv' | 'q','k','v', 'o', 'gate_up' | 'gate','up', 'down':
        DeviceTensor} for the K-quant tensors that exist, plus 'qkv_prefused' and 'n_fused' per entry."""
        lw = _lib.LayerWeights()
        st = self.lib.bpq4k_gguf_load_layer(ctx.h, self.h, layer, q6_layout, C.byref(lw))
        if st:
            raise Q4KError(st, self.lib.bpq4k_gguf_last_error(self.h).decode())
        out = {"qkv_prefused": bool(lw.qkv_prefused), "n_fused": {}, "file_types": {}}
        for name, _ in _lib.LayerWeights._fields_[:-1]:
            t = getattr(lw, name)
            out["file_types"][name] = int(t.qtype)
            if t.w:
                out[name] = DeviceTensor(ctx, t.w, t.qtype, t.N, t.K, t.rowStrideWords)
                out["n_fused"][name] = int(t.n_fused)
        return out
