"""ctypes binding of libbpq4k.so (the C ABI declared in include/bpq4k.h).

There is no fallback: if the shared library is missing, or a symbol the header
declares is absent, importing fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "lib", "libbpq4k.so")

u32 = C.c_uint32
u64 = C.c_uint64
vp = C.c_void_p

# name -> (restype, argtypes); mirrors include/bpq4k.h one to one
SIGNATURES = {
    "bpq4k_version": (C.c_int, []),
    "bpq4k_status_string": (C.c_char_p, [C.c_int]),
    "bpq4k_create": (C.c_int, [C.c_int, C.POINTER(vp)]),
    "bpq4k_destroy": (C.c_int, [vp]),
    "bpq4k_last_error_string": (C.c_char_p, [vp]),
    "bpq4k_set_option": (C.c_int, [vp, C.c_int, C.c_int]),
    "bpq4k_get_option": (C.c_int, [vp, C.c_int, C.POINTER(C.c_int)]),
    "bpq4k_read_stream_stamps": (C.c_int, [vp, vp, C.c_size_t, C.POINTER(C.c_uint32)]),
    "bpq4k_launch_count": (u64, [vp, C.c_int]),
    "bpq4k_device_status": (C.c_int, [vp, vp, C.POINTER(C.c_int)]),
    "bpq4k_n_blocks": (u32, [u32]),
    "bpq4k_row_stride_words": (u32, [u32]),
    "bpq4k_pack_q4k_host": (C.c_int, [vp, u32, u32, vp]),
    "bpq4k_upload_weights": (C.c_int, [vp, vp, u64, C.POINTER(vp)]),
    "bpq4k_free_device": (C.c_int, [vp, vp]),
    "bpq4k_dequant_f32": (C.c_int, [vp, vp, u32, u32, u32, vp, vp]),
    "bpq4k_matmul_f32": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, vp]),
    "bpq4k_matmul_moe_f32": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, vp]),
    "bpq4k_matmul_host_f32": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32, u32, vp]),
}



class HostMatmul(C.Structure):
    """bpq4k_host_matmul of include/bpq4k.h."""
    _fields_ = [("X_host", vp), ("W_dev", vp), ("bias_dev", vp), ("Y_host", vp),
                ("M", u32), ("N", u32), ("K", u32), ("rowStrideWords", u32)]


SIGNATURES["bpq4k_matmul_noalloc_f32"] = (C.c_int, [vp, vp, vp, vp, u32, u32, u32, u32, u32, vp])
SIGNATURES["bpq4k_noalloc_last_error"] = (C.c_char_p, [])
SIGNATURES["bpq4k_matmul_allgather_f32"] = (C.c_int, [vp, vp, vp, vp, C.POINTER(vp), u32, u32, u32, u32, u32, vp])
SIGNATURES["bpq4k_peer_double_buffer"] = (C.c_int, [vp, vp, u64])
SIGNATURES["bpq4k_peer_barrier"] = (C.c_int, [vp, C.POINTER(vp), u32, u32, u32, u32, vp])
SIGNATURES["bpq4k_matmul_host_batch_f32"] = (C.c_int, [vp, C.POINTER(HostMatmul), u32, vp])

SIGNATURES["bpq4k_kq_block_bytes"] = (u32, [C.c_int])
SIGNATURES["bpq4k_kq_row_stride_words"] = (u32, [C.c_int, u32])
SIGNATURES["bpq4k_kq_pack_host"] = (C.c_int, [C.c_int, vp, u32, u32, vp])
SIGNATURES["bpq4k_kq_dequant_f32"] = (C.c_int, [vp, C.c_int, vp, u32, u32, u32, vp, vp])
SIGNATURES["bpq4k_kq_gather_f32"] = (C.c_int, [vp, C.c_int, vp, u32, u32, u32, vp, u32, vp, vp])
SIGNATURES["bpq4k_kq_matmul_f32"] = (C.c_int, [vp, C.c_int, vp, vp, vp, vp, u32, u32, u32, u32, u32, vp])
SIGNATURES["bpq4k_matmul_fused_f32"] = (C.c_int, [vp, C.c_int, C.c_int, vp, vp, C.c_float, vp, vp, vp, vp, u32, u32, u32, u32, vp])
i64 = C.c_int64
cp = C.c_char_p
SIGNATURES["bpq4k_device_index"] = (C.c_int, [vp])
SIGNATURES["bpq4k_gguf_open"] = (C.c_int, [cp, C.POINTER(vp)])
SIGNATURES["bpq4k_gguf_close"] = (C.c_int, [vp])
SIGNATURES["bpq4k_gguf_last_error"] = (cp, [vp])
SIGNATURES["bpq4k_gguf_version"] = (u32, [vp])
SIGNATURES["bpq4k_gguf_n_tensors"] = (u64, [vp])
SIGNATURES["bpq4k_gguf_data_offset"] = (u64, [vp])
SIGNATURES["bpq4k_gguf_has_key"] = (C.c_int, [vp, cp])
SIGNATURES["bpq4k_gguf_get_u32"] = (u32, [vp, cp, u32])
SIGNATURES["bpq4k_gguf_get_f32"] = (C.c_float, [vp, cp, C.c_float])
SIGNATURES["bpq4k_gguf_get_bool"] = (C.c_int, [vp, cp, C.c_int])
SIGNATURES["bpq4k_gguf_get_string"] = (i64, [vp, cp, i64, vp, u64])
SIGNATURES["bpq4k_gguf_array_length"] = (i64, [vp, cp])
SIGNATURES["bpq4k_gguf_get_i32_array"] = (C.c_int, [vp, cp, u64, u64, vp])
SIGNATURES["bpq4k_gguf_find_tensor"] = (C.c_int, [vp, cp, C.POINTER(u64)])
SIGNATURES["bpq4k_gguf_tensor_info"] = (C.c_int, [vp, u64, C.POINTER(cp), C.POINTER(u32), C.POINTER(u64 * 4), C.POINTER(u32),
                                                  C.POINTER(u64), C.POINTER(u64)])
SIGNATURES["bpq4k_gguf_read_tensor"] = (C.c_int, [vp, u64, u64, u64, vp])
SIGNATURES["bpq4k_gguf_upload_tensor"] = (C.c_int, [vp, vp, u64, C.c_int, C.POINTER(vp), C.POINTER(C.c_int), C.POINTER(u32),
                                                    C.POINTER(u32), C.POINTER(u32)])
SIGNATURES["bpq4k_argmax_f32"] = (C.c_int, [vp, vp, u32, vp, vp])
SIGNATURES["bpq4k_kq_matmul_allgather_f32"] = (C.c_int, [vp, C.c_int, vp, vp, vp, C.POINTER(vp), u32, u32, u32, u32, u32, vp])
SIGNATURES["bpq4k_kq_matmul_moe_f32"] = (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, vp])
SIGNATURES["bpq4k_moe_ffn_work_floats"] = (C.c_uint64, [u32, u32, u32, u32])
SIGNATURES["bpq4k_moe_ffn_f32"] = (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, vp, C.c_uint64, vp])
SIGNATURES["bpq4k_kq_respace_device"] = (C.c_int, [vp, C.c_int, vp, u32, u32, vp, vp])

_lib = None


class LibraryMissing(ImportError):
    pass


def build() -> None:
    """Compile the CUDA sources in csrc/ for sm_100a into lib/libbpq4k.so."""
    import subprocess

    subprocess.run(["make", "-s", "-C", os.path.join(PKG_DIR, "csrc")], check=True)


def _open(path: str) -> C.CDLL:
    if not os.path.isfile(path):
        raise LibraryMissing(
            f"{path} not found. Build it with `make -C {os.path.join(PKG_DIR, 'csrc')}` "
            "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback."
        )
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # stale build
            raise LibraryMissing(f"{path} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    return lib


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _open(LIB_PATH)
    return _lib


DEBUG_LIB_PATH = os.path.join(PKG_DIR, "lib", "libbpq4k_debug.so")
_debug_lib = None


def load_debug() -> C.CDLL:
    """The debug build (`make -C csrc DEBUG=1`): the same library with index checks compiled into the kernels; a failed
    check shows up as status 9 in bpq4k_device_status and the access is skipped."""
    global _debug_lib
    if _debug_lib is None:
        _debug_lib = _open(DEBUG_LIB_PATH)
    return _debug_lib


STAMPS_LIB_PATH = os.path.join(PKG_DIR, "lib", "libbpq4k_stamps.so")
_stamps_lib = None


def load_stamps() -> C.CDLL:
    """The build with in-kernel time stamps (`make -C csrc stamps`): the product library with the streaming kernel
    compiled again with BPQ4K_OPT_STREAM_STAMPS support."""
    global _stamps_lib
    if _stamps_lib is None:
        _stamps_lib = _open(STAMPS_LIB_PATH)
    return _stamps_lib


class ModelConfig(C.Structure):
    """bpq4k_model_config of include/bpq4k.h (the reference's ModelConfig, runtime/gguf_loader.h:164-224)."""
    _fields_ = [("arch", C.c_char * 64)] + [(n, u32) for n in ("nLayer", "nHead", "nKvHeads", "nEmbd", "intermediateSize", "nVocab",
                                                                 "headDim", "kvHeadDim")] + \
               [("rmsNormEps", C.c_float), ("ropeTheta", C.c_float), ("tieWordEmbeddings", C.c_int32), ("hasQkNorm", C.c_int32),
                ("activation", C.c_int32), ("embeddingScale", C.c_float), ("logitSoftcap", C.c_float),
                ("slidingWindow", u32), ("nLayerAttnTypes", u32), ("hasSandwichNorm", C.c_int32), ("pleSize", u32),
                ("sharedKvLayers", u32), ("hasMtp", C.c_int32), ("mtpNumLayers", u32)] + \
               [(n, u32) for n in ("numExperts", "numExpertsPerTok", "moeIntermediateSize", "moeSharedIntermediateSize",
                                   "ssmInnerSize", "ssmStateSize", "ssmConvKernel", "ssmGroupCount", "ssmTimeStepRank",
                                   "fullAttentionInterval")] + [("ropeSections", C.c_int32 * 4)]


class KQTensor(C.Structure):
    """bpq4k_kq_tensor of include/bpq4k.h."""
    _fields_ = [("w", vp), ("qtype", C.c_int32), ("N", u32), ("K", u32), ("rowStrideWords", u32), ("n_fused", u32)]


class LayerWeights(C.Structure):
    """bpq4k_layer_weights of include/bpq4k.h."""
    _fields_ = [(n, KQTensor) for n in ("qkv", "q", "k", "v", "o", "gate_up", "gate", "up", "down")] + [("qkv_prefused", C.c_int32)]


SIGNATURES["bpq4k_gguf_upload_fused"] = (C.c_int, [vp, vp, C.POINTER(u64), u32, C.c_int, C.POINTER(vp), C.POINTER(C.c_int),
                                                   C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)])
SIGNATURES["bpq4k_gguf_model_config"] = (C.c_int, [vp, C.POINTER(ModelConfig), vp, u32])
SIGNATURES["bpq4k_gguf_weight_format"] = (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)])
SIGNATURES["bpq4k_gguf_load_layer"] = (C.c_int, [vp, vp, u32, C.c_int, C.POINTER(LayerWeights)])
SIGNATURES["bpq4k_free_layer"] = (C.c_int, [vp, C.POINTER(LayerWeights)])
