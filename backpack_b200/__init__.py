"""backpack_b200: the GGUF Q4_K dequantize-fused matmul of the Backpack runtime,
rebuilt for NVIDIA B200 (sm_100a) behind a C ABI (include/bpq4k.h)."""
from .q4k import (  # noqa: F401
    BLOCK_BYTES, BLOCK_WORDS, QK_K, Q4_K, Q5_K, Q6_K, Q6_K_PADDED, KQuantPacked, Q4KContext, Q4KError, Q4KWeight, fuse_kq,
    pack_kq, pack_q4k, pack_q5k, pack_q6k,
)

__all__ = ["BLOCK_BYTES", "BLOCK_WORDS", "QK_K", "Q4_K", "Q5_K", "Q6_K", "Q6_K_PADDED", "KQuantPacked", "Q4KContext", "Q4KError",
           "Q4KWeight", "fuse_kq", "pack_kq", "pack_q4k", "pack_q5k", "pack_q6k"]
