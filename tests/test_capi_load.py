"""CPU-only checks of the boundary: the shared library loads, exports every symbol the
header declares, and the entry points that need no device behave."""
import ctypes as C
import os
import re

import numpy as np

from backpack_b200 import _lib, pack_q4k, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "bpq4k.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bpq4k_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = header_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/bpq4k.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table out of sync with the header"


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.bpq4k_version() == 100
    assert lib.bpq4k_status_string(0) == b"ok"
    assert b"256" in lib.bpq4k_status_string(2) or lib.bpq4k_status_string(2) == b"unsupported shape"
    assert lib.bpq4k_status_string(99) == b"unknown status"


def test_null_handle_is_rejected_not_crashing():
    lib = _lib.load()
    assert lib.bpq4k_destroy(None) == 1
    assert lib.bpq4k_set_option(None, 1, 0) == 1
    assert lib.bpq4k_matmul_f32(None, None, None, None, None, 1, 1, 256, 36, 0, None) == 1
    assert lib.bpq4k_last_error_string(None) == b"null handle"
    assert lib.bpq4k_create(0, None) == 1


def test_strides_follow_pack_q4k():
    lib = _lib.load()
    for K, nb in [(256, 1), (512, 2), (4096, 16), (14336, 56), (300, 2)]:
        assert lib.bpq4k_n_blocks(K) == nb
        assert lib.bpq4k_row_stride_words(K) == nb * 36


def test_pack_host_is_identity():
    N, K = 9, 768
    w = synth.make_q4k_weights(N, K, 2)
    p = pack_q4k(w, N, K)
    assert p.rowStrideWords == 108 and p.nBlocks == 3 and p.N == N and p.K == K
    assert np.array_equal(p.data.view(np.uint8), w.reshape(-1))
    empty = pack_q4k(np.zeros(0, np.uint8), 0, 256)
    assert empty.data.size == 0


def test_fuse_kq_concatenates_rows():
    from backpack_b200 import fuse_kq
    from oracle import q4k_oracle as orc

    K = 512
    q, k = synth.make_q4k_weights(6, K, 1), synth.make_q4k_weights(3, K, 2)
    f = fuse_kq(pack_q4k(q, 6, K), pack_q4k(k, 3, K))
    assert (f.N, f.K, f.rowStrideWords, f.nBlocks) == (9, K, 72, 2)
    want = np.concatenate([orc.dequant(q, 6, K), orc.dequant(k, 3, K)])
    assert np.array_equal(orc.dequant(f.data.view(np.uint8), 9, K), want)


def test_kq_strides_and_pack_follow_the_reference_packers():
    """pack_q5k keeps 176-byte blocks; pack_q6k pads rows of 210-byte blocks to whole words with zeros."""
    from backpack_b200 import pack_kq
    from oracle import q4k_oracle as orc

    lib = _lib.load()
    assert [lib.bpq4k_kq_block_bytes(t) for t in (12, 13, 14, 8)] == [144, 176, 210, 0]
    for qtype, K, rs in [(12, 4096, 576), (13, 4096, 704), (14, 4096, 840), (14, 768, 158), (14, 256, 53), (13, 300, 88)]:
        assert lib.bpq4k_kq_row_stride_words(qtype, K) == rs
    for qtype in (12, 13, 14):
        N, K = 5, 768
        w = synth.make_kq_weights(qtype, N, K, 4)
        p = pack_kq(qtype, w, N, K)
        words, rs, nb = orc.kq_pack(qtype, w, N, K)
        assert (p.rowStrideWords, p.nBlocks, p.qtype) == (rs, nb, qtype)
        assert np.array_equal(p.data, words)
    assert lib.bpq4k_kq_pack_host(7, None, 0, 256, None) == 2
    # padded Q6_K: the same 210 bytes per block, then 14 zero bytes
    N, K = 3, 512
    w = synth.make_kq_weights(14, N, K, 5)
    p = pack_kq(0x10E, w, N, K)
    assert (p.rowStrideWords, lib.bpq4k_kq_block_bytes(0x10E)) == (112, 224)
    blocks = p.data.view(np.uint8).reshape(N * 2, 224)
    assert np.array_equal(blocks[:, :210], w.reshape(N * 2, 210)) and not blocks[:, 210:].any()
