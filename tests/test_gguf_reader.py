"""The GGUF reader on files written by tests/gguf_writer.py: against what was written, and against the
reference's own reader (GGUFFile::open compiled from its sources) when that is present.  CPU only."""
import ctypes as C
import os

import numpy as np
import pytest

import gguf_writer as gw
from backpack_b200 import synth
from backpack_b200.gguf import GGUFFile
from backpack_b200.q4k import Q4KError
from oracle import q4k_oracle as orc

META = [
    ("general.architecture", gw.STRING, "llama"),
    ("general.name", gw.STRING, "synthetic test model"),
    ("llama.block_count", gw.U32, 2),
    ("llama.embedding_length", gw.U64, 512),
    ("llama.attention.head_count", gw.I32, 8),
    ("llama.attention.layer_norm_rms_epsilon", gw.F32, 1e-5),
    ("llama.rope.freq_base", gw.F64, 500000.0),
    ("llama.feed_forward_length", gw.ARRAY, (gw.I32, [1024, 2048, 1536])),
    ("small.u8", gw.U8, 200), ("small.i8", gw.I8, -3), ("small.u16", gw.U16, 60000), ("small.i16", gw.I16, -1234),
    ("big.i64", gw.I64, 77),
    ("flag.yes", gw.BOOL, 1), ("flag.no", gw.BOOL, 0),
    ("tokenizer.ggml.tokens", gw.ARRAY, (gw.STRING, ["<s>", "</s>", "hello", "wörld", ""])),
    ("tokenizer.ggml.token_type", gw.ARRAY, (gw.I32, [3, 3, 1, 1, 1])),
    ("tokenizer.ggml.scores", gw.ARRAY, (gw.F32, [0.0, -1.5, 2.25])),
    ("some.bools", gw.ARRAY, (gw.BOOL, [1, 0, 1])),
    ("some.u8s", gw.ARRAY, (gw.U8, [1, 2, 3, 4])),
]


def make_file(tmp_path, alignment=32, with_alignment_key=False):
    K = 512
    tensors = [
        ("token_embd.weight", (K, 40), 14, synth.make_kq_weights(14, 40, K, 1)),
        ("blk.0.attn_q.weight", (K, 64), 12, synth.make_kq_weights(12, 64, K, 2)),
        ("blk.0.ffn_down.weight", (K, 48), 13, synth.make_kq_weights(13, 48, K, 3)),
        ("blk.0.attn_norm.weight", (K,), 0, np.linspace(0.5, 1.5, K).astype(np.float32)),
        ("blk.0.ffn_gate_exps.weight", (256, 8, 3), 12, synth.make_kq_weights(12, 24, 256, 4)),
        ("odd.q6k", (768, 5), 14, synth.make_kq_weights(14, 5, 768, 5)),
    ]
    meta = list(META) + ([("general.alignment", gw.U32, alignment)] if with_alignment_key else [])
    path = str(tmp_path / "model.gguf")
    offsets = gw.write_gguf(path, meta, tensors, alignment=alignment)
    return path, tensors, offsets


def test_reader_returns_what_was_written(tmp_path):
    path, tensors, offsets = make_file(tmp_path)
    g = GGUFFile(path)
    assert (g.version, g.n_tensors) == (3, len(tensors)) and g.data_offset % 32 == 0
    assert g.getString("general.architecture") == "llama" and g.getString("missing", "dflt") == "dflt"
    assert g.getU32("llama.block_count") == 2 and g.getU32("llama.embedding_length") == 512
    assert g.getU32("llama.attention.head_count") == 8 and g.getU32("missing", 9) == 9
    assert g.getU32("llama.feed_forward_length") == 2048              # maximum of an int array, as the reference does
    assert (g.getU32("small.u8"), g.getU32("small.u16"), g.getU32("big.i64")) == (200, 60000, 77)
    assert g.getU32("small.i8") == (-3) & 0xFFFFFFFF and g.getU32("small.i16") == (-1234) & 0xFFFFFFFF
    assert abs(g.getFloat("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12 and g.getFloat("llama.rope.freq_base") == 500000.0
    assert g.getFloat("general.name", 4.0) == 4.0                     # wrong type -> default
    assert g.getBool("flag.yes") and not g.getBool("flag.no") and g.getBool("missing", True)
    assert g.hasKey("some.u8s") and not g.hasKey("nope")
    assert g.getStringArray("tokenizer.ggml.tokens") == ["<s>", "</s>", "hello", "wörld", ""]
    assert g.getStringArray("tokenizer.ggml.token_type") is None
    assert list(g.getI32Array("tokenizer.ggml.token_type")) == [3, 3, 1, 1, 1]
    assert list(g.getI32Array("some.bools")) == [1, 0, 1]
    for (name, shape, typ, data), info in zip(tensors, g.tensors):
        assert (info.name, info.shape, info.type, info.offset) == (name, tuple(shape), typ, offsets[name])
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        assert info.n_bytes == raw.size
        assert np.array_equal(g.read(name), raw)
    g.close()


def test_alignment_key_is_honoured(tmp_path):
    path, tensors, offsets = make_file(tmp_path, alignment=64, with_alignment_key=True)
    g = GGUFFile(path)
    assert g.data_offset % 64 == 0
    name, _, _, data = tensors[1]
    assert np.array_equal(g.read(name), np.ascontiguousarray(data).view(np.uint8).reshape(-1))


@pytest.mark.parametrize("cut", [3, 10, 24, 40, 200, 700])
def test_truncated_or_foreign_files_are_errors(tmp_path, cut):
    path, _, _ = make_file(tmp_path)
    blob = open(path, "rb").read()
    bad = str(tmp_path / "cut.gguf")
    open(bad, "wb").write(blob[:cut])
    with pytest.raises(Q4KError):
        GGUFFile(bad)
    open(bad, "wb").write(b"NOPE" + blob[4:])
    with pytest.raises(Q4KError):
        GGUFFile(bad)
    huge = bytearray(blob)
    huge[16:24] = (2 ** 62).to_bytes(8, "little")          # absurd key-value count
    open(bad, "wb").write(bytes(huge))
    with pytest.raises(Q4KError):
        GGUFFile(bad)


@pytest.mark.skipif(not orc.ref_available(), reason="compiled reference not present")
def test_against_the_reference_reader(tmp_path):
    path, tensors, _ = make_file(tmp_path)
    R = orc.ref_lib()
    R.ref_gguf_open.restype = C.c_void_p
    R.ref_gguf_open.argtypes = [C.c_char_p]
    for fn, res in (("ref_gguf_version", C.c_uint32), ("ref_gguf_n_tensors", C.c_uint64), ("ref_gguf_data_offset", C.c_uint64)):
        getattr(R, fn).restype = res
        getattr(R, fn).argtypes = [C.c_void_p]
    R.ref_gguf_tensor.argtypes = [C.c_void_p, C.c_uint64, C.c_char_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64 * 4),
                                  C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
    R.ref_gguf_get_u32.restype = C.c_uint32
    R.ref_gguf_get_u32.argtypes = [C.c_void_p, C.c_char_p, C.c_uint32]
    R.ref_gguf_get_f32.restype = C.c_float
    R.ref_gguf_get_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_float]
    R.ref_gguf_get_bool.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    R.ref_gguf_has_key.argtypes = [C.c_void_p, C.c_char_p]
    R.ref_gguf_get_string.restype = C.c_int64
    R.ref_gguf_get_string.argtypes = [C.c_void_p, C.c_char_p, C.c_int64, C.c_char_p, C.c_uint64]
    R.ref_gguf_i32_array.restype = C.c_int64
    R.ref_gguf_i32_array.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]
    R.ref_gguf_close.argtypes = [C.c_void_p]
    ref = R.ref_gguf_open(path.encode())
    assert ref
    g = GGUFFile(path)
    assert g.version == R.ref_gguf_version(ref) and g.n_tensors == R.ref_gguf_n_tensors(ref)
    assert g.data_offset == R.ref_gguf_data_offset(ref)
    for i, info in enumerate(g.tensors):
        name = C.create_string_buffer(256)
        nd, shape, typ, off = C.c_uint32(), (C.c_uint64 * 4)(), C.c_uint32(), C.c_uint64()
        assert R.ref_gguf_tensor(ref, i, name, 256, C.byref(nd), C.byref(shape), C.byref(typ), C.byref(off)) == 0
        assert (info.name, info.shape, info.type, info.offset) == (name.value.decode(), tuple(shape[d] for d in range(nd.value)),
                                                                   typ.value, off.value)
    keys = [k for k, _, _ in META] + ["missing.key"]
    for k in keys:
        kb = k.encode()
        assert g.hasKey(k) == bool(R.ref_gguf_has_key(ref, kb)), k
        assert g.getU32(k, 4242) == R.ref_gguf_get_u32(ref, kb, 4242), k
        assert g.getFloat(k, -2.5) == R.ref_gguf_get_f32(ref, kb, -2.5), k
        assert g.getBool(k, False) == bool(R.ref_gguf_get_bool(ref, kb, 0)) and g.getBool(k, True) == bool(R.ref_gguf_get_bool(ref, kb, 1)), k
        if k == "some.u8s":
            continue    # the reference keeps an empty-string placeholder for arrays it skips; this reader keeps the array
        buf = C.create_string_buffer(512)
        n = R.ref_gguf_get_string(ref, kb, -1, buf, 512)
        assert g.getString(k, "\x02none") == (buf.value.decode() if n >= 0 else "\x02none"), k
    toks = g.getStringArray("tokenizer.ggml.tokens")
    for i, t in enumerate(toks):
        buf = C.create_string_buffer(512)
        assert R.ref_gguf_get_string(ref, b"tokenizer.ggml.tokens", i, buf, 512) == len(t.encode()) and buf.value.decode() == t
    arr = np.zeros(16, np.int32)
    n = R.ref_gguf_i32_array(ref, b"tokenizer.ggml.token_type", arr.ctypes.data, 16)
    assert list(arr[:n]) == list(g.getI32Array("tokenizer.ggml.token_type"))
    R.ref_gguf_close(ref)
