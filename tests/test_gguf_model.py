"""Model-level GGUF reading: extractModelConfig against the reference's own function compiled from its sources
(field for field, on files that exercise every branch: plain llama, the Gemma variants with their sliding-window
patterns, expert and state-space hyper-parameters, key_length overrides, MTP markers), and the loader's
quantisation probe.  CPU only."""
import ctypes as C

import numpy as np
import pytest

import gguf_writer as gw
from backpack_b200 import _lib, synth
from backpack_b200.gguf import GGUFFile
from oracle import q4k_oracle as orc

K = 256


def t_q(name, rows, typ=12, k=K):
    return (name, (k, rows), typ, synth.make_kq_weights(typ, rows, k, abs(hash(name)) % 1000))


def t_f32(name, n=K):
    return (name, (n,), 0, np.ones(n, np.float32))


def base_meta(arch, n_layer=3):
    return [("general.architecture", gw.STRING, arch), (f"{arch}.block_count", gw.U32, n_layer),
            (f"{arch}.embedding_length", gw.U32, 512), (f"{arch}.feed_forward_length", gw.U32, 1024),
            (f"{arch}.attention.head_count", gw.U32, 8)]


CASES = {
    "llama_plain": (base_meta("llama") + [("llama.attention.head_count_kv", gw.U32, 2),
                                          ("llama.attention.layer_norm_rms_epsilon", gw.F32, 1e-5),
                                          ("llama.rope.freq_base", gw.F32, 500000.0)],
                    [t_q("token_embd.weight", 40, 14), t_q("blk.0.attn_q.weight", 16), t_f32("blk.1.attn_q_norm.weight")]),
    "no_arch_key_defaults": ([("llama.block_count", gw.U32, 2), ("llama.embedding_length", gw.U64, 256),
                              ("llama.attention.head_count", gw.I32, 0)],
                             [("token_embd.weight", (7,), 0, np.zeros(7, np.float32))]),
    "gemma2_sliding": (base_meta("gemma2", 5) + [("gemma2.attention.sliding_window", gw.U32, 4096),
                                                  ("gemma2.final_logit_softcapping", gw.F32, 30.0)],
                       [t_q("token_embd.weight", 24), t_f32("blk.0.post_attention_norm.weight")]),
    "gemma3_sliding": (base_meta("gemma3", 13) + [("gemma3.attention.sliding_window", gw.U32, 1024),
                                                   ("gemma3.attention.key_length", gw.U32, 256)],
                       [t_q("token_embd.weight", 24), t_f32("blk.0.attn_q_norm.weight"), t_f32("blk.0.attn_post_norm.weight")]),
    "gemma4_pattern": (base_meta("gemma4", 4) + [("gemma4.attention.sliding_window", gw.U32, 512),
                                                  ("gemma4.attention.sliding_window_pattern", gw.ARRAY, (gw.BOOL, [1, 1, 0, 1])),
                                                  ("gemma4.attention.shared_kv_layers", gw.U32, 2),
                                                  ("gemma4.embedding_length_per_layer_input", gw.U32, 256)],
                       [t_q("token_embd.weight", 24), t_f32("blk.0.post_norm.weight")]),
    "gemma4_pattern_wrong_length": (base_meta("gemma4", 7) + [("gemma4.attention.sliding_window", gw.U32, 512),
                                                               ("gemma4.attention.sliding_window_pattern", gw.ARRAY, (gw.BOOL, [1, 0]))],
                                    [t_q("token_embd.weight", 24)]),
    "gemma_no_window": (base_meta("gemma", 2), [t_q("token_embd.weight", 24)]),
    "qwen3moe": (base_meta("qwen3moe", 2) + [("qwen3moe.expert_count", gw.U32, 128), ("qwen3moe.expert_used_count", gw.U32, 8),
                                              ("qwen3moe.expert_feed_forward_length", gw.U32, 768)],
                 [t_q("token_embd.weight", 24), ("blk.0.ffn_gate_exps.weight", (K, 8, 4), 12, synth.make_kq_weights(12, 32, K, 4))]),
    "qwen35moe_hybrid": (base_meta("qwen35moe", 4) + [("qwen35moe.expert_count", gw.U32, 64), ("qwen35moe.expert_used_count", gw.U32, 4),
                                                       ("qwen35moe.expert_feed_forward_length", gw.U32, 512),
                                                       ("qwen35moe.expert_shared_feed_forward_length", gw.U32, 1024),
                                                       ("qwen35moe.ssm.inner_size", gw.U32, 2048), ("qwen35moe.ssm.state_size", gw.U32, 128),
                                                       ("qwen35moe.ssm.conv_kernel", gw.U32, 4), ("qwen35moe.ssm.group_count", gw.U32, 16),
                                                       ("qwen35moe.ssm.time_step_rank", gw.U32, 32),
                                                       ("qwen35moe.full_attention_interval", gw.U32, 4),
                                                       ("qwen35moe.rope.dimension_sections", gw.ARRAY, (gw.I32, [16, 24, 24, 0, 99])),
                                                       ("qwen35moe.nextn_predict_layers", gw.U32, 1),
                                                       ("qwen35moe.attention.key_length", gw.U32, 256)],
                         [t_q("token_embd.weight", 24), t_f32("blk.3.attn_q_norm.weight")]),
    "mtp_markers": (base_meta("llama", 2), [t_q("token_embd.weight", 24), t_f32("mtp.0.enorm.weight")]),
    "short_rope_sections": (base_meta("qwen35", 2) + [("qwen35.rope.dimension_sections", gw.ARRAY, (gw.I32, [1, 2, 3]))],
                            [t_q("token_embd.weight", 24)]),
    "output_weight_as_metadata_key": (base_meta("llama", 1) + [("output.weight", gw.U32, 1)], [t_q("output.weight", 24), t_q("token_embd.weight", 24)]),
}


def ours(path):
    g = GGUFFile(path)
    cfg = _lib.ModelConfig()
    types = (C.c_uint8 * 64)()
    assert g.lib.bpq4k_gguf_model_config(g.h, C.byref(cfg), types, 64) == 0
    return g, cfg, bytes(types)


@pytest.mark.parametrize("case", sorted(CASES))
def test_model_config_reads_what_was_written(tmp_path, case):
    meta, tensors = CASES[case]
    path = str(tmp_path / "m.gguf")
    gw.write_gguf(path, meta, tensors)
    g, cfg, types = ours(path)
    d = g.model_config()
    arch = dict((k, v) for k, _, v in meta).get("general.architecture", "llama")
    assert d["arch"] == arch and d["nLayer"] == dict((k, v) for k, _, v in meta)[f"{arch}.block_count"]
    assert d["tieWordEmbeddings"] == (0 if case == "output_weight_as_metadata_key" else 1)
    if case == "gemma2_sliding":
        assert d["layerAttnTypes"] == [1, 0, 1, 0, 1] and d["activation"] == 1 and d["hasSandwichNorm"] == 1
        assert abs(d["embeddingScale"] - 512 ** 0.5) < 1e-4 and d["logitSoftcap"] == 30.0
    if case == "gemma3_sliding":
        assert d["layerAttnTypes"] == [1, 1, 1, 1, 1, 0, 1, 1, 1, 1, 1, 0, 1] and d["headDim"] == 256 and d["hasQkNorm"] == 1
    if case == "gemma4_pattern":
        assert d["layerAttnTypes"] == [1, 1, 0, 1] and d["sharedKvLayers"] == 2 and d["pleSize"] == 256
    if case == "gemma4_pattern_wrong_length":
        assert d["layerAttnTypes"] == [1, 1, 1, 1, 1, 0, 1]
    if case == "qwen35moe_hybrid":
        assert (d["numExperts"], d["numExpertsPerTok"], d["moeIntermediateSize"], d["moeSharedIntermediateSize"]) == (64, 4, 512, 1024)
        assert d["ropeSections"] == [16, 24, 24, 0] and d["hasMtp"] == 1 and d["mtpNumLayers"] == 1 and d["hasQkNorm"] == 1
        assert d["fullAttentionInterval"] == 4 and d["ssmInnerSize"] == 2048
    if case == "qwen3moe":
        assert d["moeSharedIntermediateSize"] == 768 and d["nVocab"] == 24
    if case == "short_rope_sections":
        assert d["ropeSections"] == [11, 11, 10, 0]
    if case == "no_arch_key_defaults":
        assert d["nVocab"] == 7 and d["headDim"] == 0 and d["nKvHeads"] == 0
    g.close()


@pytest.mark.skipif(not orc.ref_available(), reason="compiled reference not present")
@pytest.mark.parametrize("case", sorted(CASES))
def test_model_config_equals_the_references(tmp_path, case):
    """Byte for byte against extractModelConfig of the reference (runtime/gguf_loader.cpp:184-317)."""
    meta, tensors = CASES[case]
    path = str(tmp_path / "m.gguf")
    gw.write_gguf(path, meta, tensors)
    g, cfg, types = ours(path)
    R = orc.ref_lib()
    R.ref_gguf_open.restype = C.c_void_p
    R.ref_gguf_open.argtypes = [C.c_char_p]
    R.ref_gguf_close.argtypes = [C.c_void_p]
    R.ref_extract_model_config.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32]
    ref = R.ref_gguf_open(path.encode())
    assert ref
    rcfg = _lib.ModelConfig()
    rtypes = (C.c_uint8 * 64)()
    assert R.ref_extract_model_config(ref, C.byref(rcfg), rtypes, 64) == 0
    for name, _ in _lib.ModelConfig._fields_:
        a, b = getattr(cfg, name), getattr(rcfg, name)
        assert (list(a) == list(b)) if name == "ropeSections" else (a == b), (case, name, a, b)
    assert types == bytes(rtypes)
    R.ref_gguf_close(ref)
    g.close()


def test_weight_format_probe(tmp_path):
    def probe(tensors):
        path = str(tmp_path / "w.gguf")
        gw.write_gguf(path, base_meta("llama", 1), tensors)
        g = GGUFFile(path)
        r = g.weight_format()
        g.close()
        return r

    assert probe([t_q("blk.0.attn_q.weight", 16), t_q("blk.0.ffn_gate.weight", 16), t_q("blk.0.ffn_down.weight", 16)]) == (12, True)
    # a "Q4_K_M" style mix: ffn_down in Q6_K -> not uniform (the reference re-quantises such models to Q8)
    assert probe([t_q("blk.0.attn_q.weight", 16), t_q("blk.0.ffn_gate.weight", 16), t_q("blk.0.ffn_down.weight", 16, 14)]) == (12, False)
    assert probe([t_q("blk.0.attn_qkv.weight", 48, 13), t_q("blk.0.ffn_gate.weight", 16, 13), t_q("blk.0.ffn_down.weight", 16, 13)]) == (13, True)
    assert probe([("blk.0.attn_q.weight", (K, 4), 0, np.zeros((4, K), np.float32))]) == (0, False)
    assert probe([t_f32("blk.0.attn_norm.weight")]) == (-1, False)
