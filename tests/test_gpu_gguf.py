"""File -> device -> matmul: tensors uploaded straight from a GGUF file give the oracle's results,
and their device bytes equal what the host packers produce."""
import numpy as np
import pytest

from backpack_b200 import pack_kq, q4k
from backpack_b200.gguf import GGUFFile
from conftest import rel_l2
from oracle import q4k_oracle as orc
from test_gguf_reader import make_file

pytestmark = pytest.mark.gpu


def check(y, want):
    assert rel_l2(y, want) <= 1e-3
    assert float(np.abs(y - want).max()) <= 2e-2 * max(1.0, float(np.abs(want).max()) / 100.0)


@pytest.mark.parametrize("name,layout", [("blk.0.attn_q.weight", 0), ("blk.0.ffn_down.weight", 0), ("token_embd.weight", 0),
                                         ("token_embd.weight", q4k.Q6_K_PADDED), ("odd.q6k", 0), ("odd.q6k", q4k.Q6_K_PADDED),
                                         ("blk.0.ffn_gate_exps.weight", 0)])
def test_upload_from_file_and_multiply(ctx, tmp_path, name, layout):
    import torch

    path, tensors, _ = make_file(tmp_path)
    raw = {n: (shape, typ, np.ascontiguousarray(d).view(np.uint8).reshape(-1)) for n, shape, typ, d in tensors}
    g = GGUFFile(path)
    t = g.upload(ctx, name, layout)
    shape, ftype, bytes_ = raw[name]
    K, N = shape[0], int(np.prod(shape[1:]))
    assert (t.N, t.K, t.qtype) == (N, K, layout or ftype)
    w = t.as_weight()
    # device bytes = what the host packer writes for the same layout
    want_words = pack_kq(t.qtype, bytes_, N, K)
    assert t.rowStrideWords == want_words.rowStrideWords
    assert np.array_equal(w.buf.cpu().numpy()[: N * t.rowStrideWords * 4], want_words.data.view(np.uint8))
    # and the numbers
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, K), dtype=np.float32)
    y = ctx.matmul(torch.from_numpy(x).cuda(), w).cpu().numpy()
    check(y, orc.kq_matmul(ftype, x, bytes_, None, N, K))
    assert np.array_equal(ctx.dequant(w).cpu().numpy().view(np.uint32), orc.kq_dequant(ftype, bytes_, N, K).view(np.uint32))
    del w
    t.free()


def test_upload_rejects_other_types_and_layouts(ctx, tmp_path):
    from backpack_b200.q4k import Q4KError

    path, _, _ = make_file(tmp_path)
    g = GGUFFile(path)
    with pytest.raises(Q4KError):
        g.upload(ctx, "blk.0.attn_norm.weight")                  # F32
    with pytest.raises(Q4KError):
        g.upload(ctx, "blk.0.attn_q.weight", q4k.Q6_K_PADDED)    # a Q4_K tensor has no padded layout


def _layer_file(tmp_path):
    """Three layers that take the three roads of the loader's Q+K+V and gate+up rules."""
    import gguf_writer as gw
    from backpack_b200 import synth

    K, F = 512, 768
    def kq(name, rows, typ, k=K):
        return (name, (k, rows), typ, synth.make_kq_weights(typ, rows, k, abs(hash(name)) % 997))

    tensors = [
        # layer 0: everything Q4_K except ffn_down (Q6_K): Q+K+V and gate+up are fused by rows
        kq("blk.0.attn_q.weight", 64, 12), kq("blk.0.attn_k.weight", 16, 12), kq("blk.0.attn_v.weight", 16, 12),
        kq("blk.0.attn_output.weight", 32, 12), kq("blk.0.ffn_gate.weight", 48, 12), kq("blk.0.ffn_up.weight", 48, 12),
        kq("blk.0.ffn_down.weight", 32, 14, F),
        # layer 1: attn_v in Q6_K and ffn_up in Q5_K: nothing can be fused, every tensor goes up on its own
        kq("blk.1.attn_q.weight", 64, 12), kq("blk.1.attn_k.weight", 16, 12), kq("blk.1.attn_v.weight", 16, 14),
        kq("blk.1.attn_output.weight", 32, 13), kq("blk.1.ffn_gate.weight", 48, 12), kq("blk.1.ffn_up.weight", 48, 13),
        kq("blk.1.ffn_down.weight", 32, 12, F),
        # layer 2: a pre-fused attn_qkv (Q5_K), an F32 attn_output (not a K-quant: left to the caller), no FFN
        kq("blk.2.attn_qkv.weight", 96, 13), ("blk.2.attn_output.weight", (K, 4), 0, np.zeros((4, K), np.float32)),
        # layer 3: a layer that shares K/V with an earlier one ships attn_q only
        kq("blk.3.attn_q.weight", 64, 12),
    ]
    path = str(tmp_path / "layers.gguf")
    gw.write_gguf(path, [("general.architecture", gw.STRING, "llama"), ("llama.block_count", gw.U32, 4)], tensors)
    return path, {n: (shape, typ, np.ascontiguousarray(d).view(np.uint8).reshape(-1)) for n, shape, typ, d in tensors}


@pytest.mark.parametrize("q6_layout", [0, q4k.Q6_K_PADDED])
def test_load_layer_applies_the_loaders_fusion_rules(ctx, tmp_path, q6_layout):
    """Fused device tensors hold the members' rows one after the other (= fuseKQ of the host packers' outputs), and a
    matmul on a fused tensor gives the checker's results for the concatenated rows."""
    import torch

    path, raw = _layer_file(tmp_path)
    g = GGUFFile(path)
    rng = np.random.default_rng(5)

    def verify(t, names):
        ftype = raw[names[0]][1]
        K = raw[names[0]][0][0]
        rows = [raw[n][0][1] for n in names]
        bytes_ = np.concatenate([raw[n][2] for n in names])
        N = sum(rows)
        layout = q6_layout if (ftype == 14 and q6_layout) else ftype
        assert (t.N, t.K, t.qtype) == (N, K, layout)
        w = t.as_weight()
        want_words = pack_kq(layout, bytes_, N, K)
        assert np.array_equal(w.buf.cpu().numpy()[: N * t.rowStrideWords * 4], want_words.data.view(np.uint8))
        x = rng.standard_normal((3, K), dtype=np.float32)
        y = ctx.matmul(torch.from_numpy(x).cuda(), w).cpu().numpy()
        check(y, orc.kq_matmul(ftype, x, bytes_, None, N, K))
        del w

    l0 = g.load_layer(ctx, 0, q6_layout)
    assert set(k for k in l0 if k not in ("qkv_prefused", "n_fused", "file_types")) == {"qkv", "o", "gate_up", "down"}
    assert l0["n_fused"] == {"qkv": 3, "o": 1, "gate_up": 2, "down": 1} and not l0["qkv_prefused"]
    verify(l0["qkv"], ["blk.0.attn_q.weight", "blk.0.attn_k.weight", "blk.0.attn_v.weight"])
    verify(l0["o"], ["blk.0.attn_output.weight"])
    verify(l0["gate_up"], ["blk.0.ffn_gate.weight", "blk.0.ffn_up.weight"])
    verify(l0["down"], ["blk.0.ffn_down.weight"])

    l1 = g.load_layer(ctx, 1, q6_layout)
    assert set(k for k in l1 if k not in ("qkv_prefused", "n_fused", "file_types")) == {"q", "k", "v", "o", "gate", "up", "down"}
    for key, name in (("q", "attn_q"), ("k", "attn_k"), ("v", "attn_v"), ("o", "attn_output"), ("gate", "ffn_gate"), ("up", "ffn_up"),
                      ("down", "ffn_down")):
        verify(l1[key], [f"blk.1.{name}.weight"])

    l2 = g.load_layer(ctx, 2, q6_layout)
    assert l2["qkv_prefused"] and l2["n_fused"] == {"qkv": 1} and l2["file_types"]["o"] == 0 and "o" not in l2
    verify(l2["qkv"], ["blk.2.attn_qkv.weight"])

    l3 = g.load_layer(ctx, 3, q6_layout)
    assert set(k for k in l3 if k not in ("qkv_prefused", "n_fused", "file_types")) == {"q"}
    verify(l3["q"], ["blk.3.attn_q.weight"])
    assert g.load_layer(ctx, 9, q6_layout)["n_fused"] == {}          # a layer the file does not have: nothing, no error
    g.close()
