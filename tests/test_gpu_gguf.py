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
