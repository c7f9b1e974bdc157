"""The allocation-free entry point, bpq4k_matmul_noalloc_f32.

Some users of this library may not allocate device memory when they call it: a serving
process whose own pool already owns all free HBM, or a decode loop that cannot take the
device-wide stall of cudaMalloc/cudaFree.  For them the library keeps a fixed scratch array
on the device and offers one entry point that uses it and takes no handle.  This test calls
that entry point through the C ABI twice in a row (the second call finds the first call's
leftovers in the shared scratch) and compares each result with the regular entry point's.

The file name sorts last on purpose: if this test fails, a run that stops at the first
failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from backpack_b200 import _lib, pack_q4k, synth

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3
MAX_ABS_TOL = 2e-2


def _noalloc(lib, x, w, bias, y, M, N, K, stride, y_offset=0):
    import torch

    return lib.bpq4k_matmul_noalloc_f32(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                        y.data_ptr(), M, N, K, stride, y_offset,
                                        torch.cuda.current_stream().cuda_stream)


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    import torch

    import backpack_b200 as bp

    lib = _lib.load()
    ctx = bp.Q4KContext(0)          # only for the regular entry point we compare against
    torch.cuda.set_device(0)
    # two different problems back to back: the second must not be disturbed by what the first left behind
    for (M, N, K, seed) in [(8, 600, 4096, 1), (1, 1000, 14336, 2), (3, 130, 512, 3), (8, 600, 4096, 4)]:
        raw = synth.make_q4k_weights(N, K, seed)
        packed = pack_q4k(raw, N, K)
        w = ctx.upload(packed)
        x = torch.from_numpy(synth.make_activations(M, K, seed + 10)).cuda()
        bias = torch.linspace(-1, 1, N, device="cuda")
        want = ctx.matmul(x, w, bias)
        got = torch.full((M, N), float("nan"), device="cuda")
        st = _noalloc(lib, x, w.buf, bias, got, M, N, K, w.rowStrideWords)
        assert st == 0, lib.bpq4k_noalloc_last_error().decode()
        torch.cuda.synchronize()
        a, b = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(a).all()
        assert np.linalg.norm(a - b) / np.linalg.norm(b) <= REL_L2_TOL
        assert np.abs(a - b).max() <= MAX_ABS_TOL


def test_noalloc_rejects_sizes_beyond_its_scratch_and_bad_arguments():
    import torch

    lib = _lib.load()
    torch.cuda.set_device(0)
    K = 4096
    w = torch.zeros(16 * (K // 256) * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros(16, K, device="cuda")
    y = torch.zeros(16, 16, device="cuda")
    stride = (K // 256) * 36
    assert _noalloc(lib, x, w, None, y, 9, 16, K, stride) == 2            # M > 8
    assert b"beyond the fixed scratch" in lib.bpq4k_noalloc_last_error()
    bigK = 32768                                                          # 8 * 32768 > BPQ4K_NOALLOC_MAX_MK
    assert _noalloc(lib, x, w, None, y, 8, 16, bigK, (bigK // 256) * 36) == 2
    assert _noalloc(lib, x, w, None, y, 1, 16, 300, 72) == 2              # K not a multiple of 256
    assert _noalloc(lib, x, w, None, y, 1, 16, K, stride - 4) == 1        # stride shorter than a row
    assert lib.bpq4k_matmul_noalloc_f32(None, w.data_ptr(), None, y.data_ptr(), 1, 16, K, stride, 0, None) == 1
    assert _noalloc(lib, x, w, None, y, 0, 16, K, stride) == 0            # empty problem
    # and it still works afterwards
    assert _noalloc(lib, x, w, None, y, 2, 16, K, stride) == 0
    torch.cuda.synchronize()
    assert (y[:2] == 0).all()
