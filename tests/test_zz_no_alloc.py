"""The allocation-free entry point, bpq4k_matmul_noalloc_f32.

Some users of this library may not allocate device memory when they call it: a serving
process whose own pool already owns all free HBM, or a decode loop that cannot take the
device-wide stall of cudaMalloc/cudaFree.  For them the library keeps a fixed scratch array
on the device and offers one entry point that uses it and takes no handle.  This test calls
that entry point through the C ABI twice in a row (the second call finds the first call's
leftovers in the shared scratch) and compares each result with the regular entry point's and
with the CPU checker's, and checks the property the entry point exists for: the free device
memory is the same before and after a call.

The file name sorts last on purpose: if this test fails, a run that stops at the first
failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from backpack_b200 import _lib, pack_q4k, synth
from oracle import q4k_oracle as orc

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3
MAX_ABS_TOL = 2e-2


def _noalloc(lib, x, w, bias, y, M, N, K, stride, y_offset=0):
    import torch

    return lib.bpq4k_matmul_noalloc_f32(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                        y.data_ptr(), M, N, K, stride, y_offset,
                                        torch.cuda.current_stream().cuda_stream)


def _close(a, b):
    assert np.isfinite(a).all()
    assert np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b.astype(np.float64)) <= REL_L2_TOL
    assert np.abs(a - b).max() <= MAX_ABS_TOL


def _run_cases(device: int):
    import torch

    import backpack_b200 as bp

    lib = _lib.load()
    ctx = bp.Q4KContext(device)          # only for the regular entry point we compare against
    torch.cuda.set_device(device)
    dev = f"cuda:{device}"
    # different problems back to back: each must not be disturbed by what the one before left behind
    for (M, N, K, seed) in [(8, 600, 4096, 1), (1, 1000, 14336, 2), (3, 130, 512, 3), (8, 600, 4096, 4)]:
        raw = synth.make_q4k_weights(N, K, seed)
        w = ctx.upload(pack_q4k(raw, N, K))
        x_host = synth.make_activations(M, K, seed + 10)
        x = torch.from_numpy(x_host).to(dev)
        bias_host = np.linspace(-1, 1, N).astype(np.float32)
        bias = torch.from_numpy(bias_host).to(dev)
        want = ctx.matmul(x, w, bias).cpu().numpy()
        want_cpu = orc.matmul(x_host, raw, bias_host, N, K)
        got = torch.full((M, N), float("nan"), device=dev)
        # first call of this shape: may load the kernel's module (the driver loads code lazily)
        st = _noalloc(lib, x, w.buf, bias, got, M, N, K, w.rowStrideWords)
        assert st == 0, lib.bpq4k_noalloc_last_error().decode()
        torch.cuda.synchronize()
        _close(got.cpu().numpy(), want)
        _close(got.cpu().numpy(), want_cpu)
        # second call in a row: same result, and the device's free memory does not move across it
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(device)
        st = _noalloc(lib, x, w.buf, bias, got, M, N, K, w.rowStrideWords)
        assert st == 0, lib.bpq4k_noalloc_last_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(device)
        assert free_after == free_before, (free_before, free_after)
        _close(got.cpu().numpy(), want)
        _close(got.cpu().numpy(), want_cpu)
    ctx.close()


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    _run_cases(0)


def test_noalloc_on_a_second_device_when_there_is_one():
    """The scratch array's address is looked up once per device, with that device current."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    try:
        _run_cases(1)
    finally:
        torch.cuda.set_device(0)


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
