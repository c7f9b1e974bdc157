import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "q4k_golden.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def kq_golden():
    """Reference-generated vectors for the Q5_K / Q6_K siblings (tests/golden/make_golden_kq.py)."""
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "kq_golden.npz")))


KQ_GOLDEN_MATMUL = ["kt_q5k_matmul", "kt_q6k_matmul", "kt_q6k_matmul_wide", "kt_q5k_matmul_batched4",
                    "kt_q6k_matmul_batched4", "corner_q5k", "corner_q6k", "synthetic_q5k", "synthetic_q6k"]
KQ_GOLDEN_GATHER = ["kt_q6k_gather", "kt_q6k_gather_batched"]

GOLDEN_CASES = ["kt_q4k_matmul", "kt_q4k_matmul_128", "kt_q4k_matmul_batched4", "kt_q4k_matmul_batched8",
                "corner", "synthetic"]


@pytest.fixture(scope="session")
def ctx():
    """One library handle on cuda:0 for the GPU tests; fails loudly if the library is missing."""
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import backpack_b200 as bp

    c = bp.Q4KContext(0)
    yield c
    c.close()


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.sqrt((b * b).sum())
    return float(np.sqrt(((a - b) ** 2).sum()) / den) if den else float(np.abs(a - b).max())


def assert_close_ref(actual, expected, atol=2e-4, rtol=2e-4):
    """assertClose of the reference's kernel tests (runtime/tests/kernel_test.cpp:298-317)."""
    actual = np.asarray(actual, np.float32).ravel()
    expected = np.asarray(expected, np.float32).ravel()
    diff = np.abs(actual - expected)
    tol = atol + rtol * np.abs(expected)
    bad = diff > tol
    assert not bad.any(), (f"idx={int(np.argmax(diff * bad))}: got={actual[np.argmax(diff * bad)]} "
                           f"expected={expected[np.argmax(diff * bad)]} diff={diff.max()}")
