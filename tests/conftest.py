"""Shared fixtures.  Tests marked `gpu` need a CUDA device; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sparse-ops_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.Oracle()


@pytest.fixture(scope="session")
def ref():
    """The unmodified reference build; only where it was compiled and the host has AVX-512."""
    import oracle
    if not oracle.reference_available():
        pytest.skip("oracle/_ref not built for this host")
    return oracle.Reference()


@pytest.fixture(scope="session")
def lib():
    """ctypes view of libspx_b200.so (the C ABI)."""
    import spx_ctypes
    return spx_ctypes.Lib()


@pytest.fixture(scope="session")
def backend():
    import sparseops_backend
    return sparseops_backend


@pytest.fixture(scope="session")
def cuda():
    import torch
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_equal(a, b, what=""):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    same = a.view(np.uint32) == b.view(np.uint32)
    if not same.all():
        bad = np.argwhere(~same)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {a.size} elements differ bitwise; first at {i}: {a[i]!r} vs {b[i]!r}")
