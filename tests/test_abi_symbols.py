"""CPU: the C-ABI library loads and exports every symbol include/spx_b200.h declares, and fails
loudly (never silently falls back) when no CUDA device is present."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "spx_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spx_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path():
    names = declared_symbols()
    for must in ("spx_ell_create", "spx_spmm", "spx_spmv", "spx_conv2d", "spx_eltwise", "spx_spmm_host",
                 "spx_spmv_host", "spx_allgather_rows", "spx_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    import spx_ctypes
    dll = ctypes.CDLL(spx_ctypes.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(dll, s)]
    assert not missing, f"declared in spx_b200.h but not exported: {missing}"


def test_ctypes_stub_covers_the_header():
    import spx_ctypes
    assert sorted(spx_ctypes.SIGNATURES) == declared_symbols()


def test_python_module_surface(backend):
    """Names of the reference's pybind11 module (src/bindings.cpp:50-217) plus resize_buffers."""
    for name in ("Ellpack", "convert_to_ellpack", "decode_from_ellpack", "ellpack_matvec", "ellpack_matmul",
                 "SparseOnnxModel"):
        assert hasattr(backend, name)
    for meth in ("run", "resize_buffers", "output_shape"):
        assert hasattr(backend.SparseOnnxModel, meth)
    import cpp_backend
    assert all(hasattr(cpp_backend, f) for f in ("encode", "matvec", "matmul"))


def test_no_cpu_fallback_without_a_gpu(lib, backend):
    import numpy as np
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import spx_ctypes
    with pytest.raises(spx_ctypes.SpxError):
        lib.ell_create(np.ones((2, 1), np.float32), np.zeros((2, 1), np.uint32), np.ones(2, np.uint32), 3)
    with pytest.raises(RuntimeError):
        backend.convert_to_ellpack(np.eye(3, dtype=np.float32))
