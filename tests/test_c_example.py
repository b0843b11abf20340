"""The C ABI from plain C: the example program compiles and links against libspx_b200.so with gcc
(CPU check) and, on a GPU, runs and reproduces a scalar fmaf loop bit for bit."""
import os
import subprocess

import pytest

from conftest import PKG, ROOT

SRC = os.path.join(PKG, "examples", "spmm_example.c")


def _build(tmp_path):
    exe = str(tmp_path / "spmm_example")
    cmd = ["gcc", "-std=c11", "-Wall", "-Werror", f"-I{os.path.join(ROOT, 'include')}", SRC, f"-L{PKG}", "-lspx_b200",
           f"-Wl,-rpath,{PKG}", "-lm", "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_c_example_compiles_and_fails_loudly_without_gpu(tmp_path):
    import torch
    exe = _build(tmp_path)
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the run is covered by the gpu test")
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode != 0 and "status" in res.stderr        # no CPU fallback


@pytest.mark.gpu
def test_c_example_runs(tmp_path):
    exe = _build(tmp_path)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.startswith("ok")
