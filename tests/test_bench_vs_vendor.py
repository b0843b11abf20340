"""The vendor-comparison command line (sparse-ops_b200/bench_vs_vendor.py), counterpart of the
reference's sparse_matmul_bench / sparse_matvec_bench (benchmark-mkl/matmul/main_matmul.cpp:49-139).
CPU: flags and the seeded case generator.  GPU: a small run whose ELLPACK arm is checked against the
oracle and whose JSON line carries the agreed keys."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import bench_vs_vendor as bv
from conftest import PKG, assert_bit_equal


def test_flags_and_defaults():
    a = bv.parse_args([])
    assert (a.M, a.N, a.C, a.sparsity, a.runs, a.seed, a.irregular) == (4096, 4096, 256, 0.9, 50, 42, False)
    a = bv.parse_args("--M 300 --N 200 --C 1 --sparsity 0.5 --runs 3 --seed 7 --irregular".split())
    assert (a.M, a.N, a.C, a.sparsity, a.runs, a.seed, a.irregular) == (300, 200, 1, 0.5, 3, 7, True)
    for bad in (["--M", "0"], ["--sparsity", "1.5"], ["--runs", "0"], ["--no-such-flag"]):
        with pytest.raises(SystemExit):
            bv.parse_args(bad)


@pytest.mark.parametrize("irregular", [False, True])
def test_case_generator_is_seeded_and_well_formed(irregular):
    argv = "--M 500 --N 800 --C 12 --sparsity 0.95 --seed 5".split() + (["--irregular"] if irregular else [])
    a = bv.parse_args(argv)
    rowptr, col, val, X, bias = bv.build_case(a)
    again = bv.build_case(a)
    for u, v in zip((rowptr, col, val, X, bias), again):
        assert np.array_equal(u, v)
    assert rowptr.shape == (501,) and rowptr[0] == 0 and int(rowptr[-1]) == len(col) == len(val)
    assert X.shape == (800, 12) and X.dtype == np.float32 and bias.shape == (500,)
    assert col.max() < 800 and np.abs(X).max() <= 1.0
    cnt = np.diff(rowptr.astype(np.int64))
    for i in np.flatnonzero(cnt > 1)[:50]:                 # columns strictly ascending inside a row
        seg = col[int(rowptr[i]):int(rowptr[i + 1])]
        assert (np.diff(seg.astype(np.int64)) > 0).all()
    mean = 0.05 * 800
    assert 0.5 * mean < cnt.mean() < 1.5 * mean
    if irregular:
        assert cnt.max() > 4 * mean                        # power-law rows: a long tail
    other = bv.build_case(bv.parse_args(argv[:-2 if not irregular else -3] + ["--seed", "6"] + (["--irregular"] if irregular else [])))
    assert not np.array_equal(other[3], X)


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--C", "1"], ["--irregular", "--C", "36"]], ids=["spmm", "spmv", "irregular"])
def test_small_run_matches_oracle_and_prints_the_keys(orc, extra):
    import workloads as wl
    from oracle import EllArrays
    argv = ["--M", "256", "--N", "256", "--C", "20", "--sparsity", "0.9", "--runs", "2"] + extra
    a = bv.parse_args(argv)
    out, Y = bv.run(a)
    assert set(out) == set(bv.JSON_KEYS)
    assert out["ellpack_ms"] > 0 and out["cusparse_ms"] > 0 and out["cublas_dense_ms"] > 0
    assert out["max_abs_diff_vs_cusparse"] < 1e-3
    rowptr, col, val, X, bias = bv.build_case(a)
    Wd, idx, nnz = wl.csr_to_ell(a.M, rowptr, col, val)
    E = EllArrays(a.M, a.N, Wd.shape[1], Wd, idx, nnz)
    if a.C == 1:
        x = X[:, 0].copy()
        assert (np.abs(Y[:, 0] - orc.spmv(E, x, bias)) <= 1e-5 * orc.absbound(E, x, bias)).all()
    else:
        assert_bit_equal(Y, orc.spmm(E, X, bias), "ELLPACK arm of the vendor benchmark")
    # and as a command: one JSON line
    res = subprocess.run([sys.executable, os.path.join(PKG, "bench_vs_vendor.py")] + argv, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][0])
    assert set(line) == set(bv.JSON_KEYS) and line["nnz"] == out["nnz"]
