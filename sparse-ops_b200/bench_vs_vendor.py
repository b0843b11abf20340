#!/usr/bin/env python
"""ELLPACK kernels of this library against the vendor libraries on the same GPU.

The reference ships C++ command-line benchmarks that time its ELLPACK kernels against MKL's sparse
routines and a dense BLAS (benchmark-mkl/matmul/main_matmul.cpp:49-139, benchmark-mkl/matvec/).
This is their counterpart on the GPU, with the same flags:

    python bench_vs_vendor.py --M 4096 --N 4096 --C 256 --sparsity 0.9 --runs 50 [--seed 42] [--irregular]

  ELLPACK   this library (spx_spmm / spx_spmv through the C ABI, device-resident operands)
  cuSPARSE  torch.sparse CSR  (torch.sparse.mm / torch.mv on a sparse_csr tensor)
  cuBLAS    dense torch.matmul on the densified matrix (skipped above 2^31 elements)

--C 1 times SpMV.  --irregular draws power-law row lengths (mean N*(1-sparsity), like the reference's
irregular generator) instead of iid entries.  Median of --runs CUDA-event timings after one warm-up,
as in the reference (benchmark-mkl/matmul/bench_matmul.cpp:97-117).  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


JSON_KEYS = ("M", "N", "C", "sparsity", "irregular", "nnz", "runs", "max_abs_diff_vs_cusparse", "ellpack_ms",
             "cusparse_ms", "cublas_dense_ms", "gflops_ellpack", "speedup_vs_cusparse")


def parse_args(argv=None):
    """The flags of the reference's sparse_matmul_bench / sparse_matvec_bench
    (benchmark-mkl/matmul/main_matmul.cpp:62-91) that have a meaning on the GPU."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--C", type=int, default=256)
    ap.add_argument("--sparsity", type=float, default=0.9)
    ap.add_argument("--runs", type=int, default=50)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--irregular", action="store_true")
    a = ap.parse_args(argv)
    if a.M < 1 or a.N < 1 or a.C < 1 or a.runs < 1 or not 0.0 <= a.sparsity <= 1.0:
        ap.error("need M, N, C, runs >= 1 and 0 <= sparsity <= 1")
    return a


def build_case(a):
    """Seeded host inputs of one run: CSR of the matrix, dense operand, bias (no GPU involved)."""
    import workloads as wl
    p = 1.0 - a.sparsity
    if a.irregular:
        kmax = max(1, min(a.N, int(32 * max(1.0, p * a.N))))
        rowptr, col, val = wl.cfg5_rows(0, (a.M + 4095) // 4096 * 4096, n=a.N, kmax=kmax, mean=max(1.0, p * a.N), seed=a.seed)
        rowptr = rowptr[:a.M + 1]
        col, val = col[:int(rowptr[-1])], val[:int(rowptr[-1])]
    else:
        rowptr, col, val = wl.bernoulli_csr(a.seed, a.M, a.N, p)
    rng = np.random.default_rng([a.seed, 1])
    X = rng.uniform(-1, 1, (a.N, a.C)).astype(np.float32)
    bias = rng.standard_normal(a.M).astype(np.float32)
    return rowptr, col, val, X, bias


def run(a):
    """Times the three arms; returns (the JSON line as a dict, this library's result as a host array)."""
    import torch

    import spx_ctypes as sx

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    dev = torch.device("cuda", 0)
    lib = sx.Lib()
    rowptr, col, val, X, bias = build_case(a)
    m = a.M
    nnz = int(rowptr[-1])

    ell = lib.ell_create_csr(m, a.N, rowptr, col, val)
    dX, dB = torch.from_numpy(X).to(dev), torch.from_numpy(bias).to(dev)
    dY = torch.empty((m, a.C), device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    csr = torch.sparse_csr_tensor(torch.from_numpy(rowptr.astype(np.int64)), torch.from_numpy(col.astype(np.int64)),
                                  torch.from_numpy(val), size=(m, a.N), device=dev)
    dense = csr.to_dense() if m * a.N < 2 ** 31 else None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def ours():
        if a.C == 1:
            ell.spmv(dX.data_ptr(), dB.data_ptr(), dY.data_ptr(), stream)
        else:
            ell.spmm(dX.data_ptr(), a.C, a.C, dB.data_ptr(), sx.ACT_NONE, dY.data_ptr(), a.C, stream)

    def cusparse():
        return (torch.mv(csr, dX[:, 0]) if a.C == 1 else torch.sparse.mm(csr, dX)) + dB[:, None if a.C > 1 else ...]

    def cublas():
        return torch.addmm(dB[:, None], dense, dX)

    def median_ms(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.runs):
            flush.zero_()                               # cold L2, like the library's own benchmark
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts))

    # agreement first (cuSPARSE sums in another order: tolerance, not bit equality)
    ours()
    torch.cuda.synchronize()
    Y = dY.cpu().numpy().copy()
    ref = cusparse()
    ref = ref.reshape(m, -1)
    err = float((dY[:, :ref.shape[1]] - ref).abs().max())
    out = {"M": m, "N": a.N, "C": a.C, "sparsity": a.sparsity, "irregular": a.irregular, "nnz": nnz, "runs": a.runs,
           "max_abs_diff_vs_cusparse": err, "ellpack_ms": median_ms(ours), "cusparse_ms": median_ms(cusparse),
           "cublas_dense_ms": median_ms(cublas) if dense is not None else None}
    out["gflops_ellpack"] = 2.0 * nnz * a.C / out["ellpack_ms"] / 1e6
    out["speedup_vs_cusparse"] = out["cusparse_ms"] / out["ellpack_ms"]
    return out, Y


def main(argv=None):
    out, _ = run(parse_args(argv))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
