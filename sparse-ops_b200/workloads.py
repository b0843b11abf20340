"""Seeded synthetic inputs for the five benchmark configurations of the ELLPACK hot path.

The reference benchmarks on synthetic random matrices only (its benchmark-mkl/common/data_gen.cpp:
Bernoulli keep mask, N(0,1) values; operands U(-1,1)); no public dataset is involved.  Arrays are
drawn from ``numpy.random.default_rng([seed, k])`` (k = array index) so the CPU checker and the
GPU library see the same bytes.  Every generator takes a ``scale`` so that tests can run the same
recipe at reduced size.
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int, k: int):
    return np.random.default_rng([seed, k])


def bernoulli_matrix(seed: int, m: int, n: int, p: float, sigma=1.0, block_rows: int = 2048):
    """Dense float32 m x n, entries kept iid with probability p, values N(0, sigma^2).

    Yields (row0, block) so that huge matrices never exist densely at once."""
    for b, r0 in enumerate(range(0, m, block_rows)):
        rows = min(block_rows, m - r0)
        g = np.random.default_rng([seed, 0, b])
        mask = g.random((rows, n), dtype=np.float32) < p
        vals = g.standard_normal((rows, n), dtype=np.float32)
        if sigma != 1.0:
            vals *= np.float32(sigma)
        vals[~mask] = 0.0
        # v != 0.0f is the encoder's test; a drawn 0.0 value is vanishingly unlikely and harmless
        yield r0, vals


def dense_matrix(seed: int, m: int, n: int, p: float, sigma=1.0):
    W = np.empty((m, n), dtype=np.float32)
    for r0, blk in bernoulli_matrix(seed, m, n, p, sigma):
        W[r0:r0 + blk.shape[0]] = blk
    return W


def csr_from_blocks(blocks, m: int):
    """(rowptr u64, col u32, val f32) from an iterator of (row0, dense block)."""
    rowptr = np.zeros(m + 1, dtype=np.uint64)
    cols, vals = [], []
    for r0, blk in blocks:
        rr, cc = np.nonzero(blk)
        cnt = np.bincount(rr, minlength=blk.shape[0]).astype(np.uint64)
        rowptr[r0 + 1:r0 + 1 + blk.shape[0]] = cnt
        cols.append(cc.astype(np.uint32))
        vals.append(blk[rr, cc])
    np.cumsum(rowptr, out=rowptr)
    col = np.concatenate(cols) if cols else np.zeros(0, np.uint32)
    val = np.concatenate(vals) if vals else np.zeros(0, np.float32)
    return rowptr, col, val


def bernoulli_csr(seed: int, m: int, n: int, p: float, sigma=1.0, block_rows: int = 1024):
    """CSR of an m x n matrix whose entries are kept iid with probability p, values N(0, sigma^2).
    The keep mask is drawn block by block (the dense matrix never exists), each block from its own
    stream so the blocks can be drawn by a few host threads; values only for the kept entries."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    def block(b):
        r0 = b * block_rows
        rows = min(block_rows, m - r0)
        g = np.random.default_rng([seed, 7, b])
        keep = np.flatnonzero(g.random(rows * n, dtype=np.float32) < np.float32(p))
        rr = keep // n
        v = g.standard_normal(len(keep), dtype=np.float32)
        if sigma != 1.0:
            v *= np.float32(sigma)
        return (keep - rr * n).astype(np.uint32), np.bincount(rr, minlength=rows).astype(np.uint64), v

    nblocks = (m + block_rows - 1) // block_rows
    workers = max(1, min(16, os.cpu_count() or 1, nblocks))
    with ThreadPoolExecutor(workers) as ex:
        parts = list(ex.map(block, range(nblocks)))
    rowptr = np.zeros(m + 1, dtype=np.uint64)
    for b, (_, cnt, _) in enumerate(parts):
        rowptr[b * block_rows + 1:b * block_rows + 1 + len(cnt)] = cnt
    np.cumsum(rowptr, out=rowptr)
    col = np.concatenate([p_[0] for p_ in parts]) if parts else np.zeros(0, np.uint32)
    val = np.concatenate([p_[2] for p_ in parts]) if parts else np.zeros(0, np.float32)
    return rowptr, col, val


def csr_to_ell(m: int, rowptr, col, val):
    """Padded (Wd, idx, nnz) in the reference's host layout from CSR."""
    nnz = np.diff(rowptr).astype(np.uint32)
    r = int(nnz.max()) if m else 0
    Wd = np.zeros((m, r), dtype=np.float32)
    idx = np.zeros((m, r), dtype=np.uint32)
    if r:
        rows = np.repeat(np.arange(m, dtype=np.int64), nnz)
        pos = np.arange(len(col), dtype=np.int64) - np.repeat(rowptr[:-1].astype(np.int64), nnz)
        Wd[rows, pos] = val
        idx[rows, pos] = col
    return Wd, idx, nnz


# ---- config 1: SpMM / SpMV 4096^2, p = 0.1, C = 256 ------------------------------------------
def cfg1(scale: float = 1.0, seed: int = 42):
    m = n = max(16, int(4096 * scale))
    C = max(4, int(256 * scale))
    W = dense_matrix(seed, m, n, 0.1)
    X = _rng(seed, 1).uniform(-1, 1, (n, C)).astype(np.float32)
    bias = _rng(seed, 2).standard_normal(m).astype(np.float32)
    x = _rng(seed, 3).uniform(-1, 1, n).astype(np.float32)
    return dict(W=W, X=X, bias=bias, x=x, m=m, n=n, C=C)


# ---- config 2: SpMV sweep ----------------------------------------------------------------------
CFG2_SIZES = (4096, 16384, 65536)
CFG2_SPARSITIES = (0.80, 0.90, 0.95, 0.99)


def cfg2_case(size: int, sparsity: float, seed: int = 43):
    """CSR of a square iid-sparse matrix with values N(0, sigma), sigma = 1/sqrt(mean nnz per row)."""
    p = 1.0 - sparsity
    sigma = 1.0 / np.sqrt(max(1.0, p * size))
    case_seed = seed + CFG2_SIZES.index(size) * len(CFG2_SPARSITIES) + CFG2_SPARSITIES.index(sparsity) \
        if size in CFG2_SIZES and sparsity in CFG2_SPARSITIES else seed
    rowptr, col, val = bernoulli_csr(case_seed, size, size, p, sigma)
    x = _rng(case_seed, 1).uniform(-1, 1, size).astype(np.float32)
    bias = _rng(case_seed, 2).standard_normal(size).astype(np.float32)
    return dict(m=size, n=size, rowptr=rowptr, col=col, val=val, x=x, bias=bias)


# ---- config 3: sparse MLP 4096-4096-4096-4096-1000, 90 % sparse, batch 256 ---------------------
def cfg3(scale: float = 1.0, seed: int = 44, batch: int | None = None):
    dims = [max(8, int(d * scale)) for d in (4096, 4096, 4096, 4096, 1000)]
    B = batch if batch is not None else max(4, int(256 * scale))
    Ws, bs = [], []
    for l in range(4):
        fan_in = dims[l]
        Ws.append(dense_matrix(seed * 100 + l, dims[l + 1], dims[l], 0.1, sigma=np.sqrt(2.0 / fan_in)))
        bs.append(np.zeros(dims[l + 1], dtype=np.float32))
    x = _rng(seed, 9).uniform(0, 1, (B, dims[0])).astype(np.float32)
    acts = ["Relu", "Relu", "Relu", "Sigmoid"]
    return dict(dims=dims, B=B, weights=Ws, biases=bs, acts=acts, x=x)


# ---- config 4: sparse 3x3 conv 256->256 on 56x56, batch 32, 80 % sparse ------------------------
def cfg4(scale: float = 1.0, seed: int = 45, layers: int = 1, density: float = 0.2):
    Cc = max(4, int(256 * scale))
    H = W = max(6, int(56 * scale))
    B = max(2, int(32 * scale))
    ws, bs = [], []
    for l in range(layers):
        g = _rng(seed, 10 + l)
        w = g.standard_normal((Cc, Cc, 3, 3), dtype=np.float32) * np.float32(np.sqrt(2.0 / (9 * Cc)))
        w[g.random((Cc, Cc, 3, 3), dtype=np.float32) >= np.float32(density)] = 0.0
        ws.append(w)
        bs.append(_rng(seed, 20 + l).standard_normal(Cc).astype(np.float32))
    x = _rng(seed, 1).standard_normal((B, Cc, H, W), dtype=np.float32)
    return dict(weights=ws, biases=bs, x_nchw=x, B=B, C=Cc, H=H, W=W)


# ---- config 5: skewed SpMM 262144 x 65536, power-law row lengths (mean 64, max 2048), C = 1024 --
def powerlaw_pmf(kmax: int, mean: float):
    """P(k) ~ k^-alpha on 1..kmax with alpha solved (bisection) for the requested mean."""
    k = np.arange(1, kmax + 1, dtype=np.float64)
    lo, hi = 0.0, 4.0
    for _ in range(80):
        a = 0.5 * (lo + hi)
        w = k ** (-a)
        mu = float((k * w).sum() / w.sum())
        if mu > mean:
            lo = a
        else:
            hi = a
    w = k ** (-0.5 * (lo + hi))
    return w / w.sum()


def cfg5_rows(row0: int, rows: int, n: int = 65536, kmax: int = 2048, mean: float = 64.0,
              seed: int = 46, block_rows: int = 4096, force_max_row: int | None = 0):
    """CSR (rowptr, col, val) of rows [row0, row0+rows) of the skewed matrix.

    Generation is per block of `block_rows` rows with its own stream, so any row range (a rank's
    shard) reproduces the same rows as the whole matrix.  Column ids: the row's drawn length worth
    of uniform samples, sorted, duplicates dropped (so a row's final length can be slightly below
    the drawn one); row `force_max_row` gets exactly kmax distinct columns so that r == kmax."""
    assert row0 % block_rows == 0
    kmax = min(kmax, n)
    pmf = powerlaw_pmf(kmax, min(mean, kmax / 2))
    rowptr = [np.zeros(1, dtype=np.uint64)]
    cols, vals = [], []
    base = 0
    for b0 in range(row0, row0 + rows, block_rows):
        nb = min(block_rows, row0 + rows - b0)
        g = np.random.default_rng([seed, b0 // block_rows])
        k = g.choice(kmax, size=block_rows, p=pmf)[:nb] + 1
        rid = np.repeat(np.arange(nb, dtype=np.int64), k)
        c = g.integers(0, n, size=int(k.sum()), dtype=np.int64)
        if force_max_row is not None and b0 <= force_max_row < b0 + nb:
            # replace that row by kmax distinct columns
            loc = force_max_row - b0
            keep = rid != loc
            rid = np.concatenate([rid[keep], np.full(kmax, loc, dtype=np.int64)])
            c = np.concatenate([c[keep], g.choice(n, size=kmax, replace=False).astype(np.int64)])
        key = np.unique(rid * n + c)            # sorts by (row, col) and drops duplicates
        rid_u = key // n
        col = (key - rid_u * n).astype(np.uint32)
        cnt = np.bincount(rid_u, minlength=nb).astype(np.uint64)
        val = g.standard_normal(len(col), dtype=np.float32)
        rowptr.append(np.cumsum(cnt) + np.uint64(base))
        base += len(col)
        cols.append(col)
        vals.append(val)
    return (np.concatenate(rowptr).astype(np.uint64),
            np.concatenate(cols) if cols else np.zeros(0, np.uint32),
            np.concatenate(vals) if vals else np.zeros(0, np.float32))


def cfg5_dense_operand(n: int, C: int, seed: int = 46):
    return _rng(seed, 1_000_003).uniform(-1, 1, (n, C)).astype(np.float32)
