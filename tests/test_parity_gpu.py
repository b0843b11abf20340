"""GPU parity tests: the CUDA path, called through the C ABI (ctypes) with device pointers, against
the CPU oracle on the same seeded inputs and against the golden vectors of the reference binary.

Bars: ELLPACK encodings, SpMM and conv outputs bit-exact (a thread owns whole output elements and
runs the reference's FMA chain in storage order); SpMV within 1e-5 * (sum_j |w||x| + |bias|) per
element (the summation order differs from the reference's 16 partial sums); sigmoid / tanh
epilogues within 4 ulp-ish relative 1e-6 of the C library."""
import os

import numpy as np
import pytest
import torch

import spx_ctypes as sx
from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu

SPMV_TOL = 1e-5   # times sum|w||x| + |bias|, stated by the acceptance contract


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def ptr(t):
    return 0 if t is None else t.data_ptr()


def sparse(rng, m, n, p):
    W = rng.standard_normal((m, n)).astype(np.float32)
    W[rng.random((m, n)) >= p] = 0
    return W


def gpu_ell(lib, E):
    return lib.ell_create(E.Wd, E.idx, E.nnz, E.n)


def gpu_spmm(h, X, bias, act, cuda, ld_pad=0):
    n, C = X.shape
    ldx = C + ld_pad
    Xp = np.zeros((n, ldx), np.float32)
    Xp[:, :C] = X
    dX = dev(Xp, cuda)
    dB = None if bias is None else dev(bias, cuda)
    dY = torch.full((h.m, ldx), float("nan"), device=cuda, dtype=torch.float32)
    h.spmm(ptr(dX), C, ldx, ptr(dB), act, ptr(dY), ldx)
    torch.cuda.synchronize()
    return dY.cpu().numpy()[:, :C]


def gpu_spmv(h, x, bias, cuda):
    dx = dev(x, cuda)
    dB = None if bias is None else dev(bias, cuda)
    dy = torch.full((h.m,), float("nan"), device=cuda, dtype=torch.float32)
    h.spmv(ptr(dx), ptr(dB), ptr(dy))
    torch.cuda.synchronize()
    return dy.cpu().numpy()


# ---- golden vectors of the reference binary ---------------------------------------------------
@pytest.mark.parametrize("name", ["mm_a", "mm_b", "mm_c", "mm_d"])
def test_golden_spmm_spmv(lib, orc, golden, cuda, name):
    E = orc.encode(golden[name + "_W"])
    h = gpu_ell(lib, E)
    Wd, idx, nnz = h.download()
    assert_bit_equal(Wd, E.Wd, "Wd round trip")
    assert np.array_equal(idx, E.idx) and np.array_equal(nnz, E.nnz)
    X, b, x = golden[name + "_X"], golden[name + "_bias"], golden[name + "_x"]
    assert_bit_equal(gpu_spmm(h, X, b, sx.ACT_NONE, cuda), golden[name + "_Y_ref"], "spmm")
    assert_bit_equal(gpu_spmm(h, X, b, sx.ACT_RELU, cuda), golden[name + "_Yrelu_ref"], "spmm+relu")
    assert_bit_equal(gpu_spmm(h, X, None, sx.ACT_NONE, cuda), golden[name + "_Ynobias_ref"], "spmm no bias")
    bound = orc.absbound(E, x, b)
    assert (np.abs(gpu_spmv(h, x, b, cuda) - golden[name + "_y_ref"]) <= SPMV_TOL * bound).all()
    assert (np.abs(gpu_spmv(h, x, None, cuda) - golden[name + "_ynobias_ref"]) <= SPMV_TOL * orc.absbound(E, x, None)).all()


@pytest.mark.parametrize("name", ["conv_a", "conv_b", "conv_c", "conv_d", "conv_e"])
def test_golden_conv(lib, orc, golden, cuda, name):
    B, Cin, Cout, H, W, k, pad, dil, relu = golden[name + "_geom"].tolist()
    E = orc.encode(golden[name + "_weight"].reshape(Cout, -1))
    h = gpu_ell(lib, E)
    g = sx.conv_geom(Cin, Cout, k, k, H, W, pH=pad, pW=pad, dH=dil, dW=dil)
    x = golden[name + "_x_nchw"]
    dB = dev(golden[name + "_bias"], cuda)
    for layout, src, want in ((sx.LAYOUT_PF, np.ascontiguousarray(x.transpose(1, 2, 3, 0)), golden[name + "_pf_ref"]),
                              (sx.LAYOUT_NCHW, x, golden[name + "_nchw_ref"]),
                              (sx.LAYOUT_FMAJOR, np.ascontiguousarray(x.transpose(3, 2, 1, 0)), golden[name + "_fm_ref"])):
        dX = dev(src, cuda)
        dY = torch.full(want.shape, float("nan"), device=cuda, dtype=torch.float32)
        h.conv2d(g, layout, ptr(dX), B, ptr(dB), sx.ACT_RELU if relu else sx.ACT_NONE, ptr(dY))
        torch.cuda.synchronize()
        assert_bit_equal(dY.cpu().numpy(), want, f"{name} layout {layout}")


# ---- oracle parity on seeded inputs -----------------------------------------------------------
SPMM_CASES = [
    # (m, n, C, density)  -- the reference's tests/unit/test_matmul.py shapes and more
    (16, 32, 1, 0.7), (16, 32, 10, 0.7), (16, 32, 100, 0.7), (64, 128, 10, 0.5), (128, 256, 20, 0.3),
    (256, 512, 10, 0.1), (1, 1, 1, 1.0), (1, 1000, 1, 0.9), (1000, 1, 1, 0.9), (32, 32, 1, 0.0),
    (10, 10, 1, 1.0), (10, 10, 10, 0.5), (10, 10, 10, 0.1), (20, 20, 10, 0.8), (100, 100, 10, 0.8),
    (1000, 1000, 10, 0.9), (500, 500, 10, 0.95), (2000, 2000, 10, 0.7), (3000, 3000, 10, 0.6),
    (300, 700, 256, 0.1), (257, 129, 260, 0.2), (64, 4096, 128, 0.1), (513, 300, 36, 0.15), (40, 50, 1024, 0.3),
    # widths that are not a multiple of 4: the scalar kernel with 64- and 256-column panels
    (300, 200, 130, 0.2), (129, 333, 255, 0.1), (70, 90, 513, 0.3),
]


@pytest.mark.parametrize("m,n,C,p", SPMM_CASES)
def test_spmm_bit_exact_vs_oracle(lib, orc, cuda, m, n, C, p):
    rng = np.random.default_rng([m, n, C])
    W = sparse(rng, m, n, p)
    X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    assert_bit_equal(gpu_spmm(h, X, b, sx.ACT_NONE, cuda), orc.spmm(E, X, b), "spmm")
    assert_bit_equal(gpu_spmm(h, X, b, sx.ACT_RELU, cuda, ld_pad=4), orc.spmm(E, X, b, act=1), "spmm relu, padded ld")
    assert_bit_equal(gpu_spmm(h, X, None, sx.ACT_NONE, cuda, ld_pad=3), orc.spmm(E, X, None), "spmm odd ld")


@pytest.mark.parametrize("C", [132, 260, 512, 516, 1024])
def test_spmm_long_rows_several_panels(lib, orc, cuda, C):
    """Wide X (several column panels) together with rows of 512 and more stored entries: such rows
    are scheduled first, for all panels, on narrower panels with more gathers in flight.  Every row
    against the oracle, bit for bit."""
    m, n = 2048, 4096
    rng = np.random.default_rng([m, n, C, 9])
    W = sparse(rng, m, n, 0.02)
    for row, cnt in ((3, 600), (700, 512), (701, 511), (1500, 2000), (2047, 4096), (9, 1031)):
        W[row] = 0
        cols = rng.choice(n, cnt, replace=False)
        W[row, cols] = rng.standard_normal(cnt).astype(np.float32)
    X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    assert_bit_equal(gpu_spmm(h, X, b, sx.ACT_NONE, cuda), orc.spmm(E, X, b), "spmm, long rows")
    assert_bit_equal(gpu_spmm(h, X, None, sx.ACT_RELU, cuda, ld_pad=8), orc.spmm(E, X, None, act=1), "spmm relu, padded ld")


def test_config5_headline_shape_vs_oracle(lib, orc, cuda):
    """The shape the benchmark's headline line times, on the first 4096 rows of the same matrix:
    n = 65536, C = 1024 (four 256-column panels) and the forced 2048-entry row.  The oracle checks
    the long rows and a sample of the others, bit for bit; the rest through additivity over two
    half shards."""
    import workloads as wl
    from oracle import EllArrays
    rows, n, C = 4096, 65536, 1024
    rowptr, col, val = wl.cfg5_rows(0, rows, n=n)
    h = lib.ell_create_csr(rows, n, rowptr, col, val)
    assert h.r == 2048
    X = wl.cfg5_dense_operand(n, C)
    dX = dev(X, cuda)
    dY = torch.full((rows, C), float("nan"), device=cuda, dtype=torch.float32)
    h.spmm(dX.data_ptr(), C, C, 0, sx.ACT_NONE, dY.data_ptr(), C)
    torch.cuda.synchronize()
    got = dY.cpu().numpy()
    Wd, idx, nnz = wl.csr_to_ell(rows, rowptr, col, val)
    longest = np.argsort(nnz)[::-1][:24]
    pick = np.unique(np.concatenate([longest, np.arange(0, rows, 97), [rows - 1]]))
    assert nnz[pick].max() == 2048 and (nnz[pick] >= 512).sum() >= 8
    sub = EllArrays(len(pick), n, Wd.shape[1], Wd[pick], idx[pick], nnz[pick])
    assert_bit_equal(got[pick], orc.spmm(sub, X, None), "config 5 headline shape, sampled rows")
    half = rows // 2
    for g in range(2):
        lo, hi = int(rowptr[g * half]), int(rowptr[(g + 1) * half])
        hg = lib.ell_create_csr(half, n, rowptr[g * half:(g + 1) * half + 1] - rowptr[g * half], col[lo:hi], val[lo:hi])
        out = torch.empty((half, C), device=cuda, dtype=torch.float32)
        hg.spmm(dX.data_ptr(), C, C, 0, sx.ACT_NONE, out.data_ptr(), C)
        torch.cuda.synchronize()
        assert_bit_equal(out.cpu().numpy(), got[g * half:(g + 1) * half], f"half shard {g}")


@pytest.mark.parametrize("C", [64, 260, 1024])
def test_spmm_bcast_into_two_buffers_long_rows(lib, orc, cuda, C):
    """The SpMM whose epilogue stores every finished row into several full-size buffers (the fused
    exchange of the row-sharded path), here with two buffers on one GPU, a row offset, and rows of
    512 and more entries: with more than one destination the rows behind the long ones run shortest
    first.  Both buffers against the oracle, bit for bit; rows outside the shard stay untouched."""
    import ctypes as Ct
    m, n, row0, total = 1500, 3000, 200, 2000
    rng = np.random.default_rng([C, 77])
    W = sparse(rng, m, n, 0.01)
    for row, cnt in ((0, 700), (1, 513), (600, 3000), (1499, 1024)):
        W[row] = 0
        cols = rng.choice(n, cnt, replace=False)
        W[row, cols] = rng.standard_normal(cnt).astype(np.float32)
    X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    dX, dB = dev(X, cuda), dev(b, cuda)
    bufs = [torch.full((total, C), float("nan"), device=cuda, dtype=torch.float32) for _ in range(2)]
    arr = (Ct.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    lib.spx_spmm_bcast(h.h, dX.data_ptr(), C, C, dB.data_ptr(), sx.ACT_RELU, arr, 2, row0, C, 0)
    torch.cuda.synchronize()
    want = orc.spmm(E, X, b, act=1)
    for i, buf in enumerate(bufs):
        got = buf.cpu().numpy()
        assert_bit_equal(got[row0:row0 + m], want, f"buffer {i}")
        assert np.isnan(got[:row0]).all() and np.isnan(got[row0 + m:]).all()


@pytest.mark.parametrize("C,slices,self_index", [(64, 3, 0), (260, 7, 1), (1024, 0, 0), (96, 16, 1)])
def test_spmm_exchange_slices_into_two_buffers(lib, orc, cuda, C, slices, self_index):
    """The SpMM in row slices whose finished slices the copy engines send to the other buffers
    (the row-sharded exchange), here with two buffers on one GPU, a row offset and rows of 512 and
    more entries; slices = 0 is the default of 4.  Both buffers against the oracle, bit for bit;
    rows outside the shard stay untouched.  A second call with another slice count rebuilds the
    slices; one buffer alone (no copies) works too."""
    import ctypes as Ct
    m, n, row0, total = 1500, 3000, 200, 2000
    rng = np.random.default_rng([C, 78])
    W = sparse(rng, m, n, 0.01)
    for row, cnt in ((0, 700), (1, 513), (600, 3000), (1499, 1024)):
        W[row] = 0
        cols = rng.choice(n, cnt, replace=False)
        W[row, cols] = rng.standard_normal(cnt).astype(np.float32)
    X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    dX, dB = dev(X, cuda), dev(b, cuda)
    want = orc.spmm(E, X, b, act=1)
    stream = torch.cuda.current_stream().cuda_stream
    for sl in (slices, 2):
        bufs = [torch.full((total, C), float("nan"), device=cuda, dtype=torch.float32) for _ in range(2)]
        arr = (Ct.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
        lib.spx_spmm_exchange(h.h, dX.data_ptr(), C, C, dB.data_ptr(), sx.ACT_RELU, arr, 2, self_index, row0, C, sl, stream)
        torch.cuda.synchronize()
        for i, buf in enumerate(bufs):
            got = buf.cpu().numpy()
            assert_bit_equal(got[row0:row0 + m], want, f"buffer {i}, {sl} slices")
            assert np.isnan(got[:row0]).all() and np.isnan(got[row0 + m:]).all()
    one = torch.full((total, C), float("nan"), device=cuda, dtype=torch.float32)
    arr1 = (Ct.c_void_p * 1)(one.data_ptr())
    lib.spx_spmm_exchange(h.h, dX.data_ptr(), C, C, dB.data_ptr(), sx.ACT_RELU, arr1, 1, 0, row0, C, 5, stream)
    torch.cuda.synchronize()
    assert_bit_equal(one.cpu().numpy()[row0:row0 + m], want, "one buffer")
    with pytest.raises(sx.SpxError):
        lib.spx_spmm_exchange(h.h, dX.data_ptr(), C, C, dB.data_ptr(), sx.ACT_RELU, arr, 2, 2, row0, C, 4, stream)   # self outside the list
    with pytest.raises(sx.SpxError):
        lib.spx_spmm_exchange(h.h, dX.data_ptr(), C, C, dB.data_ptr(), sx.ACT_RELU, arr, 2, 0, row0, C, 17, stream)  # too many slices


@pytest.mark.parametrize("env", [{"SPX_SPMM_STAGED": "0"}, {"SPX_SPMM_STAGED": "1"}], ids=["gather_vec", "gather_staged"])
def test_spmm_each_wide_kernel_forced(env):
    """Wide X with long rows runs on one of two kernels, chosen by an estimate of whether the longest
    row's chain decides the duration; the switch is read once per process, so each kernel is forced
    in a child process that reruns the SpMM parity cases with long rows (among them the headline
    shape: n = 65536, C = 1024, four panels, the 2048-entry row)."""
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(here, "test_parity_gpu.py"), "-k", "long_rows_several_panels or headline_shape or config5_shard or bcast_into_two_buffers"]
    r = subprocess.run(cmd, env={**os.environ, **env}, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


@pytest.mark.parametrize("act", [sx.ACT_SIGMOID, sx.ACT_TANH])
def test_spmm_sigmoid_tanh_epilogue(lib, orc, cuda, act):
    rng = np.random.default_rng(act)
    W = sparse(rng, 200, 300, 0.1)
    X = rng.uniform(-1, 1, (300, 64)).astype(np.float32)
    b = rng.standard_normal(200).astype(np.float32)
    E = orc.encode(W)
    got = gpu_spmm(gpu_ell(lib, E), X, b, act, cuda)
    want = orc.spmm(E, X, b, act=act)
    # expf / tanhf of CUDA vs glibc differ by a few ulp; outputs are in (-1, 1)
    assert np.abs(got - want).max() <= 4e-7


SPMV_CASES = [(16, 32, 0.7), (64, 128, 0.5), (128, 256, 0.3), (256, 512, 0.1), (1, 1, 1.0), (1, 1000, 0.9),
              (1000, 1, 0.9), (32, 32, 0.0), (10, 10, 1.0), (10, 10, 0.5), (20, 20, 0.8), (100, 100, 0.8),
              (1000, 1000, 0.9), (500, 500, 0.95), (2000, 2000, 0.7), (3000, 3000, 0.6), (4096, 4096, 0.01),
              (300, 20000, 0.05), (70, 70000, 0.02), (50, 210000, 0.01), (20, 450000, 0.002)]


@pytest.mark.parametrize("m,n,p", SPMV_CASES)
def test_spmv_within_tolerance(lib, orc, cuda, m, n, p):
    rng = np.random.default_rng([m, n, 17])
    W = sparse(rng, m, n, p)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    for bias in (b, None):
        got = gpu_spmv(h, x, bias, cuda)
        want = orc.spmv(E, x, bias)
        bound = orc.absbound(E, x, bias)
        assert (np.abs(got - want) <= SPMV_TOL * bound + 0.0).all(), np.abs(got - want).max()
    y64 = W.astype(np.float64) @ x.astype(np.float64) + b
    assert (np.abs(gpu_spmv(h, x, b, cuda) - y64) <= SPMV_TOL * orc.absbound(E, x, b)).all()


def test_padding_is_never_multiplied(lib, orc, cuda):
    """Rows shorter than r: padding slots (Wd=0, idx=0) must not touch X[0], even if it is inf/NaN."""
    rng = np.random.default_rng(5)
    W = sparse(rng, 64, 96, 0.2)
    W[:, 0] = 0.0                       # column 0 is referenced by padding only
    W[3, :] = 1.0
    W[3, 0] = 0.0
    X = rng.uniform(-1, 1, (96, 8)).astype(np.float32)
    X[0, :] = np.inf
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    got = gpu_spmm(h, X, None, sx.ACT_NONE, cuda)
    assert np.isfinite(got).all()
    assert_bit_equal(got, orc.spmm(E, X, None), "spmm with inf in an unreferenced row")
    assert np.isfinite(gpu_spmv(h, X[:, 0].copy(), None, cuda)).all()


def test_empty_and_degenerate_shapes(lib, orc, cuda):
    z = lib.ell_create(np.zeros((0, 0), np.float32), np.zeros((0, 0), np.uint32), np.zeros(0, np.uint32), 0)
    z.spmm(0, 0, 0, 0, sx.ACT_NONE, 0, 0)          # m = 0, C = 0: nothing to do, no error
    z.spmv(0, 0, 0)
    E = orc.encode(np.zeros((8, 5), np.float32))   # r = 0: output is the bias
    h = gpu_ell(lib, E)
    b = np.arange(8, dtype=np.float32)
    X = np.ones((5, 3), np.float32)
    assert_bit_equal(gpu_spmm(h, X, b, sx.ACT_NONE, cuda), np.repeat(b[:, None], 3, 1), "bias only")
    assert_bit_equal(gpu_spmv(h, X[:, 0].copy(), b, cuda), b, "bias only spmv")
    with pytest.raises(sx.SpxError):               # column id out of range is rejected at upload
        lib.ell_create(np.ones((1, 1), np.float32), np.full((1, 1), 9, np.uint32), np.ones(1, np.uint32), 4)
    with pytest.raises(sx.SpxError):
        h.spmm(1, 3, 2, 0, sx.ACT_NONE, 1, 3)      # ldx < C


def test_csr_and_device_encoder(lib, orc, cuda):
    import workloads as wl
    rng = np.random.default_rng(11)
    W = sparse(rng, 300, 1000, 0.05)
    W[7, :] = 0
    W[9, 5] = -0.0
    E = orc.encode(W)
    rowptr, col, val = wl.csr_from_blocks([(0, W)], 300)
    hc = lib.ell_create_csr(300, 1000, rowptr, col, val)
    hd = lib.ell_encode_device(dev(W, cuda).data_ptr(), 300, 1000)
    for h in (hc, hd):
        Wd, idx, nnz = h.download()
        assert h.r == E.r and h.nnz_total == int(E.nnz.sum())
        assert_bit_equal(Wd, E.Wd, "Wd")
        assert np.array_equal(idx, E.idx) and np.array_equal(nnz, E.nnz)
    out = torch.empty((300, 1000), device=cuda, dtype=torch.float32)
    lib.spx_ell_decode_device(hd.h, out.data_ptr(), 0)
    torch.cuda.synchronize()
    assert_bit_equal(out.cpu().numpy(), orc.decode(E), "device decode")


def test_device_encoder_on_a_non_blocking_stream(lib, orc, cuda):
    """spx_ell_encode_device on a stream made by spx_stream_create (non-blocking: not ordered behind
    the default stream): the zero fill of the slabs must be ordered before the pack on that same
    stream.  A slab of about 200 MB per array, so that a fill on another stream would still be
    running when the pack starts; compared with the host encoder's result."""
    import ctypes as C
    m, n = 24000, 4096
    rng = np.random.default_rng(41)
    W = rng.standard_normal((m, n)).astype(np.float32)
    W[rng.random((m, n), dtype=np.float32) >= 0.5] = 0
    dW = dev(W, cuda)
    torch.cuda.synchronize()
    st = C.c_void_p()
    lib.spx_stream_create(C.byref(st))
    try:
        h = lib.ell_encode_device(dW.data_ptr(), m, n, st)
        lib.spx_stream_sync(st)
    finally:
        lib.spx_stream_destroy(st)
    Wd, idx, nnz = h.download()
    cnt = np.count_nonzero(W, axis=1)
    assert h.r == cnt.max() and np.array_equal(nnz, cnt)
    # every row: packed values and ascending column ids, zero padding behind them
    rows = np.concatenate([np.arange(0, m, 997), [m - 1, int(cnt.argmax()), int(cnt.argmin())]])
    for i in rows:
        c = int(cnt[i])
        cols = np.flatnonzero(W[i])
        assert np.array_equal(idx[i, :c], cols) and np.array_equal(Wd[i, :c].view(np.uint32), W[i, cols].view(np.uint32))
    pad = np.arange(h.r)[None, :] >= cnt[:, None]
    assert not Wd[pad].any() and not idx[pad].any()
    sub = orc.encode(W[:512])
    assert np.array_equal(idx[:512, :sub.r], sub.idx) and np.array_equal(Wd[:512, :sub.r].view(np.uint32), sub.Wd.view(np.uint32))


CONV_CASES = [
    # B, Cin, Cout, H, W, k, stride, pad, dil
    (4, 8, 16, 12, 12, 3, 1, 1, 1), (32, 16, 24, 14, 14, 3, 1, 1, 1), (3, 5, 7, 9, 11, 3, 1, 0, 1),
    (8, 16, 8, 10, 10, 1, 1, 0, 1), (2, 6, 6, 13, 9, 5, 1, 2, 1), (4, 8, 8, 12, 12, 3, 2, 1, 1),
    (5, 4, 6, 11, 11, 3, 1, 2, 2), (16, 32, 32, 8, 8, 3, 1, 1, 1), (1, 3, 4, 6, 6, 3, 1, 1, 1),
    # more work units than SMs with a last wave under half full: the tail goes out as half-height tiles
    (32, 8, 64, 56, 56, 3, 1, 1, 1), (32, 8, 64, 54, 50, 3, 1, 1, 1),
    # a last block of output channels that is not full (38 = 9 blocks of 4 + 2), batch tiles of 16 / 8 / 4
    (16, 6, 38, 10, 10, 3, 1, 1, 1), (8, 6, 38, 10, 10, 3, 1, 1, 1), (4, 6, 38, 10, 10, 3, 1, 1, 1),
    # input channels staged in several chunks (the merged kernel double-buffers them): 70 channels
    # end inside a chunk; stride 2, a 5x5 kernel and dilation change the staged patch's extent
    (32, 70, 32, 12, 12, 3, 1, 1, 1), (16, 100, 38, 14, 14, 3, 2, 1, 1), (8, 64, 32, 12, 12, 5, 1, 2, 1),
    (16, 96, 40, 13, 11, 3, 1, 2, 2),
    # batches that the merged kernel runs in segments: 16 + 8, 16 + 4, 8 + 4, 32 + 8 + 4, 16 + 8 + 4
    (24, 12, 40, 10, 10, 3, 1, 1, 1), (20, 40, 32, 9, 12, 3, 1, 1, 1), (12, 8, 36, 10, 10, 3, 2, 1, 1),
    (44, 6, 32, 8, 8, 3, 1, 1, 1), (28, 10, 33, 7, 9, 3, 1, 1, 1),
]


def as_layout(x_nchw, layout):
    """The logical NCHW tensor in the memory order of a layout."""
    perm = {sx.LAYOUT_PF: (1, 2, 3, 0), sx.LAYOUT_NCHW: (0, 1, 2, 3), sx.LAYOUT_FMAJOR: (3, 2, 1, 0)}[layout]
    return np.ascontiguousarray(x_nchw.transpose(perm))


def to_nchw(y, layout):
    perm = {sx.LAYOUT_PF: (3, 0, 1, 2), sx.LAYOUT_NCHW: (0, 1, 2, 3), sx.LAYOUT_FMAJOR: (3, 2, 1, 0)}[layout]
    return y.transpose(perm)


@pytest.mark.parametrize("B,Cin,Cout,H,W,k,s,pad,dil", CONV_CASES)
@pytest.mark.parametrize("layout", [sx.LAYOUT_PF, sx.LAYOUT_NCHW, sx.LAYOUT_FMAJOR])
def test_conv_bit_exact_vs_oracle(lib, orc, cuda, layout, B, Cin, Cout, H, W, k, s, pad, dil):
    rng = np.random.default_rng([B, Cin, Cout, H, k, s])
    wt = sparse(rng, Cout, Cin * k * k, 0.25) * np.float32(0.3)
    bias = rng.standard_normal(Cout).astype(np.float32)
    x = rng.standard_normal((B, Cin, H, W)).astype(np.float32)
    src = as_layout(x, layout)
    E = orc.encode(wt)
    gd = dict(Cin=Cin, kH=k, kW=k, sH=s, sW=s, pH=pad, pW=pad, dH=dil, dW=dil, H=H, W=W)
    want = orc.conv2d(E, gd, layout, src, B, bias, 1)
    h = gpu_ell(lib, E)
    g = sx.conv_geom(Cin, Cout, k, k, H, W, s, s, pad, pad, dil, dil)
    dX, dB = dev(src, cuda), dev(bias, cuda)
    dY = torch.full(want.shape, float("nan"), device=cuda, dtype=torch.float32)
    h.conv2d(g, layout, ptr(dX), B, ptr(dB), sx.ACT_RELU, ptr(dY))
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), want, "conv")
    # and against a dense fp32 convolution (mathematical check, independent of the ELLPACK chain)
    ref = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(wt.reshape(Cout, Cin, k, k)),
                                     torch.from_numpy(bias), stride=s, padding=pad, dilation=dil).relu().numpy()
    assert np.abs(to_nchw(dY.cpu().numpy(), layout) - ref).max() <= 1e-4


@pytest.mark.parametrize("layout", [sx.LAYOUT_PF, sx.LAYOUT_NCHW, sx.LAYOUT_FMAJOR])
def test_conv_unsorted_columns(lib, orc, cuda, layout):
    """Raw ELLPACK arrays may store a row's columns in any order (spx_ell_create only checks the range).
    The tiled kernels need ascending columns; such a handle must take the general kernel and still
    apply the FMAs in storage order, like the CPU restatement does."""
    B, Cin, Cout, H, W, k = 16, 16, 12, 10, 10, 3
    rng = np.random.default_rng(77)
    wt = sparse(rng, Cout, Cin * k * k, 0.3) * np.float32(0.3)
    E = orc.encode(wt)
    for i in range(E.m):                                  # shuffle every row's stored entries
        c = int(E.nnz[i])
        perm = rng.permutation(c)
        E.Wd[i, :c] = E.Wd[i, :c][perm]
        E.idx[i, :c] = E.idx[i, :c][perm]
    bias = rng.standard_normal(Cout).astype(np.float32)
    x = rng.standard_normal((B, Cin, H, W)).astype(np.float32)
    src = as_layout(x, layout)
    gd = dict(Cin=Cin, kH=k, kW=k, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
    want = orc.conv2d(E, gd, layout, src, B, bias, 1)
    h = gpu_ell(lib, E)
    g = sx.conv_geom(Cin, Cout, k, k, H, W, 1, 1, 1, 1, 1, 1)
    dX, dB = dev(src, cuda), dev(bias, cuda)
    dY = torch.full(want.shape, float("nan"), device=cuda, dtype=torch.float32)
    h.conv2d(g, layout, ptr(dX), B, ptr(dB), sx.ACT_RELU, ptr(dY))
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), want, "conv, unsorted columns")


@pytest.mark.parametrize("env", [{"SPX_CONV_RBM": "0"}, {"SPX_CONV_RBM_MIN_SHARE": "0"},
                                 {"SPX_CONV_RBM_MIN_SHARE": "0", "SPX_CONV_TMA": "0"}, {"SPX_CONV_DIRECT": "1"}],
                         ids=["per-row-tiles", "row-block-merged", "row-block-merged-cp-async", "direct"])
def test_conv_each_kernel_forced(env):
    """The library picks a convolution kernel from batch size and density; the switches are read
    once per process, so each kernel is forced in a child process that reruns the conv parity cases."""
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(here, "test_parity_gpu.py"), os.path.join(here, "test_fuzz_gpu.py"),
           "-k", "conv_bit_exact or conv_random or golden_conv"]
    r = subprocess.run(cmd, env={**os.environ, **env}, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_conv_bulk_copy_timeout_child(lib, orc, cuda):
    """Body of test_conv_bulk_copy_timeout_is_reported; needs the switch set before the library loads."""
    if os.environ.get("SPX_CONV_TMA_TEST_TIMEOUT") != "1":
        pytest.skip("runs in a child process of test_conv_bulk_copy_timeout_is_reported")
    B, Cin, Cout, H, W, k = 16, 40, 32, 12, 12, 3          # merged kernel, several channel chunks
    rng = np.random.default_rng(5)
    wt = sparse(rng, Cout, Cin * k * k, 0.25) * np.float32(0.3)
    bias = rng.standard_normal(Cout).astype(np.float32)
    x = rng.standard_normal((B, Cin, H, W)).astype(np.float32)
    src = as_layout(x, sx.LAYOUT_PF)
    E = orc.encode(wt)
    gd = dict(Cin=Cin, kH=k, kW=k, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
    want = orc.conv2d(E, gd, sx.LAYOUT_PF, src, B, bias, 1)
    h = gpu_ell(lib, E)
    g = sx.conv_geom(Cin, Cout, k, k, H, W, 1, 1, 1, 1, 1, 1)
    dX, dB = dev(src, cuda), dev(bias, cuda)
    dY = torch.full(want.shape, float("nan"), device=cuda, dtype=torch.float32)
    # 1st call: enqueued fine; on the GPU the barrier expects 16 bytes that never come, the wait
    # gives up after a second and the kernel raises the handle's status word
    h.conv2d(g, sx.LAYOUT_PF, ptr(dX), B, ptr(dB), sx.ACT_RELU, ptr(dY))
    torch.cuda.synchronize()                               # the context is still usable
    # 2nd call: reports it, once
    with pytest.raises(sx.SpxError) as err:
        h.conv2d(g, sx.LAYOUT_PF, ptr(dX), B, ptr(dB), sx.ACT_RELU, ptr(dY))
    assert err.value.status == 2 and "bulk tensor copy" in str(err.value)
    # 3rd call: the handle stages with per-thread copies from here on, results are right again
    dY.fill_(float("nan"))
    h.conv2d(g, sx.LAYOUT_PF, ptr(dX), B, ptr(dB), sx.ACT_RELU, ptr(dY))
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), want, "conv after the reported timeout")


def test_conv_bulk_copy_timeout_is_reported():
    """The merged kernel's wait for its bulk tensor copies is bounded.  With the test switch the
    barrier expects more bytes than the copy delivers, so the wait runs out (nothing faults, nothing
    hangs): the kernel returns, the next call on the handle fails with SPX_ERR_CUDA, the one after
    works and is bit-exact."""
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(here, "test_parity_gpu.py"), "-k", "bulk_copy_timeout_child"]
    env = {**os.environ, "SPX_CONV_TMA_TEST_TIMEOUT": "1", "SPX_CONV_RBM_MIN_SHARE": "0"}
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "1 passed" in r.stdout, r.stdout[-3000:] + r.stderr[-2000:]


def test_conv_rejects_bad_geometry(lib, orc, cuda):
    E = orc.encode(np.ones((4, 18), np.float32))
    h = gpu_ell(lib, E)
    g = sx.conv_geom(2, 4, 3, 3, 8, 8, pH=1, pW=1)
    g.Ho += 1
    with pytest.raises(sx.SpxError):
        h.conv2d(g, sx.LAYOUT_PF, 1, 1, 0, 0, 1)
    g = sx.conv_geom(3, 4, 3, 3, 8, 8)            # Cin*9 != E.n
    with pytest.raises(sx.SpxError):
        h.conv2d(g, sx.LAYOUT_PF, 1, 1, 0, 0, 1)


@pytest.mark.parametrize("op,fn", [(sx.OP_RELU, lambda a, b: np.maximum(a, 0)), (sx.OP_ADD, lambda a, b: a + b)])
@pytest.mark.parametrize("count", [1, 7, 1024, 100003])
def test_eltwise_exact(lib, cuda, op, fn, count):
    rng = np.random.default_rng(count)
    a = rng.standard_normal(count).astype(np.float32)
    b = rng.standard_normal(count).astype(np.float32)
    da, db = dev(a, cuda), dev(b, cuda)
    out = torch.empty(count, device=cuda, dtype=torch.float32)
    lib.spx_eltwise(op, da.data_ptr(), db.data_ptr(), out.data_ptr(), count, 0)
    torch.cuda.synchronize()
    assert_bit_equal(out.cpu().numpy(), fn(a, b).astype(np.float32), "eltwise")
    lib.spx_eltwise(op, da.data_ptr(), db.data_ptr(), da.data_ptr(), count, 0)   # in place
    torch.cuda.synchronize()
    assert_bit_equal(da.cpu().numpy(), fn(a, b).astype(np.float32), "eltwise in place")


def test_eltwise_sigmoid_tanh(lib, orc, cuda):
    a = np.linspace(-12, 12, 5001).astype(np.float32)
    for op, act in ((sx.OP_SIGMOID, 2), (sx.OP_TANH, 3)):
        da = dev(a, cuda)
        out = torch.empty_like(da)
        lib.spx_eltwise(op, da.data_ptr(), 0, out.data_ptr(), a.size, 0)
        torch.cuda.synchronize()
        assert np.abs(out.cpu().numpy() - orc.activation(a, act)).max() <= 4e-7


def test_host_buffer_entry_points(lib, orc, cuda):
    rng = np.random.default_rng(23)
    W = sparse(rng, 500, 400, 0.1)
    X = rng.uniform(-1, 1, (400, 48)).astype(np.float32)
    b = rng.standard_normal(500).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    assert_bit_equal(h.spmm_host(X, b), orc.spmm(E, X, b), "spmm_host")
    assert_bit_equal(h.spmm_host(X, None, sx.ACT_RELU), orc.spmm(E, X, None, act=1), "spmm_host relu")
    y = h.spmv_host(X[:, 0].copy(), b)
    assert (np.abs(y - orc.spmv(E, X[:, 0].copy(), b)) <= SPMV_TOL * orc.absbound(E, X[:, 0].copy(), b)).all()
    before = lib.spx_launch_count()
    h.spmm_host(X, b)
    assert lib.spx_launch_count() == before + 1


def test_sharded_host_entry_point_without_a_communicator(lib, orc, cuda):
    """spx_spmm_host_sharded with no communicator (one process, one GPU) is spx_spmm_host: same
    bytes out, stage times reported as zero."""
    import ctypes as C
    rng = np.random.default_rng(29)
    W = sparse(rng, 300, 200, 0.1)
    X = rng.uniform(-1, 1, (200, 40)).astype(np.float32)
    b = rng.standard_normal(300).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    Y = np.full((300, 40), np.nan, np.float32)
    phases = (C.c_float * 4)(1, 1, 1, 1)
    fp = lambda a: a.ctypes.data_as(C.c_void_p)
    lib.spx_spmm_host_sharded(None, h.h, fp(X), 40, fp(b), sx.ACT_RELU, fp(Y), phases)
    assert_bit_equal(Y, orc.spmm(E, X, b, act=1), "sharded entry point, world of one")
    assert list(phases) == [0.0, 0.0, 0.0, 0.0]
    with pytest.raises(sx.SpxError):
        lib.spx_spmm_host_sharded(None, None, fp(X), 40, fp(b), sx.ACT_RELU, fp(Y), None)


def test_config1_scaled_and_linearity(lib, orc, cuda):
    """Config 1 recipe at reduced size: oracle parity, plus linearity at the full size where the
    oracle would take too long for a unit test: E(aX1 + X2) == a E X1 + E X2 within rounding."""
    import workloads as wl
    d = wl.cfg1(0.25)
    E = orc.encode(d["W"])
    h = gpu_ell(lib, E)
    assert_bit_equal(gpu_spmm(h, d["X"], d["bias"], sx.ACT_NONE, cuda), orc.spmm(E, d["X"], d["bias"]), "cfg1/4")
    full = wl.cfg1(1.0)
    Ef = orc.encode(full["W"])
    hf = gpu_ell(lib, Ef)
    X1 = full["X"]
    X2 = np.roll(X1, 1, axis=0)
    lhs = gpu_spmm(hf, (2.0 * X1 + X2).astype(np.float32), None, sx.ACT_NONE, cuda)
    rhs = 2.0 * gpu_spmm(hf, X1, None, sx.ACT_NONE, cuda) + gpu_spmm(hf, X2, None, sx.ACT_NONE, cuda)
    scale = np.abs(full["W"]).sum(1, keepdims=True) * 3.0
    assert (np.abs(lhs - rhs) <= 1e-5 * scale).all()
    # row 0..63 of the full problem against the oracle (cheap slice of the same matrix)
    sub = orc.encode(full["W"][:64])
    assert_bit_equal(gpu_spmm(gpu_ell(lib, sub), X1, full["bias"][:64], sx.ACT_NONE, cuda),
                     orc.spmm(sub, X1, full["bias"][:64]), "cfg1 rows 0..63")


@pytest.mark.parametrize("B,C,H,W,k,s,pad", [(3, 5, 9, 8, 3, 2, 1), (8, 4, 12, 12, 2, 2, 0), (1, 2, 7, 5, 3, 1, 1), (16, 8, 6, 6, 3, 3, 0)])
def test_pools_bit_exact(lib, orc, golden, cuda, B, C, H, W, k, s, pad):
    rng = np.random.default_rng([B, C, H, W])
    x = golden["pool_x_nchw"] if (B, C, H, W) == (3, 5, 9, 8) else rng.standard_normal((B, C, H, W)).astype(np.float32)
    pf = np.ascontiguousarray(x.transpose(1, 2, 3, 0))
    want = orc.maxpool_pf(pf, (k, k), (s, s), (pad, pad, pad, pad))
    dX = dev(pf, cuda)
    out = torch.full(want.shape, float("nan"), device=cuda, dtype=torch.float32)
    lib.spx_maxpool2d(dX.data_ptr(), C, H, W, B, k, k, s, s, pad, pad, pad, pad, out.data_ptr(), 0)
    gap = torch.full((C, B), float("nan"), device=cuda, dtype=torch.float32)
    lib.spx_global_avgpool(dX.data_ptr(), C, H, W, B, gap.data_ptr(), 0)
    torch.cuda.synchronize()
    assert_bit_equal(out.cpu().numpy(), want, "maxpool")
    assert_bit_equal(gap.cpu().numpy(), orc.gap_pf(pf), "global average pool")
    ref = torch.nn.functional.max_pool2d(torch.from_numpy(x), k, s, pad).numpy()
    assert np.array_equal(out.cpu().numpy().transpose(3, 0, 1, 2), ref)
    if (B, C, H, W) == (3, 5, 9, 8):        # the reference binary's own outputs on this tensor
        assert_bit_equal(out.cpu().numpy().transpose(3, 0, 1, 2), golden["pool_max_ref"], "maxpool vs reference")
        assert_bit_equal(gap.cpu().numpy().T, golden["pool_gap_ref"], "gap vs reference")


def test_config5_shard_skewed_rows_vs_oracle(lib, orc, cuda):
    """The 8-GPU row shard of config 5 (32768 power-law rows, r = 2048, n = 65536) built from CSR,
    against the oracle on a narrower X, plus: two half shards reproduce the whole bit for bit."""
    import workloads as wl
    rows, n, C = 32768, 65536, 64
    rowptr, col, val = wl.cfg5_rows(0, rows, n=n)
    h = lib.ell_create_csr(rows, n, rowptr, col, val)
    assert h.r == 2048 and h.nnz_total == len(col)
    X = wl.cfg5_dense_operand(n, C)
    dX = dev(X, cuda)
    dY = torch.full((rows, C), float("nan"), device=cuda, dtype=torch.float32)
    h.spmm(dX.data_ptr(), C, C, 0, sx.ACT_NONE, dY.data_ptr(), C)
    torch.cuda.synchronize()
    Wd, idx, nnz = wl.csr_to_ell(rows, rowptr, col, val)
    from oracle import EllArrays
    want = orc.spmm(EllArrays(rows, n, Wd.shape[1], Wd, idx, nnz), X, None)
    assert_bit_equal(dY.cpu().numpy(), want, "config 5 shard")
    half = rows // 2
    for g in range(2):
        rp, cc, vv = wl.cfg5_rows(g * half, half, n=n)
        hg = lib.ell_create_csr(half, n, rp, cc, vv)
        out = torch.empty((half, C), device=cuda, dtype=torch.float32)
        hg.spmm(dX.data_ptr(), C, C, 0, sx.ACT_NONE, out.data_ptr(), C)
        torch.cuda.synchronize()
        assert_bit_equal(out.cpu().numpy(), want[g * half:(g + 1) * half], f"half shard {g}")
    # SpMV on the same skewed matrix (long and short rows share warps)
    x = X[:, 0].copy()
    y = gpu_spmv(h, x, None, cuda)
    E = EllArrays(rows, n, Wd.shape[1], Wd, idx, nnz)
    assert (np.abs(y - orc.spmv(E, x, None)) <= SPMV_TOL * orc.absbound(E, x, None)).all()


def test_config4_full_size_subset_vs_oracle(lib, orc, cuda):
    """Config 4 at full size (256 -> 256 channels, 56 x 56, batch 32, 80 % sparse, bias + ReLU) on the
    GPU in both layouts; the oracle checks 6 of the 256 output channels on 8 of the 32 images (the
    scalar CPU restatement needs seconds for that slice, minutes for everything)."""
    import workloads as wl
    d = wl.cfg4(1.0)
    Cc, H, W, B = d["C"], d["H"], d["W"], d["B"]
    wt = d["weights"][0].reshape(Cc, -1)
    E = orc.encode(wt)
    h = gpu_ell(lib, E)
    g = sx.conv_geom(Cc, Cc, 3, 3, H, W, pH=1, pW=1)
    x = d["x_nchw"]
    pf = np.ascontiguousarray(x.transpose(1, 2, 3, 0))
    dB = dev(d["biases"][0], cuda)
    dX = dev(pf, cuda)
    out_pf = torch.full((Cc, H, W, B), float("nan"), device=cuda, dtype=torch.float32)
    h.conv2d(g, sx.LAYOUT_PF, dX.data_ptr(), B, dB.data_ptr(), sx.ACT_RELU, out_pf.data_ptr())
    dXn = dev(x, cuda)
    out_n = torch.full((B, Cc, H, W), float("nan"), device=cuda, dtype=torch.float32)
    h.conv2d(g, sx.LAYOUT_NCHW, dXn.data_ptr(), B, dB.data_ptr(), sx.ACT_RELU, out_n.data_ptr())
    torch.cuda.synchronize()
    got = out_pf.cpu().numpy()
    assert np.isfinite(got).all()
    # both layouts hold the same values
    assert_bit_equal(out_n.cpu().numpy(), got.transpose(3, 0, 1, 2), "NCHW vs [C,H,W,B]")
    rows = [0, 1, 77, 128, 200, 255]
    from oracle import EllArrays
    sub = EllArrays(len(rows), E.n, E.r, E.Wd[rows], E.idx[rows], E.nnz[rows])
    gd = dict(Cin=Cc, kH=3, kW=3, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
    want = orc.conv2d(sub, gd, 0, np.ascontiguousarray(pf[..., :8]), 8, d["biases"][0][rows], 1)
    assert_bit_equal(got[rows][..., :8], want, "config 4 slice")


def test_host_buffer_spmm_pipelined_panels(lib, orc, cuda):
    """Wide, large operands take the panel-pipelined route of spx_spmm_host (three streams, strided
    copies); the result must equal the plain route bit for bit, including a ragged last panel."""
    rng = np.random.default_rng(31)
    m, n, C = 30000, 900, 772            # m*C*4 = 92 MB >= 64 MB, C = 3 panels + 4 columns
    W = sparse(rng, m, n, 0.02)
    X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    got = h.spmm_host(X, b, sx.ACT_RELU)
    assert_bit_equal(got, gpu_spmm(h, X, b, sx.ACT_RELU, cuda), "pipelined host route vs device route")
    assert_bit_equal(got[:500], orc.spmm(oracle_rows(E, 500), X, b[:500], act=1), "first rows vs oracle")


def oracle_rows(E, k):
    from oracle import EllArrays
    return EllArrays(k, E.n, E.r, E.Wd[:k], E.idx[:k], E.nnz[:k])


@pytest.mark.parametrize("name", ["mm_a", "mm_b", "mm_c", "mm_d"])
def test_spmv_reference_order_is_bit_exact(lib, orc, golden, cuda, name):
    """The checking variant of SpMV reproduces the reference binary's result bit for bit."""
    E = orc.encode(golden[name + "_W"])
    h = gpu_ell(lib, E)
    for bias, want in ((golden[name + "_bias"], golden[name + "_y_ref"]), (None, golden[name + "_ynobias_ref"])):
        dx = dev(golden[name + "_x"], cuda)
        dB = None if bias is None else dev(bias, cuda)
        dy = torch.full((h.m,), float("nan"), device=cuda, dtype=torch.float32)
        lib.spx_spmv_reference_order(h.h, ptr(dx), ptr(dB), ptr(dy), 0)
        torch.cuda.synchronize()
        assert_bit_equal(dy.cpu().numpy(), want, "reference-order spmv")
    rng = np.random.default_rng(77)
    W = sparse(rng, 1500, 2100, 0.07)
    x = rng.uniform(-1, 1, 2100).astype(np.float32)
    b = rng.standard_normal(1500).astype(np.float32)
    E2 = orc.encode(W)
    h2 = gpu_ell(lib, E2)
    dy = torch.empty(1500, device=cuda)
    dx2, db2 = dev(x, cuda), dev(b, cuda)
    lib.spx_spmv_reference_order(h2.h, dx2.data_ptr(), db2.data_ptr(), dy.data_ptr(), 0)
    torch.cuda.synchronize()
    assert_bit_equal(dy.cpu().numpy(), orc.spmv(E2, x, b), "reference-order spmv vs oracle")


def test_abi_rejects_misuse_with_status_codes(lib, orc, cuda):
    """Failures are made on the host: every bad call returns a status and a message, nothing is
    launched, and the context stays usable afterwards."""
    import ctypes as C
    E = orc.encode(np.eye(8, dtype=np.float32))
    h = gpu_ell(lib, E)
    hz = gpu_ell(lib, orc.encode(np.zeros((8, 8), np.float32)))
    x = torch.ones(8, device=cuda)
    y = torch.zeros(8, device=cuda)
    before = lib.spx_launch_count()
    arr9 = (C.c_void_p * 9)(*([y.data_ptr()] * 9))
    for call in (
        lambda: lib.spx_spmm(h.h, x.data_ptr(), 1, 1, 0, 7, y.data_ptr(), 1, 0),                   # unknown activation
        lambda: lib.spx_spmm(0, x.data_ptr(), 1, 1, 0, 0, y.data_ptr(), 1, 0),                     # null handle
        lambda: lib.spx_spmm(h.h, x.data_ptr(), 1, 1, 0, 0, 0, 1, 0),                              # null output
        lambda: lib.spx_spmv(h.h, 0, 0, y.data_ptr(), 0),                                          # null x with nonzeros
        lambda: lib.spx_spmv(hz.h, 0, 0, y.data_ptr(), 0),                                         # null x, no nonzeros but n > 0
        lambda: lib.spx_spmv_reference_order(hz.h, 0, 0, y.data_ptr(), 0),
        lambda: lib.spx_spmm_bcast(h.h, x.data_ptr(), 1, 1, 0, 0, arr9, 9, 0, 1, 0),               # more than 8 buffers
        lambda: lib.spx_spmm_bcast(h.h, x.data_ptr(), 1, 1, 0, 0, None, 1, 0, 1, 0),               # null list
        lambda: lib.spx_eltwise(9, x.data_ptr(), 0, y.data_ptr(), 8, 0),                           # unknown op
        lambda: lib.spx_eltwise(sx.OP_ADD, x.data_ptr(), 0, y.data_ptr(), 8, 0),                   # add without b
        lambda: lib.spx_maxpool2d(x.data_ptr(), 1, 2, 2, 2, 3, 3, 1, 1, 0, 0, 0, 0, y.data_ptr(), 0),   # window > input
        lambda: lib.spx_comm_create(3, 2, b"\0" * 128, C.byref(C.c_void_p())),                     # rank >= world
        lambda: lib.spx_allgather_rows(0, y.data_ptr(), 1, 1, 0),                                  # null communicator
        lambda: lib.spx_ipc_export(0, C.create_string_buffer(64)),                                 # null pointer
        lambda: lib.spx_graph_capture_begin(0),                                                    # default stream
        lambda: lib.spx_ell_create_csr(2, 4, np.array([0, 2, 1], np.uint64).ctypes.data_as(C.c_void_p), 0, 0, C.byref(C.c_void_p())),
    ):
        with pytest.raises(sx.SpxError) as info:
            call()
        assert info.value.status in (1, 2, 4, 5) and str(info.value)
    assert lib.spx_launch_count() == before
    # unsorted CSR columns are refused too
    with pytest.raises(sx.SpxError, match="ascending"):
        lib.ell_create_csr(1, 4, np.array([0, 2], np.uint64), np.array([3, 1], np.uint32), np.ones(2, np.float32))
    h.spmv(x.data_ptr(), 0, y.data_ptr())              # still works
    torch.cuda.synchronize()
    assert y.cpu().numpy().tolist() == [1.0] * 8


def test_l2_gather_probe_runs(cuda):
    """The benchmark's measurement aid (its own small library) reads what it reports and leaves the sink alone."""
    import ctypes

    import bench
    probe = bench.load_probe()
    assert probe is not None, "libspx_bench_probe.so is missing: run sparse-ops_b200/build_cuda.sh"
    buf = torch.zeros(8 << 20, dtype=torch.uint8, device=cuda)
    sink = torch.full((1,), 7.0, dtype=torch.float32, device=cuda)
    n = ctypes.c_uint64(0)
    assert probe(buf.data_ptr(), 8 << 20, 4, sink.data_ptr(), 0, ctypes.byref(n)) == 0
    torch.cuda.synchronize()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert n.value == sms * 8 * 8 * 4 * 8 * 512 and float(sink.item()) == 7.0
    assert probe(buf.data_ptr(), 512, 4, sink.data_ptr(), 0, ctypes.byref(n)) == -1
