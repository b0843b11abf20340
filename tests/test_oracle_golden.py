"""CPU: the C restatement (oracle/ellpack_oracle.c) against the golden vectors produced by the
unmodified reference binary (tests/golden/make_golden.py).  Integer / index work and the
sequential-FMA kernels must match bit for bit; this is what pins the oracle."""
import numpy as np
import pytest

from conftest import assert_bit_equal
from oracle import EllArrays


@pytest.mark.parametrize("name", ["enc_hand", "enc_special", "enc_zero", "enc_rand"])
def test_encoder_matches_reference(orc, golden, name):
    E = orc.encode(golden[name + "_W"])
    assert E.r == golden[name + "_Wd_ref"].shape[1]
    assert_bit_equal(E.Wd, golden[name + "_Wd_ref"], "Wd")
    assert np.array_equal(E.idx, golden[name + "_idx_ref"])
    assert np.array_equal(E.nnz, golden[name + "_nnz_ref"])
    assert_bit_equal(orc.decode(E), golden[name + "_decoded_ref"], "decode")


def test_encoder_known_answers(orc, golden):
    """The hand matrix of the reference's tests/unit/test_ellpack_encoder.py:51-77."""
    E = orc.encode(golden["enc_hand_W"])
    assert E.Wd.shape == (4, 2)
    assert E.Wd[0, 0] == 1.0 and E.Wd[0, 1] == 2.0 and E.Wd[1, 0] == 3.0 and E.Wd[1, 1] == 0.0 and E.Wd[2, 0] == 4.0
    assert E.idx.tolist() == [[0, 3], [1, 0], [2, 0], [3, 0]]
    # special values: -0.0 dropped, NaN / inf / denormal kept
    S = orc.encode(golden["enc_special_W"])
    assert S.nnz[4] == 0 and S.nnz[5] == 13 and S.r == 13
    assert np.isnan(S.Wd).sum() == 1 and np.isinf(S.Wd).sum() == 1


@pytest.mark.parametrize("name", ["mm_a", "mm_b", "mm_c", "mm_d"])
def test_spmm_spmv_match_reference(orc, golden, name):
    E = orc.encode(golden[name + "_W"])
    X, b, x = golden[name + "_X"], golden[name + "_bias"], golden[name + "_x"]
    assert_bit_equal(orc.spmm(E, X, b), golden[name + "_Y_ref"], "spmm")
    assert_bit_equal(orc.spmm(E, X, b, act=1), golden[name + "_Yrelu_ref"], "spmm+relu")
    assert_bit_equal(orc.spmm(E, X, None), golden[name + "_Ynobias_ref"], "spmm no bias")
    assert_bit_equal(orc.spmv(E, x, b), golden[name + "_y_ref"], "spmv")
    assert_bit_equal(orc.spmv(E, x, None), golden[name + "_ynobias_ref"], "spmv no bias")


@pytest.mark.parametrize("name", ["conv_a", "conv_b", "conv_c", "conv_d", "conv_e"])
def test_conv_matches_reference(orc, golden, name):
    B, Cin, Cout, H, W, k, pad, dil, relu = golden[name + "_geom"].tolist()
    g = dict(Cin=Cin, kH=k, kW=k, sH=1, sW=1, pH=pad, pW=pad, dH=dil, dW=dil, H=H, W=W)
    E = orc.encode(golden[name + "_weight"].reshape(Cout, -1))
    x = golden[name + "_x_nchw"]
    pf = np.ascontiguousarray(x.transpose(1, 2, 3, 0))
    assert_bit_equal(orc.conv2d(E, g, 0, pf, B, golden[name + "_bias"], relu), golden[name + "_pf_ref"], "PF")
    assert_bit_equal(orc.conv2d(E, g, 1, x, B, golden[name + "_bias"], relu), golden[name + "_nchw_ref"], "NCHW")
    # F-major [W,H,C,B]: the bytes conv2d_tiled_im2col_fmajor and conv2d_rbm_fmajor_implicit both produce
    fm = np.ascontiguousarray(x.transpose(3, 2, 1, 0))
    assert_bit_equal(orc.conv2d(E, g, 2, fm, B, golden[name + "_bias"], relu), golden[name + "_fm_ref"], "F-major")


def test_oracle_agrees_with_live_reference(orc, ref):
    """Where the reference binary can run (this host), compare on fresh seeded inputs too."""
    rng = np.random.default_rng(7)
    W = rng.standard_normal((200, 333)).astype(np.float32)
    W[rng.random(W.shape) >= 0.2] = 0
    X = rng.uniform(-1, 1, (333, 48)).astype(np.float32)
    b = rng.standard_normal(200).astype(np.float32)
    Er, Eo = ref.encode(W), orc.encode(W)
    A = Er.arrays()
    assert np.array_equal(A.idx, Eo.idx) and np.array_equal(A.nnz, Eo.nnz)
    assert_bit_equal(A.Wd, Eo.Wd, "Wd")
    assert_bit_equal(orc.spmm(Eo, X, b), ref.matmul(Er, X, b), "spmm")
    assert_bit_equal(orc.spmv(Eo, X[:, 0].copy(), b), ref.matvec(Er, X[:, 0].copy(), b), "spmv")


def test_tolerance_bound_is_meaningful(orc, golden):
    """fp64 evaluation of y stays within 1e-5 * sum|w||x| of the oracle's fp32 result."""
    E = orc.encode(golden["mm_d_W"])
    x, b = golden["mm_d_x"], golden["mm_d_bias"]
    y = orc.spmv(E, x, b)
    y64 = golden["mm_d_W"].astype(np.float64) @ x.astype(np.float64) + b
    assert (np.abs(y - y64) <= 1e-5 * orc.absbound(E, x, b)).all()


def test_pools_match_reference(orc, golden):
    """The reference indexes its pool layers in an older layout; on the same LOGICAL tensor the
    [C,H,W,B] restatement gives bit-identical values."""
    x = golden["pool_x_nchw"]
    pf = np.ascontiguousarray(x.transpose(1, 2, 3, 0))
    mx = orc.maxpool_pf(pf, (3, 3), (2, 2), (1, 1, 1, 1)).transpose(3, 0, 1, 2)
    assert_bit_equal(mx, golden["pool_max_ref"], "maxpool")
    assert_bit_equal(orc.gap_pf(pf).T, golden["pool_gap_ref"], "global average pool")
