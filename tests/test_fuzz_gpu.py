"""GPU: seeded random shapes against the oracle -- odd sizes, ragged tails, every batch-tile width of
the tiled convolution, strides / dilations / asymmetric kernels, both layouts.  Bit-exact bars as in
test_parity_gpu.py (SpMV within tolerance)."""
import numpy as np
import pytest
import torch

import spx_ctypes as sx
from conftest import assert_bit_equal
from test_parity_gpu import SPMV_TOL, dev, gpu_ell, gpu_spmm, gpu_spmv, ptr, sparse

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(24))
def test_spmm_spmv_random_shapes(lib, orc, cuda, seed):
    rng = np.random.default_rng([seed, 101])
    m = int(rng.integers(1, 700))
    n = int(rng.integers(1, 900))
    C = int(rng.choice([1, 2, 3, 4, 7, 8, 12, 16, 28, 32, 36, 60, 64, 68, 100, 128, 132, 255, 256, 300, 516]))
    p = float(rng.choice([0.01, 0.05, 0.2, 0.6, 1.0]))
    W = sparse(rng, m, n, p)
    if m > 3:
        W[rng.integers(0, m)] = 0                      # an empty row
        W[rng.integers(0, m)] = rng.standard_normal(n).astype(np.float32) + 3.0   # a full row
    X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    act = int(rng.integers(0, 2))
    E = orc.encode(W)
    h = gpu_ell(lib, E)
    assert_bit_equal(gpu_spmm(h, X, b, act, cuda, ld_pad=int(rng.choice([0, 0, 1, 4]))), orc.spmm(E, X, b, act=act),
                     f"spmm m={m} n={n} C={C} p={p}")
    x = X[:, 0].copy()
    got = gpu_spmv(h, x, b, cuda)
    assert (np.abs(got - orc.spmv(E, x, b)) <= SPMV_TOL * orc.absbound(E, x, b)).all()


@pytest.mark.parametrize("seed", range(28))
def test_conv_random_geometry(lib, orc, cuda, seed):
    rng = np.random.default_rng([seed, 202])
    B = int(rng.choice([1, 2, 3, 4, 5, 8, 12, 16, 20, 24, 28, 32, 36, 40, 44, 64]))
    Cin, Cout = int(rng.integers(1, 20)), int(rng.integers(1, 40))
    kH, kW = int(rng.choice([1, 2, 3, 5])), int(rng.choice([1, 3, 4]))
    sH, sW = int(rng.choice([1, 1, 2, 3])), int(rng.choice([1, 1, 2]))
    dH, dW = int(rng.choice([1, 1, 2])), int(rng.choice([1, 1, 3]))
    pH, pW = int(rng.integers(0, 3)), int(rng.integers(0, 3))
    H = int(rng.integers(dH * (kH - 1) + 1, dH * (kH - 1) + 14))
    W = int(rng.integers(dW * (kW - 1) + 1, dW * (kW - 1) + 14))
    layout = int(rng.integers(0, 2))
    wt = sparse(rng, Cout, Cin * kH * kW, float(rng.choice([0.1, 0.4, 1.0]))) * np.float32(0.3)
    bias = rng.standard_normal(Cout).astype(np.float32) if rng.random() < 0.8 else None
    x = rng.standard_normal((B, Cin, H, W)).astype(np.float32)
    src = np.ascontiguousarray(x.transpose(1, 2, 3, 0)) if layout == sx.LAYOUT_PF else x
    E = orc.encode(wt)
    gd = dict(Cin=Cin, kH=kH, kW=kW, sH=sH, sW=sW, pH=pH, pW=pW, dH=dH, dW=dW, H=H, W=W)
    act = int(rng.integers(0, 2))
    want = orc.conv2d(E, gd, layout, src, B, bias, act)
    h = gpu_ell(lib, E)
    g = sx.conv_geom(Cin, Cout, kH, kW, H, W, sH, sW, pH, pW, dH, dW)
    dX = dev(src, cuda)
    dB = None if bias is None else dev(bias, cuda)
    dY = torch.full(want.shape, float("nan"), device=cuda, dtype=torch.float32)
    h.conv2d(g, layout, ptr(dX), B, ptr(dB), act, ptr(dY))
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), want, f"conv B={B} {Cin}->{Cout} k={kH}x{kW} s={sH},{sW} d={dH},{dW} p={pH},{pW} {H}x{W} layout={layout}")
    ref = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(wt.reshape(Cout, Cin, kH, kW)),
                                     None if bias is None else torch.from_numpy(bias), stride=(sH, sW), padding=(pH, pW),
                                     dilation=(dH, dW))
    ref = (ref.relu() if act else ref).numpy()
    got = dY.cpu().numpy()
    assert np.abs((got.transpose(3, 0, 1, 2) if layout == sx.LAYOUT_PF else got) - ref).max() <= 2e-4
