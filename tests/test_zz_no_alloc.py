"""GPU: the allocation-free convolution entry point `spx_conv2d_static`.

Some callers of this library cannot allocate device memory while they run: a server that handed
the whole GPU to its own memory pool at start-up, or a serving loop that cannot tolerate the
device-wide synchronisation an allocation may bring.  For them the library offers a variant of
the convolution whose tap table lives in a fixed array inside the library instead of a buffer
allocated on first use.  This test calls it through the C ABI twice in a row (the array is
shared between calls and keeps the previous contents, so the second call, with a different
weight matrix and kernel shape, must not be disturbed by what the first one left) and requires
results bit-identical to `spx_conv2d`, the bar all convolution tests here use.  It also checks
that a weight matrix larger than the fixed table is refused with a clear error, and that the
amount of free device memory is the same before and after a call -- the property the entry point
exists for.

The file name sorts last so that a run stopping at the first failure has already run every
other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import spx_ctypes as sx
from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu


def _case(seed, B, Cin, Cout, H, W, k, pad, layout, density):
    rng = np.random.default_rng(seed)
    wt = (rng.standard_normal((Cout, Cin * k * k)) * 0.3).astype(np.float32)
    wt[rng.random(wt.shape) >= density] = 0
    bias = rng.standard_normal(Cout).astype(np.float32)
    x = rng.standard_normal((B, Cin, H, W)).astype(np.float32)
    src = np.ascontiguousarray(x.transpose(1, 2, 3, 0)) if layout == sx.LAYOUT_PF else x
    return wt, bias, src


def test_static_conv_matches_allocating_conv_twice(lib, orc, cuda):
    cases = [(1, 4, 8, 16, 12, 10, 3, 1, sx.LAYOUT_PF, 0.3), (2, 3, 6, 9, 9, 11, 5, 2, sx.LAYOUT_NCHW, 0.5)]
    for seed, B, Cin, Cout, H, W, k, pad, layout, density in cases:
        wt, bias, src = _case(seed, B, Cin, Cout, H, W, k, pad, layout, density)
        E = orc.encode(wt)
        h = lib.ell_create(E.Wd, E.idx, E.nnz, E.n)
        g = sx.conv_geom(Cin, Cout, k, k, H, W, pH=pad, pW=pad)
        shape = (Cout, g.Ho, g.Wo, B) if layout == sx.LAYOUT_PF else (B, Cout, g.Ho, g.Wo)
        dX = torch.from_numpy(src).to(cuda)
        dB = torch.from_numpy(bias).to(cuda)
        want = torch.full(shape, float("nan"), device=cuda, dtype=torch.float32)
        got = torch.full(shape, float("nan"), device=cuda, dtype=torch.float32)
        h.conv2d(g, layout, dX.data_ptr(), B, dB.data_ptr(), sx.ACT_RELU, want.data_ptr())
        lib.spx_conv2d_static(h.h, C.byref(g), layout, dX.data_ptr(), B, dB.data_ptr(), sx.ACT_RELU, got.data_ptr(), 0)
        torch.cuda.synchronize()
        assert_bit_equal(got.cpu().numpy(), want.cpu().numpy(), f"static conv, case {seed}")
        gd = dict(Cin=Cin, kH=k, kW=k, sH=1, sW=1, pH=pad, pW=pad, dH=1, dW=1, H=H, W=W)
        assert_bit_equal(got.cpu().numpy(), orc.conv2d(E, gd, layout, src, B, bias, 1), f"static conv vs oracle, case {seed}")


def test_static_conv_rejects_oversized_weights(lib, cuda):
    # 4096 output channels x a padded row of 288 slots = 1 179 648 slots > the 1 048 576 the table holds
    Cout, Cin = 4096, 32
    Wd = np.ones((Cout, Cin * 9), np.float32)
    idx = np.tile(np.arange(Cin * 9, dtype=np.uint32), (Cout, 1))
    h = lib.ell_create(Wd, idx, np.full(Cout, Cin * 9, np.uint32), Cin * 9)
    g = sx.conv_geom(Cin, Cout, 3, 3, 4, 4, pH=1, pW=1)
    x = torch.zeros((Cin, 4, 4, 1), device=cuda)
    y = torch.zeros((Cout, 4, 4, 1), device=cuda)
    with pytest.raises(sx.SpxError, match="fixed tap table") as info:
        lib.spx_conv2d_static(h.h, C.byref(g), sx.LAYOUT_PF, x.data_ptr(), 1, 0, sx.ACT_NONE, y.data_ptr(), 0)
    assert info.value.status == 4   # SPX_ERR_LIMIT


def test_static_conv_leaves_free_device_memory_unchanged(lib, orc, cuda):
    """After one warm-up call (the library's device code, with the fixed table, is placed on the GPU
    when it is first used), a further call with another weight matrix and shape takes nothing from
    the device: free memory as the driver reports it is identical before and after."""
    made = []
    for seed, B, Cin, Cout, H, W, k, pad, layout, density in [(5, 2, 4, 8, 8, 8, 3, 1, sx.LAYOUT_PF, 0.4),
                                                             (6, 4, 12, 20, 15, 13, 5, 2, sx.LAYOUT_PF, 0.2)]:
        wt, bias, src = _case(seed, B, Cin, Cout, H, W, k, pad, layout, density)
        E = orc.encode(wt)
        h = lib.ell_create(E.Wd, E.idx, E.nnz, E.n)
        g = sx.conv_geom(Cin, Cout, k, k, H, W, pH=pad, pW=pad)
        dX, dB = torch.from_numpy(src).to(cuda), torch.from_numpy(bias).to(cuda)
        out = torch.full((Cout, g.Ho, g.Wo, B), float("nan"), device=cuda, dtype=torch.float32)
        made.append((h, g, layout, dX, B, dB, out, E, src, bias, (Cin, k, pad, H, W)))
    h, g, layout, dX, B, dB, out = made[0][:7]
    lib.spx_conv2d_static(h.h, C.byref(g), layout, dX.data_ptr(), B, dB.data_ptr(), sx.ACT_RELU, out.data_ptr(), 0)   # warm-up
    torch.cuda.synchronize()
    h, g, layout, dX, B, dB, out, E, src, bias, (Cin, k, pad, H, W) = made[1]
    free_before = torch.cuda.mem_get_info()[0]
    lib.spx_conv2d_static(h.h, C.byref(g), layout, dX.data_ptr(), B, dB.data_ptr(), sx.ACT_RELU, out.data_ptr(), 0)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    gd = dict(Cin=Cin, kH=k, kW=k, sH=1, sW=1, pH=pad, pW=pad, dH=1, dW=1, H=H, W=W)
    assert_bit_equal(out.cpu().numpy(), orc.conv2d(E, gd, layout, src, B, bias, 1), "static conv vs oracle")
