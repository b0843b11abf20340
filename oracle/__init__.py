"""CPU checkers for the ELLPACK hot path -- TEST INFRASTRUCTURE ONLY.

Two libraries, both driven through ctypes with numpy arrays:

* ``Oracle``  -- ``oracle/liboracle.so``, the plain-C restatement in ``ellpack_oracle.c``.
* ``Reference`` -- ``oracle/_ref/libsparseops_ref.so``, the reference project's own C++
  sources compiled unchanged (see ``oracle/Makefile``) behind ``ref_shim.cpp``.

Only the tests, the smoke test and the CPU-baseline / reference arm of the benchmark may
import this package; the product library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libsparseops_ref.so")

_f32p = C.POINTER(C.c_float)
_u32p = C.POINTER(C.c_uint32)
_u16p = C.POINTER(C.c_uint16)
_f64p = C.POINTER(C.c_double)
_u64p = C.POINTER(C.c_uint64)


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _up(a):
    return None if a is None else a.ctypes.data_as(_u32p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def build(ref: bool = True) -> None:
    """Run ``make`` in this directory (the reference is only built when its sources exist)."""
    subprocess.run(["make", "-s", "-C", _HERE, "liboracle.so"] + (["ref"] if ref else []), check=True)


def cpu_has_avx512() -> bool:
    """The reference build uses AVX-512F/DQ instructions unconditionally."""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    return {"avx512f", "avx512dq", "avx512bw", "avx512vl", "avx512cd"} <= flags
    except OSError:
        pass
    return False


def reference_available() -> bool:
    return os.path.exists(REF_SO) and cpu_has_avx512()


class EllArrays:
    """ELLPACK arrays in the reference's host layout: Wd/idx are (m, r) row-major."""

    def __init__(self, m, n, r, Wd, idx, nnz):
        self.m, self.n, self.r = int(m), int(n), int(r)
        self.Wd = np.ascontiguousarray(Wd, dtype=np.float32).reshape(self.m, self.r)
        self.idx = np.ascontiguousarray(idx, dtype=np.uint32).reshape(self.m, self.r)
        self.nnz = np.ascontiguousarray(nnz, dtype=np.uint32).reshape(self.m)


class Oracle:
    """ctypes front end of ``liboracle.so`` (see ellpack_oracle.c for the citations)."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build(ref=False)
        L = self.lib = C.CDLL(path)
        L.orc_ell_count.restype = C.c_uint32
        L.orc_ell_count.argtypes = [_f32p, C.c_uint32, C.c_uint32, _u32p]
        L.orc_ell_pack.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p, _u32p]
        L.orc_ell_decode.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, _f32p, _u32p, _u32p, _f32p]
        L.orc_activation.argtypes = [_f32p, _f32p, C.c_size_t, C.c_int]
        L.orc_add.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.orc_spmm.argtypes = [C.c_uint32, C.c_uint32, _f32p, _u32p, _u32p, _f32p, C.c_uint32,
                               C.c_size_t, _f32p, C.c_int, _f32p, C.c_size_t]
        L.orc_spmv.argtypes = [C.c_uint32, C.c_uint32, _f32p, _u32p, _u32p, _f32p, _f32p, _f32p]
        L.orc_spmv_absbound.argtypes = [C.c_uint32, C.c_uint32, _f32p, _u32p, _u32p, _f32p, _f32p, _f64p]
        L.orc_maxpool_pf.argtypes = [_f32p] + [C.c_uint32] * 12 + [_f32p]
        L.orc_gap_pf.argtypes = [_f32p] + [C.c_uint32] * 4 + [_f32p]
        L.orc_conv2d.argtypes = [C.c_uint32, C.c_uint32, _f32p, _u32p, _u32p] + [C.c_uint32] * 13 + \
                                [C.c_int, _f32p, C.c_uint32, _f32p, C.c_int, _f32p]

    def encode(self, W) -> EllArrays:
        W = _f32(W)
        m, n = W.shape
        nnz = np.zeros(m, dtype=np.uint32)
        r = self.lib.orc_ell_count(_fp(W), m, n, _up(nnz))
        Wd = np.empty((m, r), dtype=np.float32)
        idx = np.empty((m, r), dtype=np.uint32)
        self.lib.orc_ell_pack(_fp(W), m, n, r, _fp(Wd), _up(idx))
        return EllArrays(m, n, r, Wd, idx, nnz)

    def decode(self, E: EllArrays):
        W = np.empty((E.m, E.n), dtype=np.float32)
        self.lib.orc_ell_decode(E.m, E.n, E.r, _fp(E.Wd), _up(E.idx), _up(E.nnz), _fp(W))
        return W

    def spmm(self, E: EllArrays, X, bias=None, act: int = 0):
        X = _f32(X)
        bias = _f32(bias)
        Cc = X.shape[1]
        Y = np.empty((E.m, Cc), dtype=np.float32)
        self.lib.orc_spmm(E.m, E.r, _fp(E.Wd), _up(E.idx), _up(E.nnz), _fp(X), Cc, Cc, _fp(bias),
                          act, _fp(Y), Cc)
        return Y

    def spmv(self, E: EllArrays, x, bias=None):
        x = _f32(x)
        bias = _f32(bias)
        y = np.empty(E.m, dtype=np.float32)
        self.lib.orc_spmv(E.m, E.r, _fp(E.Wd), _up(E.idx), _up(E.nnz), _fp(x), _fp(bias), _fp(y))
        return y

    def absbound(self, E: EllArrays, x, bias=None):
        """sum_j |w||x| (+|bias|) per row, in float64; the tolerance is 1e-5 times this."""
        x = _f32(x)
        bias = _f32(bias)
        b = np.empty(E.m, dtype=np.float64)
        self.lib.orc_spmv_absbound(E.m, E.r, _fp(E.Wd), _up(E.idx), _up(E.nnz), _fp(x), _fp(bias),
                                   b.ctypes.data_as(_f64p))
        return b

    def conv2d(self, E: EllArrays, geom: dict, layout: int, src, B: int, bias=None, act: int = 0):
        """geom keys: Cin kH kW sH sW pH pW dH dW H W.  layout 0 = [C,H,W,B], 1 = NCHW,
        2 = F-major [W,H,C,B] (input and output)."""
        g = geom
        Ho = (g["H"] + 2 * g["pH"] - (g["dH"] * (g["kH"] - 1) + 1)) // g["sH"] + 1
        Wo = (g["W"] + 2 * g["pW"] - (g["dW"] * (g["kW"] - 1) + 1)) // g["sW"] + 1
        src = _f32(src)
        bias = _f32(bias)
        shape = (E.m, Ho, Wo, B) if layout == 0 else (Wo, Ho, E.m, B) if layout == 2 else (B, E.m, Ho, Wo)
        dst = np.empty(shape, dtype=np.float32)
        self.lib.orc_conv2d(E.m, E.r, _fp(E.Wd), _up(E.idx), _up(E.nnz), g["Cin"], g["kH"], g["kW"],
                            g["sH"], g["sW"], g["pH"], g["pW"], g["dH"], g["dW"], g["H"], g["W"],
                            Ho, Wo, layout, _fp(src), B, _fp(bias), act, _fp(dst))
        return dst

    def maxpool_pf(self, x, k, s, pad):
        """x: [C,H,W,B]; k, s: (h, w); pad: (h0, w0, h1, w1)."""
        x = _f32(x)
        Cc, H, W, B = x.shape
        Ho = (H + pad[0] + pad[2] - k[0]) // s[0] + 1
        Wo = (W + pad[1] + pad[3] - k[1]) // s[1] + 1
        out = np.empty((Cc, Ho, Wo, B), dtype=np.float32)
        self.lib.orc_maxpool_pf(_fp(x), Cc, H, W, B, k[0], k[1], s[0], s[1], pad[0], pad[1], pad[2], pad[3], _fp(out))
        return out

    def gap_pf(self, x):
        x = _f32(x)
        Cc, H, W, B = x.shape
        out = np.empty((Cc, B), dtype=np.float32)
        self.lib.orc_gap_pf(_fp(x), Cc, H, W, B, _fp(out))
        return out

    def activation(self, x, act: int):
        x = _f32(x)
        y = np.empty_like(x)
        self.lib.orc_activation(_fp(x), _fp(y), x.size, act)
        return y


class RefEll:
    """Owning handle of a reference ``Ellpack`` object."""

    def __init__(self, ref: "Reference", handle, owned: bool = True):
        self._ref, self._h, self._owned = ref, handle, owned
        m, n, r = C.c_uint32(), C.c_uint32(), C.c_uint32()
        ref.lib.ref_ell_dims(handle, C.byref(m), C.byref(n), C.byref(r))
        self.m, self.n, self.r = m.value, n.value, r.value

    def arrays(self) -> EllArrays:
        Wd = np.empty((self.m, self.r), dtype=np.float32)
        idx = np.empty((self.m, self.r), dtype=np.uint32)
        nnz = np.empty(self.m, dtype=np.uint32)
        self._ref.lib.ref_ell_copy(self._h, _fp(Wd), _up(idx), _up(nnz))
        return EllArrays(self.m, self.n, self.r, Wd, idx, nnz)

    def __del__(self):
        if getattr(self, "_owned", False) and self._h:
            self._ref.lib.ref_ell_free(self._h)
            self._h = None


class Reference:
    """ctypes front end of the unmodified reference build (``oracle/_ref``)."""

    def __init__(self, path: str = REF_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        if not cpu_has_avx512():
            raise RuntimeError("reference build needs an AVX-512 host")
        L = self.lib = C.CDLL(path)
        vp = C.c_void_p
        L.ref_ell_encode.restype = vp
        L.ref_ell_encode.argtypes = [_f32p, C.c_uint32, C.c_uint32]
        L.ref_ell_from_arrays.restype = vp
        L.ref_ell_from_arrays.argtypes = [C.c_uint32] * 3 + [_f32p, _u32p, _u32p]
        L.ref_ell_free.argtypes = [vp]
        L.ref_ell_dims.argtypes = [vp, _u32p, _u32p, _u32p]
        L.ref_ell_copy.argtypes = [vp, _f32p, _u32p, _u32p]
        L.ref_ell_decode.argtypes = [vp, _f32p]
        L.ref_matmul.argtypes = [vp, _f32p, C.c_uint32, _f32p, _f32p]
        L.ref_matmul_fused.argtypes = [vp, _f32p, C.c_uint32, _f32p, _f32p, C.c_int]
        L.ref_matvec.argtypes = [vp, _f32p, _f32p, _f32p]
        L.ref_conv_create.restype = vp
        L.ref_conv_create.argtypes = [_f32p] + [C.c_uint32] * 12 + [_f32p, C.c_int]
        L.ref_conv_free.argtypes = [vp]
        L.ref_conv_out_dims.argtypes = [vp, _u32p, _u32p]
        L.ref_conv_ell.restype = vp
        L.ref_conv_ell.argtypes = [vp]
        L.ref_conv_run.argtypes = [vp, C.c_int, _f32p, C.c_uint32, _f32p]
        L.ref_rbm_build.restype = vp
        L.ref_rbm_build.argtypes = [vp, _f32p, C.c_uint32]
        L.ref_rbm_free.argtypes = [vp]
        L.ref_rbm_num_blocks.restype = C.c_uint32
        L.ref_rbm_num_blocks.argtypes = [vp]
        L.ref_rbm_block_sizes.argtypes = [vp, C.c_uint32] + [_u32p] * 5
        L.ref_rbm_block_copy.argtypes = [vp, C.c_uint32, _u32p, _u32p, _u16p, _f32p, _f32p]
        L.ref_model_load.restype = vp
        L.ref_model_load.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
        L.ref_model_free.argtypes = [vp]
        L.ref_model_output_shape.restype = C.c_int
        L.ref_model_output_shape.argtypes = [vp, _u64p, C.c_int]
        L.ref_model_run.restype = C.c_int
        L.ref_model_run.argtypes = [vp, _f32p, C.c_uint32, _f32p, C.c_char_p, C.c_size_t]

    # -- Ellpack ------------------------------------------------------------------
    def encode(self, W) -> RefEll:
        W = _f32(W)
        return RefEll(self, self.lib.ref_ell_encode(_fp(W), W.shape[0], W.shape[1]))

    def from_arrays(self, E: EllArrays) -> RefEll:
        return RefEll(self, self.lib.ref_ell_from_arrays(E.m, E.n, E.r, _fp(E.Wd), _up(E.idx), _up(E.nnz)))

    def decode(self, E: RefEll):
        W = np.empty((E.m, E.n), dtype=np.float32)
        self.lib.ref_ell_decode(E._h, _fp(W))
        return W

    # -- kernels ------------------------------------------------------------------
    def matmul(self, E: RefEll, X, bias=None, relu=None, out=None):
        """relu=None: the dispatcher the Python binding calls; True/False: the fused template."""
        X = _f32(X)
        bias = _f32(bias)
        Cc = X.shape[1]
        Y = np.empty((E.m, Cc), dtype=np.float32) if out is None else out
        if relu is None:
            self.lib.ref_matmul(E._h, _fp(X), Cc, _fp(bias), _fp(Y))
        else:
            self.lib.ref_matmul_fused(E._h, _fp(X), Cc, _fp(bias), _fp(Y), int(relu))
        return Y

    def matvec(self, E: RefEll, x, bias=None, out=None):
        x = _f32(x)
        bias = _f32(bias)
        y = np.empty(E.m, dtype=np.float32) if out is None else out
        self.lib.ref_matvec(E._h, _fp(x), _fp(bias), _fp(y))
        return y

    # -- conv ---------------------------------------------------------------------
    def conv_create(self, weight, geom: dict, bias=None, relu: bool = False):
        weight = _f32(weight)
        Cout, Cin, kH, kW = weight.shape
        g = geom
        self._keep_bias = _f32(bias)
        return self.lib.ref_conv_create(_fp(weight), Cout, Cin, kH, kW, g["sH"], g["sW"], g["pH"],
                                        g["pW"], g["dH"], g["dW"], g["H"], g["W"], _fp(self._keep_bias),
                                        int(relu))

    def conv_ell(self, h) -> RefEll:
        return RefEll(self, self.lib.ref_conv_ell(h), owned=False)

    def conv_run(self, h, layout: int, src, B: int, Cout: int, out=None):
        Ho, Wo = C.c_uint32(), C.c_uint32()
        self.lib.ref_conv_out_dims(h, C.byref(Ho), C.byref(Wo))
        src = _f32(src)
        # layouts 2 and 3 both write F-major [W,H,C,B]; 2 reads [C,H,W,B], 3 reads F-major
        shape = (Cout, Ho.value, Wo.value, B) if layout == 0 else \
            (Wo.value, Ho.value, Cout, B) if layout in (2, 3) else (B, Cout, Ho.value, Wo.value)
        dst = np.empty(shape, dtype=np.float32) if out is None else out
        self.lib.ref_conv_run(h, layout, _fp(src), B, _fp(dst))
        return dst

    def conv_free(self, h):
        self.lib.ref_conv_free(h)

    # -- RBM plan -----------------------------------------------------------------
    def rbm(self, E: RefEll, bias=None, ct_max: int = 8):
        bias = _f32(bias)
        p = self.lib.ref_rbm_build(E._h, _fp(bias), ct_max)
        blocks = []
        for b in range(self.lib.ref_rbm_num_blocks(p)):
            v = [C.c_uint32() for _ in range(5)]
            self.lib.ref_rbm_block_sizes(p, b, *[C.byref(x) for x in v])
            M0, Ct, U, npairs, nbias = [x.value for x in v]
            krel = np.empty(U, dtype=np.uint32)
            colptr = np.empty(U + 1 if (U or npairs == 0) else 1, dtype=np.uint32)
            rows = np.empty(npairs, dtype=np.uint16)
            w = np.empty(npairs, dtype=np.float32)
            bb = np.empty(nbias, dtype=np.float32)
            self.lib.ref_rbm_block_copy(p, b, _up(krel), _up(colptr), rows.ctypes.data_as(_u16p), _fp(w), _fp(bb))
            blocks.append(dict(M0=M0, Ct=Ct, krel=krel, colptr=colptr, rows=rows, w=w, bias=bb))
        self.lib.ref_rbm_free(p)
        return blocks

    # -- model --------------------------------------------------------------------
    def model_load(self, path: str):
        err = C.create_string_buffer(512)
        h = self.lib.ref_model_load(path.encode(), err, 512)
        if not h:
            raise RuntimeError(err.value.decode())
        return h

    def model_output_shape(self, h):
        dims = (C.c_uint64 * 8)()
        n = self.lib.ref_model_output_shape(h, dims, 8)
        return tuple(int(dims[i]) for i in range(n))

    def model_run(self, h, x_mem, B: int):
        """x_mem: the input MEMORY (feature-major / [C,H,W,B]); returns the output memory, flat."""
        x_mem = _f32(x_mem)
        out = np.empty(int(np.prod(self.model_output_shape(h))), dtype=np.float32)
        err = C.create_string_buffer(512)
        if self.lib.ref_model_run(h, _fp(x_mem), B, _fp(out), err, 512):
            raise RuntimeError(err.value.decode())
        return out

    def model_free(self, h):
        self.lib.ref_model_free(h)
