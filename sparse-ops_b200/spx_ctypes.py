"""ctypes binding of the C ABI in include/spx_b200.h (libspx_b200.so).

This is the stub a maintainer of another host language would write against the header; the
parity tests and the benchmark use it to call the CUDA path with raw device pointers
(e.g. ``tensor.data_ptr()`` of torch CUDA tensors).  Every call raises ``SpxError`` on a
non-zero status -- there is no CPU fallback behind it.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libspx_b200.so")

ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3
LAYOUT_PF, LAYOUT_NCHW, LAYOUT_FMAJOR = 0, 1, 2
OP_RELU, OP_SIGMOID, OP_TANH, OP_ADD = 1, 2, 3, 4
UNIQUE_ID_BYTES = 128
IPC_HANDLE_BYTES = 64


class SpxError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"spx status {status}: {message}")
        self.status = status


class ConvGeom(C.Structure):
    _fields_ = [(k, C.c_uint32) for k in
                ("Cin", "Cout", "kH", "kW", "sH", "sW", "pH", "pW", "dH", "dW", "H", "W", "Ho", "Wo")]


def conv_geom(Cin, Cout, kH, kW, H, W, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1) -> ConvGeom:
    Ho = (H + 2 * pH - (dH * (kH - 1) + 1)) // sH + 1
    Wo = (W + 2 * pW - (dW * (kW - 1) + 1)) // sW + 1
    return ConvGeom(Cin, Cout, kH, kW, sH, sW, pH, pW, dH, dW, H, W, Ho, Wo)


_vp = C.c_void_p
_f32p = C.POINTER(C.c_float)
_u32p = C.POINTER(C.c_uint32)
_u64p = C.POINTER(C.c_uint64)

# name -> (restype, argtypes); every symbol include/spx_b200.h declares
SIGNATURES = {
    "spx_last_error": (C.c_char_p, []),
    "spx_version": (C.c_int, []),
    "spx_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "spx_set_device": (C.c_int, [C.c_int]),
    "spx_get_device": (C.c_int, [C.POINTER(C.c_int)]),
    "spx_device_sync": (C.c_int, []),
    "spx_launch_count": (C.c_uint64, []),
    "spx_malloc": (C.c_int, [C.POINTER(_vp), C.c_size_t]),
    "spx_free": (C.c_int, [_vp]),
    "spx_host_alloc": (C.c_int, [C.POINTER(_vp), C.c_size_t]),
    "spx_host_free": (C.c_int, [_vp]),
    "spx_memcpy_h2d": (C.c_int, [_vp, _vp, C.c_size_t, _vp]),
    "spx_memcpy_d2h": (C.c_int, [_vp, _vp, C.c_size_t, _vp]),
    "spx_memcpy_d2d": (C.c_int, [_vp, _vp, C.c_size_t, _vp]),
    "spx_memset": (C.c_int, [_vp, C.c_int, C.c_size_t, _vp]),
    "spx_stream_create": (C.c_int, [C.POINTER(_vp)]),
    "spx_stream_destroy": (C.c_int, [_vp]),
    "spx_stream_sync": (C.c_int, [_vp]),
    "spx_event_create": (C.c_int, [C.POINTER(_vp)]),
    "spx_event_destroy": (C.c_int, [_vp]),
    "spx_event_record": (C.c_int, [_vp, _vp]),
    "spx_event_elapsed_ms": (C.c_int, [_vp, _vp, C.POINTER(C.c_float)]),
    "spx_graph_capture_begin": (C.c_int, [_vp]),
    "spx_graph_capture_end": (C.c_int, [_vp, C.POINTER(_vp)]),
    "spx_graph_launch": (C.c_int, [_vp, _vp]),
    "spx_graph_destroy": (C.c_int, [_vp]),
    "spx_ell_create": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, _vp, _vp, _vp, C.POINTER(_vp)]),
    "spx_ell_create_csr": (C.c_int, [C.c_uint32, C.c_uint32, _vp, _vp, _vp, C.POINTER(_vp)]),
    "spx_ell_encode_device": (C.c_int, [_vp, C.c_uint32, C.c_uint32, _vp, C.POINTER(_vp)]),
    "spx_ell_destroy": (C.c_int, [_vp]),
    "spx_ell_dims": (C.c_int, [_vp, _u32p, _u32p, _u32p, _u64p]),
    "spx_ell_download": (C.c_int, [_vp, _vp, _vp, _vp]),
    "spx_ell_decode_device": (C.c_int, [_vp, _vp, _vp]),
    "spx_spmm": (C.c_int, [_vp, _vp, C.c_uint32, C.c_uint64, _vp, C.c_int, _vp, C.c_uint64, _vp]),
    "spx_spmv": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "spx_spmv_reference_order": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "spx_conv2d": (C.c_int, [_vp, C.POINTER(ConvGeom), C.c_int, _vp, C.c_uint32, _vp, C.c_int, _vp, _vp]),
    "spx_conv2d_static": (C.c_int, [_vp, C.POINTER(ConvGeom), C.c_int, _vp, C.c_uint32, _vp, C.c_int, _vp, _vp]),
    "spx_eltwise": (C.c_int, [C.c_int, _vp, _vp, _vp, C.c_uint64, _vp]),
    "spx_maxpool2d": (C.c_int, [_vp] + [C.c_uint32] * 12 + [_vp, _vp]),
    "spx_global_avgpool": (C.c_int, [_vp] + [C.c_uint32] * 4 + [_vp, _vp]),
    "spx_spmm_host": (C.c_int, [_vp, _vp, C.c_uint32, _vp, C.c_int, _vp]),
    "spx_spmv_host": (C.c_int, [_vp, _vp, _vp, _vp]),
    "spx_comm_unique_id": (C.c_int, [C.c_char_p]),
    "spx_comm_create": (C.c_int, [C.c_int, C.c_int, C.c_char_p, C.POINTER(_vp)]),
    "spx_comm_destroy": (C.c_int, [_vp]),
    "spx_allgather_rows": (C.c_int, [_vp, _vp, C.c_uint64, C.c_uint64, _vp]),
    "spx_comm_barrier": (C.c_int, [_vp, _vp]),
    "spx_comm_info": (C.c_int, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "spx_spmm_host_sharded": (C.c_int, [_vp, _vp, _vp, C.c_uint32, _vp, C.c_int, _vp, _f32p]),
    "spx_ipc_export": (C.c_int, [_vp, C.c_char_p]),
    "spx_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(_vp)]),
    "spx_ipc_close": (C.c_int, [_vp]),
    "spx_spmm_bcast": (C.c_int, [_vp, _vp, C.c_uint32, C.c_uint64, _vp, C.c_int, C.POINTER(_vp), C.c_uint32, C.c_uint64,
                                 C.c_uint64, _vp]),
    "spx_spmm_exchange": (C.c_int, [_vp, _vp, C.c_uint32, C.c_uint64, _vp, C.c_int, C.POINTER(_vp), C.c_uint32, C.c_uint32,
                                    C.c_uint64, C.c_uint64, C.c_uint32, _vp]),
    "spx_spmm_mcast": (C.c_int, [_vp, _vp, C.c_uint32, C.c_uint64, _vp, C.c_int, _vp, C.c_uint64, C.c_uint64, _vp]),
}

_STATUS_FREE = {"spx_last_error", "spx_version", "spx_launch_count"}


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(_vp)


class Lib:
    """Loaded libspx_b200.so with typed, status-checked calls (``lib.spx_spmm(...)``)."""

    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: build it with sparse-ops_b200/build_cuda.sh")
        self._dll = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self._dll, name)
            fn.restype = res
            fn.argtypes = args
            setattr(self, "raw_" + name, fn)
            setattr(self, name, fn if name in _STATUS_FREE else self._checked(fn))

    def _checked(self, fn):
        def call(*args):
            st = fn(*args)
            if st != 0:
                raise SpxError(st, self._dll.spx_last_error().decode(errors="replace"))
            return st
        return call

    # ---- convenience -------------------------------------------------------------------
    def ell_create(self, Wd, idx, nnz, n) -> "Ell":
        Wd = np.ascontiguousarray(Wd, dtype=np.float32)
        idx = np.ascontiguousarray(idx, dtype=np.uint32)
        nnz = np.ascontiguousarray(nnz, dtype=np.uint32)
        m, r = Wd.shape
        h = _vp()
        self.spx_ell_create(m, n, r, _np_ptr(Wd), _np_ptr(idx), _np_ptr(nnz), C.byref(h))
        return Ell(self, h)

    def ell_create_csr(self, m, n, rowptr, col, val) -> "Ell":
        rowptr = np.ascontiguousarray(rowptr, dtype=np.uint64)
        col = np.ascontiguousarray(col, dtype=np.uint32)
        val = np.ascontiguousarray(val, dtype=np.float32)
        h = _vp()
        self.spx_ell_create_csr(m, n, _np_ptr(rowptr), _np_ptr(col), _np_ptr(val), C.byref(h))
        return Ell(self, h)

    def ell_encode_device(self, dW_ptr: int, m: int, n: int, stream: int = 0) -> "Ell":
        h = _vp()
        self.spx_ell_encode_device(dW_ptr, m, n, stream, C.byref(h))
        return Ell(self, h)


class Ell:
    """Owning wrapper of an ``spx_ell*``."""

    def __init__(self, lib: Lib, handle):
        self.lib, self.h = lib, handle
        m, n, r, t = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64()
        lib.spx_ell_dims(handle, C.byref(m), C.byref(n), C.byref(r), C.byref(t))
        self.m, self.n, self.r, self.nnz_total = m.value, n.value, r.value, t.value

    def download(self):
        Wd = np.empty((self.m, self.r), dtype=np.float32)
        idx = np.empty((self.m, self.r), dtype=np.uint32)
        nnz = np.empty(self.m, dtype=np.uint32)
        self.lib.spx_ell_download(self.h, _np_ptr(Wd), _np_ptr(idx), _np_ptr(nnz))
        return Wd, idx, nnz

    def spmm(self, X_ptr, C_, ldx, bias_ptr, act, Y_ptr, ldy, stream=0):
        self.lib.spx_spmm(self.h, X_ptr, C_, ldx, bias_ptr, act, Y_ptr, ldy, stream)

    def spmv(self, x_ptr, bias_ptr, y_ptr, stream=0):
        self.lib.spx_spmv(self.h, x_ptr, bias_ptr, y_ptr, stream)

    def conv2d(self, geom: ConvGeom, layout, in_ptr, B, bias_ptr, act, out_ptr, stream=0):
        self.lib.spx_conv2d(self.h, C.byref(geom), layout, in_ptr, B, bias_ptr, act, out_ptr, stream)

    def spmm_host(self, X, bias, act=ACT_NONE):
        X = np.ascontiguousarray(X, dtype=np.float32)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        Y = np.empty((self.m, X.shape[1]), dtype=np.float32)
        self.lib.spx_spmm_host(self.h, _np_ptr(X), X.shape[1], _np_ptr(bias), act, _np_ptr(Y))
        return Y

    def spmv_host(self, x, bias):
        x = np.ascontiguousarray(x, dtype=np.float32)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        y = np.empty(self.m, dtype=np.float32)
        self.lib.spx_spmv_host(self.h, _np_ptr(x), _np_ptr(bias), _np_ptr(y))
        return y

    def close(self):
        if self.h:
            self.lib.raw_spx_ell_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
