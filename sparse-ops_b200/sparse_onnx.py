"""Pure-Python layer loop over the ELLPACK bindings: the counterpart of the reference's
python/sparse_onnx.py:6-53 (class OnnxSparseModel), with the same plan and the same run()
semantics, on top of `cpp_backend` (encode / matvec / matmul) of this package.

This file is a drop-in shim, not an independent design: the class body restates the reference's
class line for line (same plan tuples, same branches in run()), because its observable behaviour
is the contract.  The one change: the reference reads the file with the `onnx` package; here the
in-tree wire-format reader (`onnx_wire.read_model`) is used, so nothing beyond numpy is needed.

Plan (python/sparse_onnx.py:19-34): every Gemm / MatMul node becomes ('matmul', E, bias) with
E = encode(initializer named by input[1]) taken AS STORED (no transpose attribute is read) and
bias = the Gemm's third input when present; Relu / Sigmoid / Tanh nodes become numpy
activations; any other op raises NotImplementedError.

run(x) (python/sparse_onnx.py:36-53): a 1-D x goes through matvec, a 2-D x of shape (n, C)
through matmul; activations are applied with numpy on the host.  A layer without bias passes
None, which these bindings take as "no bias".
"""
from __future__ import annotations

import numpy as np

from cpp_backend import encode, matmul, matvec
from onnx_wire import read_model


class OnnxSparseModel:
    def __init__(self, onnx_path: str):
        with open(onnx_path, "rb") as f:
            model = read_model(f.read())
        self._initializers = model["initializers"]
        self.layers = []
        for node in model["nodes"]:
            op = node["op_type"]
            if op in ("Gemm", "MatMul"):
                W = self._initializers[node["input"][1]]
                b = None
                if op == "Gemm" and len(node["input"]) > 2:
                    b = self._initializers[node["input"][2]]
                self.layers.append(("matmul", encode(W), b, {}))
            elif op in ("Relu", "Sigmoid", "Tanh"):
                self.layers.append((op.lower(), None, None, {}))
            else:
                raise NotImplementedError(f"Unsupported op {op}")

    def run(self, x: np.ndarray) -> np.ndarray:
        """x is (n,) for one sample or (n, C) for C samples in columns."""
        v = np.asarray(x, dtype=np.float32)
        for op, E, b, _ in self.layers:
            if op == "matmul":
                v = matvec(E, v, b) if v.ndim == 1 else matmul(E, v, b)
            elif op == "relu":
                v = np.maximum(v, 0, out=v)
            elif op == "sigmoid":
                v = 1 / (1 + np.exp(-v))
            elif op == "tanh":
                v = np.tanh(v)
        return v
