"""Thin Python wrappers over `sparseops_backend`, same names and signatures as the reference's
python/cpp_backend.py:4-37 (encode / matvec / matmul)."""
import numpy as np
import sparseops_backend


def encode(sparse_matrix: np.ndarray) -> sparseops_backend.Ellpack:
    """Dense (M, K) array -> device-resident ELLPACK handle."""
    return sparseops_backend.convert_to_ellpack(sparse_matrix)


def matvec(E, x, bias: np.ndarray) -> np.ndarray:
    """y = E x + bias; x is (n,), bias (m,), returns (m,) float32."""
    return sparseops_backend.ellpack_matvec(E, x, bias)


def matmul(E: sparseops_backend.Ellpack, X: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """Y = E X + bias[:, None]; X is (n, C), returns (m, C) float32."""
    return sparseops_backend.ellpack_matmul(E, X, bias)
