"""Generates tests/golden/reference_vectors.npz from the UNMODIFIED reference implementation.

Run where the reference sources are available (they are compiled in place by oracle/Makefile):

    python tests/golden/make_golden.py

Every array named ``*_ref`` is an output of the reference binary (oracle/_ref) on the seeded
inputs stored next to it; the file is the parity pin for the C restatement in oracle/ and for
the CUDA library.  Model-level vectors hold the ONNX file bytes, the input MEMORY (feature-major
or [C,H,W,B]) and the output memory exactly as the reference's run() reads and writes them.
"""
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "sparse-ops_b200"))

import oracle  # noqa: E402
import onnx_wire  # noqa: E402


def sparse(rng, m, n, p, scale=1.0):
    W = (rng.standard_normal((m, n)) * scale).astype(np.float32)
    W[rng.random((m, n)) >= p] = 0.0
    return W


def main():
    oracle.build(ref=True)
    R = oracle.Reference()
    rng = np.random.default_rng(20240611)
    out = {}

    # --- encoder: the hand matrix of the reference's unit test + special values -----------------
    hand = np.array([[1, 0, 0, 2], [0, 3, 0, 0], [0, 0, 4, 0], [0, 0, 0, 5]], dtype=np.float32)
    special = sparse(rng, 9, 13, 0.4)
    special[0, 0] = -0.0
    special[1, 2] = np.nan
    special[2, 3] = np.inf
    special[3, 4] = np.float32(1e-42)      # denormal
    special[4, :] = 0.0                    # empty row
    special[5, :] = 1.5                    # full row
    for name, W in (("enc_hand", hand), ("enc_special", special), ("enc_zero", np.zeros((5, 7), np.float32)),
                    ("enc_rand", sparse(rng, 33, 77, 0.3))):
        E = R.encode(W).arrays()
        out[name + "_W"] = W
        out[name + "_Wd_ref"], out[name + "_idx_ref"], out[name + "_nnz_ref"] = E.Wd, E.idx, E.nnz
        out[name + "_decoded_ref"] = R.decode(R.encode(W))

    # --- SpMM / SpMV ----------------------------------------------------------------------------
    for name, (m, n, C, p) in {"mm_a": (48, 64, 20, 0.3), "mm_b": (96, 80, 32, 0.1), "mm_c": (17, 300, 7, 0.5),
                               "mm_d": (130, 257, 260, 0.15)}.items():
        W = sparse(rng, m, n, p)
        X = rng.uniform(-1, 1, (n, C)).astype(np.float32)
        b = rng.standard_normal(m).astype(np.float32)
        x = rng.uniform(-1, 1, n).astype(np.float32)
        E = R.encode(W)
        out[name + "_W"], out[name + "_X"], out[name + "_bias"], out[name + "_x"] = W, X, b, x
        out[name + "_Y_ref"] = R.matmul(E, X, b)                  # the binding's dispatcher
        out[name + "_Yrelu_ref"] = R.matmul(E, X, b, relu=True)   # fused template (model path)
        out[name + "_Ynobias_ref"] = R.matmul(E, X, None, relu=False)
        out[name + "_y_ref"] = R.matvec(E, x, b)
        out[name + "_ynobias_ref"] = R.matvec(E, x, None)

    # --- conv kernels, both layouts (stride 1: the reference mis-indexes stride_w > 1) -----------
    convs = {"conv_a": (3, 8, 16, 9, 11, 3, 1, 1, True), "conv_b": (1, 4, 5, 7, 7, 3, 0, 1, False),
             "conv_c": (4, 6, 7, 10, 8, 3, 2, 2, True), "conv_d": (8, 16, 12, 6, 6, 1, 0, 1, True),
             "conv_e": (2, 5, 9, 12, 8, 5, 2, 1, False)}   # W=8: the reference's PF kernel overruns its tile when a width tile is narrower than the right overhang (e.g. W=9, k=5, pad=2)
    for name, (B, Cin, Cout, H, W_, k, pad, dil, relu) in convs.items():
        wt = sparse(rng, Cout, Cin * k * k, 0.3, 0.3).reshape(Cout, Cin, k, k)
        bias = rng.standard_normal(Cout).astype(np.float32)
        g = dict(Cin=Cin, kH=k, kW=k, sH=1, sW=1, pH=pad, pW=pad, dH=dil, dW=dil, H=H, W=W_)
        x = rng.standard_normal((B, Cin, H, W_)).astype(np.float32)
        h = R.conv_create(wt, g, bias, relu)
        out[name + "_weight"], out[name + "_bias"], out[name + "_x_nchw"] = wt, bias, x
        out[name + "_geom"] = np.array([B, Cin, Cout, H, W_, k, pad, dil, int(relu)], dtype=np.int64)
        out[name + "_pf_ref"] = R.conv_run(h, 0, np.ascontiguousarray(x.transpose(1, 2, 3, 0)), B, Cout)
        out[name + "_nchw_ref"] = R.conv_run(h, 1, x, B, Cout)
        # F-major [W,H,C,B]: conv2d_tiled_im2col_fmajor reads [C,H,W,B] and writes F-major,
        # conv2d_rbm_fmajor_implicit reads and writes F-major; both must give the same bytes
        fm = R.conv_run(h, 2, np.ascontiguousarray(x.transpose(1, 2, 3, 0)), B, Cout)
        fm_rbm = R.conv_run(h, 3, np.ascontiguousarray(x.transpose(3, 2, 1, 0)), B, Cout)
        assert np.array_equal(fm.view(np.uint32), fm_rbm.view(np.uint32)), name
        out[name + "_fm_ref"] = fm
        if name == "conv_a":
            blocks = R.rbm(R.conv_ell(h), bias, 8)
            out["rbm_M0"] = np.array([b["M0"] for b in blocks], dtype=np.uint32)
            out["rbm_Ct"] = np.array([b["Ct"] for b in blocks], dtype=np.uint32)
            out["rbm_krel_ref"] = np.concatenate([b["krel"] for b in blocks])
            out["rbm_krel_len"] = np.array([len(b["krel"]) for b in blocks], dtype=np.uint32)
            out["rbm_colptr_ref"] = np.concatenate([b["colptr"] for b in blocks])
            out["rbm_rows_ref"] = np.concatenate([b["rows"] for b in blocks])
            out["rbm_w_ref"] = np.concatenate([b["w"] for b in blocks])
            out["rbm_bias_ref"] = np.concatenate([b["bias"] for b in blocks])
        R.conv_free(h)

    # --- models through SparseOnnxModel::run -------------------------------------------------------
    def run_model(blob, x_mem, B):
        with tempfile.NamedTemporaryFile(suffix=".onnx", delete=False) as f:
            f.write(blob)
            path = f.name
        try:
            h = R.model_load(path)
            shape = R.model_output_shape(h)
            y = R.model_run(h, x_mem, B)
            R.model_free(h)
        finally:
            os.unlink(path)
        return np.array(shape, dtype=np.int64), y

    dims, B = [40, 48, 24, 10], 16        # B % 16 == 0: the reference's unmasked AVX-512 kernel
    Ws = [sparse(rng, dims[i + 1], dims[i], 0.3, 0.4) for i in range(3)]
    bs = [rng.standard_normal(dims[i + 1]).astype(np.float32) * 0.1 for i in range(3)]
    blob = onnx_wire.mlp_model(Ws, bs, ["Relu", "Tanh", "Sigmoid"], B)
    x = rng.uniform(0, 1, (B, dims[0])).astype(np.float32)
    out["mlp_onnx"] = np.frombuffer(blob, dtype=np.uint8)
    out["mlp_x_mem"] = np.ascontiguousarray(x.T)              # [features][B]
    out["mlp_shape_ref"], out["mlp_y_mem_ref"] = run_model(blob, out["mlp_x_mem"], B)

    B = 5                                   # masked kernel path
    blob = onnx_wire.mlp_model(Ws[:2], [bs[0], None], ["Relu", None], B)
    x = rng.uniform(0, 1, (B, dims[0])).astype(np.float32)
    out["mlp2_onnx"] = np.frombuffer(blob, dtype=np.uint8)
    out["mlp2_x_mem"] = np.ascontiguousarray(x.T)
    out["mlp2_shape_ref"], out["mlp2_y_mem_ref"] = run_model(blob, out["mlp2_x_mem"], B)

    B, Cc, H, W_ = 3, 6, 8, 7
    cw = [sparse(rng, Cc, Cc * 9, 0.3, 0.3).reshape(Cc, Cc, 3, 3) for _ in range(2)]
    cb = [rng.standard_normal(Cc).astype(np.float32) * 0.1 for _ in range(2)]
    blob = onnx_wire.conv_model(cw, cb, [True, True], B, H, W_)
    x = rng.standard_normal((B, Cc, H, W_)).astype(np.float32)
    out["cnn_onnx"] = np.frombuffer(blob, dtype=np.uint8)
    out["cnn_x_mem"] = np.ascontiguousarray(x.transpose(1, 2, 3, 0))    # [C,H,W,B]
    out["cnn_shape_ref"], out["cnn_y_mem_ref"] = run_model(blob, out["cnn_x_mem"], B)

    # --- pools: the reference runs them only inside a model and indexes them b + B*(c + C*(h + H*w)),
    # so the logical NCHW tensor is handed over (and read back) in that memory order ---------------
    B, Cc, H, W_ = 3, 5, 9, 8
    x = rng.standard_normal((B, Cc, H, W_)).astype(np.float32)
    x_f = np.ascontiguousarray(x.transpose(3, 2, 1, 0))                   # [w][h][c][b]
    mp = onnx_wire.model([onnx_wire.node("MaxPool", ["input"], ["y"], [
        onnx_wire.attr_ints("kernel_shape", [3, 3]), onnx_wire.attr_ints("strides", [2, 2]),
        onnx_wire.attr_ints("pads", [1, 1, 1, 1])])], [], ("input", (B, Cc, H, W_)), ("y", (B, Cc, 5, 4)))
    shape, y = run_model(mp, x_f, B)
    out["pool_x_nchw"] = x
    out["pool_max_ref"] = np.ascontiguousarray(y.reshape(4, 5, Cc, B).transpose(3, 2, 1, 0))   # logical NCHW
    gp = onnx_wire.model([onnx_wire.node("GlobalAveragePool", ["input"], ["y"])], [],
                         ("input", (B, Cc, H, W_)), ("y", (B, Cc)))
    shape, y = run_model(gp, x_f, B)
    out["pool_gap_ref"] = np.ascontiguousarray(y[:Cc * B].reshape(Cc, B).T)                     # logical (B, C)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
