"""GPU tests of the drop-in Python module `sparseops_backend`.  The first three tests restate the
reference's own unit tests (tests/unit/test_ellpack_encoder.py, test_matvec.py, test_matmul.py: same
shapes, same atol=1e-5 against dense numpy); the rest check the model loop against the golden
vectors of the reference binary and the extensions (resize_buffers, device pointers, sharding)."""
import os
import tempfile

import numpy as np
import pytest
import torch

from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu


def generate_sparse_matrix(M, K, sparsity=0.3, seed=0):
    dense = np.random.default_rng([M, K, seed]).random((M, K)).astype(np.float32)
    dense[dense < sparsity] = 0
    return dense


def test_encoder_unit_cases(backend, cuda):
    W = generate_sparse_matrix(64, 64)
    E = backend.convert_to_ellpack(W)
    assert np.allclose(W, backend.decode_from_ellpack(E), atol=1e-5)
    assert (E.m, E.n) == (64, 64) and E.r == np.max(np.count_nonzero(W, axis=1)) and E.on_device
    Z = backend.convert_to_ellpack(np.zeros((32, 32), dtype=np.float32))
    assert (Z.m, Z.n, Z.r) == (32, 32, 0)
    hand = np.array([[1, 0, 0, 2], [0, 3, 0, 0], [0, 0, 4, 0], [0, 0, 0, 5]], dtype=np.float32)
    H = backend.convert_to_ellpack(hand)
    assert H.Wd.shape == (4, 2) and H.Wd[0, 1] == 2.0 and H.Wd[1, 1] == 0.0
    assert H.idx.tolist() == [[0, 3], [1, 0], [2, 0], [3, 0]]
    N = backend.convert_to_ellpack(generate_sparse_matrix(64, 32))
    assert (N.m, N.n) == (64, 32) and backend.decode_from_ellpack(N).shape == (64, 32)


MATVEC = [(16, 32, 0.3), (64, 128, 0.5), (128, 256, 0.7), (256, 512, 0.9), (1, 1, 0.0), (1, 1000, 0.1), (1000, 1, 0.1),
          (0, 0, 0.0), (32, 32, 1.0), (10, 10, 0.0), (10, 10, 0.5), (10, 10, 0.9), (20, 20, 0.2), (100, 100, 0.2),
          (1000, 1000, 0.1), (500, 500, 0.05), (2000, 2000, 0.3), (3000, 3000, 0.4)]


@pytest.mark.parametrize("M,K,sparsity", MATVEC)
def test_matvec_unit_cases(backend, cuda, M, K, sparsity):
    W = generate_sparse_matrix(M, K, sparsity)
    E = backend.convert_to_ellpack(W)
    x = np.random.default_rng(1).random(K).astype(np.float32)
    bias = np.random.default_rng(2).random(M).astype(np.float32)
    y = backend.ellpack_matvec(E, x, bias)
    assert y.shape == (M,)
    assert np.allclose(y, W @ x + bias, atol=1e-5)          # the reference's own assertion, as written there
    y64 = W.astype(np.float64) @ x + bias
    assert (np.abs(y - y64) <= 1e-5 * (np.abs(W) @ np.abs(x) + np.abs(bias)) + 1e-12).all()


MATMUL = [(16, 32, 1, 0.3), (16, 32, 10, 0.3), (16, 32, 100, 0.3), (64, 128, 10, 0.5), (128, 256, 20, 0.7),
          (256, 512, 10, 0.9), (1, 1, 1, 0.0), (1, 1000, 1, 0.1), (1000, 1, 1, 0.1), (0, 0, 0, 0.0), (32, 32, 1, 1.0),
          (10, 10, 1, 0.0), (10, 10, 10, 0.5), (10, 10, 10, 0.9), (20, 20, 10, 0.2), (100, 100, 10, 0.2),
          (1000, 1000, 10, 0.1), (500, 500, 10, 0.05), (2000, 2000, 10, 0.3), (3000, 3000, 10, 0.4)]


@pytest.mark.parametrize("M,K,C,sparsity", MATMUL)
def test_matmul_unit_cases(backend, cuda, M, K, C, sparsity):
    W = generate_sparse_matrix(M, K, sparsity)
    E = backend.convert_to_ellpack(W)
    X = np.random.default_rng(1).random((K, C)).astype(np.float32)
    bias = np.random.default_rng(2).random(M).astype(np.float32)
    Y = backend.ellpack_matmul(E, X, bias)
    assert Y.shape == (M, C)
    assert np.allclose(Y, W @ X + bias[:, None], atol=1e-5)   # the reference's own assertion, as written there
    Y64 = W.astype(np.float64) @ X + bias[:, None]
    assert (np.abs(Y - Y64) <= 1e-5 * (np.abs(W) @ np.abs(X) + np.abs(bias)[:, None]) + 1e-12).all()


def test_reference_unit_tests_in_place(cuda):
    """The reference's own tests/unit, unmodified and where they lie, against this module (found
    through PYTHONPATH).  Needs a machine that has both a GPU and the reference's tree; skipped
    elsewhere -- the three tests above restate the same cases for those machines."""
    import subprocess
    import sys
    unit = os.environ.get("SPX_REFERENCE_TESTS", "/root/reference/tests/unit")
    if not os.path.isdir(unit):
        pytest.skip(f"{unit} is not present on this machine")
    from conftest import PKG
    env = dict(os.environ, PYTHONPATH=PKG + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--rootdir", unit, unit],
                         env=env, capture_output=True, text=True, timeout=900, cwd=tempfile.gettempdir())
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]


def test_binding_errors_and_extras(backend, cuda):
    E = backend.convert_to_ellpack(generate_sparse_matrix(8, 6))
    with pytest.raises(RuntimeError, match="X must be 2D"):
        backend.ellpack_matmul(E, np.ones(6, np.float32), np.ones(8, np.float32))
    with pytest.raises(RuntimeError, match="Input row count must equal E.n"):
        backend.ellpack_matmul(E, np.ones((5, 2), np.float32), np.ones(8, np.float32))
    with pytest.raises(RuntimeError, match="Bias length must equal E.m"):
        backend.ellpack_matmul(E, np.ones((6, 2), np.float32), np.ones(7, np.float32))
    x = np.arange(6, dtype=np.float32)
    y0 = backend.ellpack_matvec(E, x, None)                 # bias=None means no bias
    assert np.allclose(y0, backend.decode_from_ellpack(E) @ x, atol=1e-5)
    assert np.array_equal(E.Xt, x[E.idx])                   # what the reference leaves in Xt
    import cpp_backend
    assert np.array_equal(cpp_backend.matvec(E, x, np.zeros(8, np.float32)), y0)
    # float64 / Fortran-ordered inputs are force-cast like the reference does
    Y = backend.ellpack_matmul(E, np.asfortranarray(np.ones((6, 3))), np.zeros(8))
    assert Y.dtype == np.float32 and Y.shape == (8, 3)


def test_device_pointer_calls_and_row_shards(backend, orc, cuda):
    rng = np.random.default_rng(9)
    W = generate_sparse_matrix(100, 64, 0.8)
    X = rng.uniform(-1, 1, (64, 32)).astype(np.float32)
    b = rng.standard_normal(100).astype(np.float32)
    E = backend.convert_to_ellpack(W)
    want = orc.spmm(orc.encode(W), X, b)
    dX, dB = torch.from_numpy(X).to(cuda), torch.from_numpy(b).to(cuda)
    dY = torch.empty((100, 32), device=cuda)
    backend.ellpack_matmul_device(E, dX.data_ptr(), 32, 32, dB.data_ptr(), 0, dY.data_ptr(), 32)
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), want, "device spmm")
    # three row shards reproduce the unsharded result bit for bit
    parts = [backend.ellpack_matmul(E.shard_rows(g, 3), X, b[g * 34:(g + 1) * 34]) for g in range(3)]
    assert [p.shape[0] for p in parts] == [34, 34, 32]
    assert_bit_equal(np.concatenate(parts), want, "row shards")


def _load(backend, blob):
    f = tempfile.NamedTemporaryFile(suffix=".onnx", delete=False)
    f.write(blob)
    f.close()
    try:
        return backend.SparseOnnxModel(f.name)
    finally:
        os.unlink(f.name)


def test_model_mlp_golden(backend, golden, cuda):
    m = _load(backend, golden["mlp_onnx"].tobytes())
    x_mem = golden["mlp_x_mem"]                              # [features][B] memory
    B = x_mem.shape[1]
    y = m.run(x_mem.reshape(B, -1))                          # labelled (B, N): only the bytes matter
    assert list(y.shape) == golden["mlp_shape_ref"].tolist()
    want = golden["mlp_y_mem_ref"]
    # layers 1-2 are bit-exact; the final sigmoid/tanh differ from glibc by a few ulp
    assert np.abs(y.ravel() - want).max() <= 1e-6
    m2 = _load(backend, golden["mlp2_onnx"].tobytes())      # relu-only model: bit-exact end to end
    x2 = golden["mlp2_x_mem"]
    y2 = m2.run(x2.reshape(x2.shape[1], -1))
    assert_bit_equal(y2.ravel(), golden["mlp2_y_mem_ref"], "relu MLP")


def test_model_cnn_golden(backend, golden, cuda):
    m = _load(backend, golden["cnn_onnx"].tobytes())
    x_mem = golden["cnn_x_mem"]                              # [C,H,W,B]
    B = x_mem.shape[3]
    y = m.run(x_mem.reshape(B, *x_mem.shape[:3]))
    assert list(y.shape) == golden["cnn_shape_ref"].tolist()
    assert_bit_equal(y.ravel(), golden["cnn_y_mem_ref"], "conv-relu-conv-relu")


def test_model_resize_and_device_run(backend, golden, orc, cuda):
    m = _load(backend, golden["mlp2_onnx"].tobytes())
    x_mem = golden["mlp2_x_mem"]
    want = golden["mlp2_y_mem_ref"].reshape(-1, x_mem.shape[1])
    m.resize_buffers(3)                                      # a different batch: first three columns
    y3 = m.run(np.ascontiguousarray(x_mem[:, :3]).reshape(3, -1))
    assert_bit_equal(y3.ravel().reshape(-1, 3), want[:, :3], "batch 3")
    y5 = m.run(x_mem.reshape(5, -1))                         # back to 5: re-plans by itself
    assert_bit_equal(y5.ravel().reshape(-1, 5), want, "batch 5")
    dX = torch.from_numpy(x_mem).to(cuda)
    dY = torch.empty(want.shape, device=cuda)
    m.run_device(dX.data_ptr(), 5, dY.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), want, "device run")
    # resident replay of the captured loop on the model's own buffers
    m.resize_buffers(5)
    dX2 = torch.from_numpy(x_mem).to(cuda)
    n_in = dX2.numel() * 4
    import spx_ctypes as sx
    sx.Lib().spx_memcpy_d2d(m.device_input_ptr(), dX2.data_ptr(), n_in, 0)
    torch.cuda.synchronize()
    before = backend.launch_count()
    m.run_resident(0)
    assert backend.launch_count() == before + 2          # graph replays count their kernels (two fused layers)
    out = torch.empty(want.shape, device=cuda)
    sx.Lib().spx_memcpy_d2d(out.data_ptr(), m.device_output_ptr(), out.numel() * 4, 0)
    torch.cuda.synchronize()
    assert_bit_equal(out.cpu().numpy(), want, "resident run")


def test_model_scaled_config3_vs_oracle(backend, orc, cuda):
    import onnx_wire
    import workloads as wl
    d = wl.cfg3(0.1)
    m = _load(backend, onnx_wire.mlp_model(d["weights"], d["biases"], d["acts"], d["B"]))
    x_mem = np.ascontiguousarray(d["x"].T)
    y = m.run(x_mem.reshape(d["B"], -1)).ravel().reshape(-1, d["B"])
    a = x_mem
    for W, b, act in zip(d["weights"][:3], d["biases"][:3], (1, 1, 1)):
        a = orc.spmm(orc.encode(W), a, b, act=act)
    pre = orc.spmm(orc.encode(d["weights"][3]), a, d["biases"][3])
    assert np.abs(y - orc.activation(pre, 2)).max() <= 1e-6
    assert m.flops_per_run(d["B"]) == 2.0 * d["B"] * sum(int(np.count_nonzero(W)) for W in d["weights"])


def test_model_resnet_style_graph_vs_torch(backend, cuda):
    """conv-relu-maxpool, a residual block (conv-relu-conv, add, relu), global average pool, flatten,
    fully connected, sigmoid -- all in [C,H,W,B].  The reference itself is inconsistent on such graphs,
    so the check is against a dense fp32 torch evaluation (tolerance 1e-4 like the reference's scripts)."""
    import onnx_wire as ow
    import torch.nn.functional as F
    rng = np.random.default_rng(21)
    B, Cin, Cm, H, W = 4, 3, 8, 16, 16

    def sp(shape, p, scale):
        w = (rng.standard_normal(shape) * scale).astype(np.float32)
        w[rng.random(shape) >= p] = 0
        return w
    w1, b1 = sp((Cm, Cin, 3, 3), 0.5, 0.3), rng.standard_normal(Cm).astype(np.float32) * 0.1
    w2, b2 = sp((Cm, Cm, 3, 3), 0.3, 0.2), rng.standard_normal(Cm).astype(np.float32) * 0.1
    w3, b3 = sp((Cm, Cm, 3, 3), 0.3, 0.2), rng.standard_normal(Cm).astype(np.float32) * 0.1
    wf, bf = sp((10, Cm), 0.6, 0.5), rng.standard_normal(10).astype(np.float32) * 0.1
    conv = lambda i, w, b, o: ow.node("Conv", [i, w, b], [o], [ow.attr_ints("kernel_shape", [3, 3]), ow.attr_ints("pads", [1, 1, 1, 1])])
    nodes = [conv("input", "w1", "b1", "c1"), ow.node("Relu", ["c1"], ["r1"]),
             ow.node("MaxPool", ["r1"], ["p1"], [ow.attr_ints("kernel_shape", [3, 3]), ow.attr_ints("strides", [2, 2]), ow.attr_ints("pads", [1, 1, 1, 1])]),
             conv("p1", "w2", "b2", "c2"), ow.node("Relu", ["c2"], ["r2"]), conv("r2", "w3", "b3", "c3"),
             ow.node("Add", ["c3", "p1"], ["s"]), ow.node("Relu", ["s"], ["r3"]),
             ow.node("GlobalAveragePool", ["r3"], ["g"]), ow.node("Flatten", ["g"], ["f"]),
             ow.node("Gemm", ["f", "wf", "bf"], ["fc"], [ow.attr_int("transB", 1)]), ow.node("Sigmoid", ["fc"], ["y"])]
    inits = [ow.tensor(n, a) for n, a in (("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2), ("w3", w3), ("b3", b3), ("wf", wf), ("bf", bf))]
    m = _load(backend, ow.model(nodes, inits, ("input", (B, Cin, H, W)), ("y", (B, 10))))
    ops = [l["op"] for l in m.layer_summary()]
    assert ops == ["Conv", "MaxPool", "Conv", "Conv", "Add", "Relu", "GlobalAveragePool", "MatMul"]
    x = rng.standard_normal((B, Cin, H, W)).astype(np.float32)
    y_mem = m.run(np.ascontiguousarray(x.transpose(1, 2, 3, 0)).reshape(B, Cin, H, W))     # [C,H,W,B] bytes
    got = y_mem.ravel().reshape(10, B).T
    t = torch.from_numpy
    p1 = F.max_pool2d(F.relu(F.conv2d(t(x), t(w1), t(b1), padding=1)), 3, 2, 1)
    r3 = F.relu(F.conv2d(F.relu(F.conv2d(p1, t(w2), t(b2), padding=1)), t(w3), t(b3), padding=1) + p1)
    want = torch.sigmoid(F.linear(r3.mean((2, 3)), t(wf), t(bf))).numpy()
    assert np.abs(got - want).max() <= 1e-4
    # Activation buffers are reused by liveness (the reference frees an intermediate after its last
    # reader, src/model_run.cpp:116-127): nine tensors live in fewer buffers, p1 survives until the
    # Add that reads it, and the result is the same bytes as with one buffer per tensor.
    assert m.activation_buffers < len(ops) + 1
    again = m.run(np.ascontiguousarray(x.transpose(1, 2, 3, 0)).reshape(B, Cin, H, W))     # graph replay
    assert np.array_equal(again.view(np.uint32), y_mem.view(np.uint32))
    os.environ["SPX_NO_BUFFER_REUSE"] = "1"
    try:
        m2 = _load(backend, ow.model(nodes, inits, ("input", (B, Cin, H, W)), ("y", (B, 10))))
        y2 = m2.run(np.ascontiguousarray(x.transpose(1, 2, 3, 0)).reshape(B, Cin, H, W))
    finally:
        del os.environ["SPX_NO_BUFFER_REUSE"]
    assert m2.activation_buffers == len(ops) + 1
    assert np.array_equal(y2.view(np.uint32), y_mem.view(np.uint32))


def test_model_full_config3_vs_oracle(backend, orc, cuda):
    """Config 3 at its full size (4096-4096-4096-4096-1000, 90 % sparse, batch 256) through
    SparseOnnxModel.run against the oracle's layer loop: pre-sigmoid values are bit-identical
    chains, the final sigmoid may differ by a few ulp."""
    import onnx_wire
    import workloads as wl
    d = wl.cfg3(1.0)
    m = _load(backend, onnx_wire.mlp_model(d["weights"], d["biases"], d["acts"], d["B"]))
    assert [l["act"] for l in m.layer_summary()] == [1, 1, 1, 2]
    x_mem = np.ascontiguousarray(d["x"].T)
    y = m.run(x_mem.reshape(d["B"], -1)).ravel().reshape(-1, d["B"])
    a = x_mem
    for W, b in zip(d["weights"][:3], d["biases"][:3]):
        a = orc.spmm(orc.encode(W), a, b, act=1)
    want = orc.activation(orc.spmm(orc.encode(d["weights"][3]), a, d["biases"][3]), 2)
    assert y.shape == want.shape == (1000, 256)
    assert np.abs(y - want).max() <= 1e-6
    # the hidden layers on their own, bit for bit, through the device-pointer call
    E = backend.convert_to_ellpack(d["weights"][0])
    dX = torch.from_numpy(x_mem).to(cuda)
    dB = torch.from_numpy(d["biases"][0]).to(cuda)
    dY = torch.empty((4096, 256), device=cuda)
    backend.ellpack_matmul_device(E, dX.data_ptr(), 256, 256, dB.data_ptr(), 1, dY.data_ptr(), 256)
    torch.cuda.synchronize()
    assert_bit_equal(dY.cpu().numpy(), orc.spmm(orc.encode(d["weights"][0]), x_mem, d["biases"][0], act=1), "layer 1")


def test_model_conv_stack_config4_scaled_vs_oracle(backend, orc, cuda):
    """The 4-layer conv + bias + ReLU stack of config 4 at a quarter of its size, through
    SparseOnnxModel.run in [C,H,W,B] memory, bit-identical to the oracle layer by layer."""
    import onnx_wire
    import workloads as wl
    d = wl.cfg4(0.25, layers=4)
    B, Cc, H, W = d["B"], d["C"], d["H"], d["W"]
    m = _load(backend, onnx_wire.conv_model(d["weights"], d["biases"], [True] * 4, B, H, W))
    assert [l["op"] for l in m.layer_summary()] == ["Conv"] * 4 and all(l["act"] == 1 for l in m.layer_summary())
    x_pf = np.ascontiguousarray(d["x_nchw"].transpose(1, 2, 3, 0))
    y = m.run(x_pf.reshape(B, Cc, H, W)).ravel().reshape(Cc, H, W, B)
    g = dict(Cin=Cc, kH=3, kW=3, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
    a = x_pf
    for wgt, b in zip(d["weights"], d["biases"]):
        a = orc.conv2d(orc.encode(wgt.reshape(Cc, -1)), g, 0, a, B, b, 1)
    assert_bit_equal(y, a, "conv stack")


def test_python_onnx_sparse_model(backend, cuda):
    """OnnxSparseModel (the pure-Python loop of the reference's python/sparse_onnx.py) over these
    bindings: weights are encoded as stored, a 1-D input takes matvec, a 2-D (n, C) input matmul."""
    import onnx_wire as ow
    from sparse_onnx import OnnxSparseModel
    rng = np.random.default_rng(31)
    dims = [40, 64, 48, 10]
    Ws = [generate_sparse_matrix(dims[l + 1], dims[l], 0.6, seed=l) - 0.5 * (generate_sparse_matrix(dims[l + 1], dims[l], 0.6, seed=l) != 0)
          for l in range(3)]
    bs = [rng.standard_normal(dims[l + 1]).astype(np.float32) for l in range(3)]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mlp.onnx")
        with open(path, "wb") as f:
            f.write(ow.mlp_model(Ws, bs, ["Relu", "Tanh", "Sigmoid"], 8))
        model = OnnxSparseModel(path)
        bad = os.path.join(d, "conv.onnx")
        with open(bad, "wb") as f:
            f.write(ow.conv_model([rng.standard_normal((4, 3, 3, 3)).astype(np.float32)], [np.zeros(4, np.float32)], [True], 2, 8, 8))
        with pytest.raises(NotImplementedError):
            OnnxSparseModel(bad)
    assert [l[0] for l in model.layers] == ["matmul", "relu", "matmul", "tanh", "matmul", "sigmoid"]

    def dense(v):
        v = np.maximum(Ws[0].astype(np.float64) @ v + bs[0][(...,) + (None,) * (v.ndim - 1)], 0)
        v = np.tanh(Ws[1].astype(np.float64) @ v + bs[1][(...,) + (None,) * (v.ndim - 1)])
        return 1 / (1 + np.exp(-(Ws[2].astype(np.float64) @ v + bs[2][(...,) + (None,) * (v.ndim - 1)])))

    x1 = rng.standard_normal(40).astype(np.float32)
    X = rng.standard_normal((40, 8)).astype(np.float32)
    y1, Y = model.run(x1), model.run(X)
    assert y1.shape == (10,) and Y.shape == (10, 8) and Y.dtype == np.float32
    assert np.abs(y1 - dense(x1)).max() <= 1e-5 and np.abs(Y - dense(X)).max() <= 1e-5
