"""CPU: host-side logic above the C ABI -- encoder, ONNX wire reader + planner, RBM plan,
workload generators -- against the golden vectors of the reference."""
import os
import tempfile

import numpy as np
import pytest

from conftest import assert_bit_equal


@pytest.mark.parametrize("name", ["enc_hand", "enc_special", "enc_zero", "enc_rand"])
def test_host_encoder_bit_exact(backend, golden, name):
    E = backend.encode_host(golden[name + "_W"])
    assert (E.m, E.n) == golden[name + "_W"].shape
    assert E.r == golden[name + "_Wd_ref"].shape[1]
    assert_bit_equal(E.Wd, golden[name + "_Wd_ref"], "Wd")
    assert np.array_equal(E.idx, golden[name + "_idx_ref"])
    assert np.array_equal(E.nnz, golden[name + "_nnz_ref"])
    assert_bit_equal(backend.decode_from_ellpack(E), golden[name + "_decoded_ref"], "decode")
    assert not E.on_device


def test_host_encoder_accepts_float64_and_fortran_input(backend, golden):
    W = golden["enc_rand_W"]
    for variant in (W.astype(np.float64), np.asfortranarray(W)):
        E = backend.encode_host(variant)
        assert np.array_equal(E.idx, golden["enc_rand_idx_ref"])
    with pytest.raises(RuntimeError):
        backend.encode_host(np.zeros(5, np.float32))


def test_large_encode_uses_threads_and_matches_numpy(backend):
    rng = np.random.default_rng(3)
    W = rng.standard_normal((1500, 1200)).astype(np.float32)
    W[rng.random(W.shape) >= 0.1] = 0
    E = backend.encode_host(W)
    assert E.r == np.count_nonzero(W, axis=1).max()
    assert np.array_equal(backend.decode_from_ellpack(E), W)


def _write(blob):
    f = tempfile.NamedTemporaryFile(suffix=".onnx", delete=False)
    f.write(blob)
    f.close()
    return f.name


def test_planner_mlp(backend, golden):
    path = _write(golden["mlp_onnx"].tobytes())
    try:
        m = backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)
    assert m.output_shape() == golden["mlp_shape_ref"].tolist()
    assert (m.batch, m.in_features, m.out_features) == (16, 40, 10)
    L = m.layer_summary()
    # Gemm+Relu, Gemm+Tanh, Gemm+Sigmoid collapse to three fused MatMul layers
    assert [l["op"] for l in L] == ["MatMul"] * 3
    assert [l["act"] for l in L] == [1, 3, 2]
    assert all(l["bias"] for l in L)


def test_planner_gemm_matmul_orientation(backend):
    import onnx_wire as ow
    rng = np.random.default_rng(5)
    W = rng.standard_normal((6, 4)).astype(np.float32)      # (M=6 out, N=4 in)
    cases = {
        "gemm_transB1": ow.node("Gemm", ["input", "W"], ["y"], [ow.attr_int("transB", 1)]),
        "gemm_default": ow.node("Gemm", ["input", "W"], ["y"]),               # missing transB means 1
        "gemm_transB0": ow.node("Gemm", ["input", "Wt"], ["y"], [ow.attr_int("transB", 0)]),
        "matmul": ow.node("MatMul", ["input", "Wt"], ["y"]),
    }
    for name, nd in cases.items():
        inits = [ow.tensor("W", W), ow.tensor("Wt", W.T.copy(), packed_float_data=True)]
        path = _write(ow.model([nd], inits, ("input", (2, 4)), ("y", (2, 6))))
        try:
            m = backend.SparseOnnxModel(path, upload_weights=False)
        finally:
            os.unlink(path)
        l = m.layer_summary()[0]
        assert (l["m"], l["n"]) == (6, 4), name
        assert l["nnz"] == 24


def test_planner_conv_and_errors(backend, golden):
    path = _write(golden["cnn_onnx"].tobytes())
    try:
        m = backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)
    assert m.output_shape() == golden["cnn_shape_ref"].tolist()
    L = m.layer_summary()
    assert [l["op"] for l in L] == ["Conv", "Conv"] and [l["act"] for l in L] == [1, 1]
    assert L[0]["n"] == 6 * 9

    import onnx_wire as ow
    with pytest.raises(RuntimeError, match="Failed to open/parse ONNX file"):
        backend.SparseOnnxModel("/nonexistent/model.onnx", upload_weights=False)
    bad = ow.model([ow.node("Softmax", ["input"], ["y"])], [], ("input", (2, 4)), ("y", (2, 4)))
    path = _write(bad)
    try:
        with pytest.raises(RuntimeError, match="Unsupported ONNX op: Softmax"):
            backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)
    w = np.ones((4, 2, 3, 3), np.float32)
    grouped = ow.model([ow.node("Conv", ["input", "W"], ["y"], [ow.attr_int("group", 2)])], [ow.tensor("W", w)],
                       ("input", (1, 4, 5, 5)), ("y", (1, 4, 3, 3)))
    path = _write(grouped)
    try:
        with pytest.raises(RuntimeError):
            backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)


def test_identity_alias_and_unfusable_activation(backend):
    import onnx_wire as ow
    W = np.eye(3, dtype=np.float32)
    nodes = [ow.node("Gemm", ["input", "W"], ["a"]), ow.node("Identity", ["a"], ["b"]),
             ow.node("Relu", ["b"], ["c"]), ow.node("Add", ["c", "b"], ["d"])]
    path = _write(ow.model(nodes, [ow.tensor("W", W)], ("input", (2, 3)), ("d", (2, 3))))
    try:
        m = backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)
    L = m.layer_summary()
    # the Gemm output feeds both Relu and Add, so the Relu must stay a separate layer
    assert [l["op"] for l in L] == ["MatMul", "Relu", "Add"]
    assert L[0]["act"] == 0 and L[2]["inputs"] == ["c", "a"]


def test_rbm_plan_matches_reference(backend, golden):
    E = backend.encode_host(golden["conv_a_weight"].reshape(16, -1))
    blocks = backend.build_rbm_from_ellpack(E, golden["conv_a_bias"], 8)
    assert [b["M0"] for b in blocks] == golden["rbm_M0"].tolist()
    assert [b["Ct"] for b in blocks] == golden["rbm_Ct"].tolist()
    assert [len(b["krel"]) for b in blocks] == golden["rbm_krel_len"].tolist()
    cat = lambda k: np.concatenate([b[k] for b in blocks])
    assert np.array_equal(cat("krel"), golden["rbm_krel_ref"])
    assert np.array_equal(cat("colptr"), golden["rbm_colptr_ref"])
    assert np.array_equal(cat("rows"), golden["rbm_rows_ref"])
    assert_bit_equal(cat("w"), golden["rbm_w_ref"], "pair weights")
    assert_bit_equal(cat("bias"), golden["rbm_bias_ref"], "bias")


def test_workload_generators_are_seeded_and_shardable():
    import workloads as wl
    a, b = wl.cfg1(0.02), wl.cfg1(0.02)
    assert np.array_equal(a["W"], b["W"]) and np.array_equal(a["X"], b["X"])
    # a rank's row range of config 5 reproduces the rows of the whole matrix
    rp, col, val = wl.cfg5_rows(0, 8192, n=4096, kmax=256, mean=16, block_rows=4096)
    rp2, col2, val2 = wl.cfg5_rows(4096, 4096, n=4096, kmax=256, mean=16, block_rows=4096)
    s = int(rp[4096])
    assert np.array_equal(col[s:], col2) and np.array_equal(val[s:], val2)
    nnz = np.diff(rp)
    assert nnz.max() == 256 and 8 < nnz.mean() < 24
    # strictly ascending columns inside every row
    d = np.diff(col.astype(np.int64))
    row_starts = rp[1:-1].astype(np.int64)
    mask = np.ones(len(d), bool)
    mask[row_starts[(row_starts > 0) & (row_starts < len(col))] - 1] = False
    assert (d[mask] > 0).all()
    Wd, idx, n3 = wl.csr_to_ell(8192, rp, col, val)
    assert Wd.shape == (8192, 256) and np.array_equal(n3, nnz.astype(np.uint32))


def test_planner_cnn_with_pools_and_flatten(backend):
    import onnx_wire as ow
    rng = np.random.default_rng(8)
    w1 = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    wf = rng.standard_normal((7, 4 * 4 * 4)).astype(np.float32)
    nodes = [ow.node("Conv", ["input", "w1"], ["c1"], [ow.attr_ints("kernel_shape", [3, 3]), ow.attr_ints("pads", [1, 1, 1, 1])]),
             ow.node("Relu", ["c1"], ["r1"]),
             ow.node("MaxPool", ["r1"], ["p1"], [ow.attr_ints("kernel_shape", [2, 2]), ow.attr_ints("strides", [2, 2])]),
             ow.node("Flatten", ["p1"], ["f"], [ow.attr_int("axis", 1)]),
             ow.node("Gemm", ["f", "wf"], ["y"], [ow.attr_int("transB", 1)])]
    path = _write(ow.model(nodes, [ow.tensor("w1", w1), ow.tensor("wf", wf)], ("input", (2, 3, 8, 8)), ("y", (2, 7))))
    try:
        m = backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)
    L = m.layer_summary()
    assert [l["op"] for l in L] == ["Conv", "MaxPool", "MatMul"]      # Relu fused, Flatten is an alias
    assert L[0]["act"] == 1 and L[2]["inputs"] == ["p1"] and L[2]["n"] == 64
    assert m.output_shape() == [2, 7]
    gap = [ow.node("GlobalAveragePool", ["input"], ["g"]), ow.node("Flatten", ["g"], ["y"])]
    path = _write(ow.model(gap, [], ("input", (2, 3, 8, 8)), ("y", (2, 3))))
    try:
        m = backend.SparseOnnxModel(path, upload_weights=False)
    finally:
        os.unlink(path)
    assert [l["op"] for l in m.layer_summary()] == ["GlobalAveragePool"] and m.output_shape() == [2, 3]


def test_python_onnx_reader_round_trip():
    """The pure-Python reader behind sparse_onnx.OnnxSparseModel parses what the writer emits:
    nodes, attributes, raw_data and packed float_data initialisers."""
    import onnx_wire as ow
    rng = np.random.default_rng(5)
    Ws = [rng.standard_normal((6, 5)).astype(np.float32), rng.standard_normal((3, 6)).astype(np.float32)]
    bs = [rng.standard_normal(6).astype(np.float32), rng.standard_normal(3).astype(np.float32)]
    m = ow.read_model(ow.mlp_model(Ws, bs, ["Relu", "Sigmoid"], 4))
    assert [n["op_type"] for n in m["nodes"]] == ["Gemm", "Relu", "Gemm", "Sigmoid"]
    assert m["nodes"][0]["input"] == ["input", "W0", "b0"] and m["nodes"][0]["attrs"] == {"transB": 1}
    for l in range(2):
        assert np.array_equal(m["initializers"][f"W{l}"], Ws[l]) and np.array_equal(m["initializers"][f"b{l}"], bs[l])
    packed = ow.model([ow.node("MatMul", ["input", "W"], ["out"])], [ow.tensor("W", Ws[0].T, packed_float_data=True)],
                      ("input", (4, 6)), ("out", (4, 5)))
    assert np.array_equal(ow.read_model(packed)["initializers"]["W"], Ws[0].T)
    conv = ow.read_model(ow.conv_model([rng.standard_normal((4, 3, 3, 3)).astype(np.float32)], [np.zeros(4, np.float32)],
                                       [True], 2, 8, 8, stride=2, pad=1, dil=1))
    assert conv["nodes"][0]["attrs"]["strides"] == [2, 2] and conv["nodes"][0]["attrs"]["pads"] == [1, 1, 1, 1]
    with pytest.raises(ValueError):
        ow.read_model(ow.mlp_model(Ws, bs, ["Relu", None], 4)[:-7])      # truncated file


def test_python_onnx_reader_random_graphs():
    """Writer -> reader round trip over random small graphs: node order, operand names, integer
    attributes (negative values too) and tensors of any rank survive."""
    import onnx_wire as ow
    rng = np.random.default_rng(11)
    for trial in range(25):
        n_nodes = int(rng.integers(1, 6))
        inits, nodes, want = [], [], []
        prev = "input"
        for i in range(n_nodes):
            op = str(rng.choice(["Gemm", "MatMul", "Relu", "Conv", "Identity"]))
            shape = tuple(int(d) for d in rng.integers(1, 5, size=int(rng.integers(1, 5))))
            t = rng.standard_normal(shape).astype(np.float32)
            name = f"t{trial}_{i}"
            inits.append(ow.tensor(name, t, packed_float_data=bool(rng.integers(0, 2))))
            attrs = {"a": int(rng.integers(-5, 6)), "ks": [int(v) for v in rng.integers(0, 9, size=3)]}
            nodes.append(ow.node(op, [prev, name], [f"o{i}"], [ow.attr_int("a", attrs["a"]), ow.attr_ints("ks", attrs["ks"])]))
            want.append((op, [prev, name], [f"o{i}"], attrs, name, t))
            prev = f"o{i}"
        m = ow.read_model(ow.model(nodes, inits, ("input", (2, 3)), (prev, (2, 3))))
        assert len(m["nodes"]) == n_nodes
        for nd, (op, ins, outs, attrs, name, t) in zip(m["nodes"], want):
            assert nd["op_type"] == op and nd["input"] == ins and nd["output"] == outs and nd["attrs"] == attrs
            got = m["initializers"][name]
            assert got.shape == t.shape and np.array_equal(got, t)


def test_conv_workload_density_parameter():
    import workloads as wl
    d = wl.cfg4(0.1, layers=1, density=0.5)
    w = d["weights"][0]
    frac = np.count_nonzero(w) / w.size
    assert 0.35 < frac < 0.65
    d2 = wl.cfg4(0.1, layers=1)                     # default: 80 % sparse
    assert 0.1 < np.count_nonzero(d2["weights"][0]) / d2["weights"][0].size < 0.3


def test_balanced_row_split(backend):
    """Row ranges of near-equal work for matrices whose long rows cluster; equal row counts
    (shard_rows) would give the first rank most of the nonzeros here."""
    rng = np.random.default_rng(8)
    m, n, G = 4000, 300, 8
    W = rng.standard_normal((m, n)).astype(np.float32)
    W[rng.random(W.shape) >= 0.02] = 0
    W[:200] = rng.standard_normal((200, n)).astype(np.float32)       # 200 dense rows up front
    E = backend.encode_host(W)
    b = E.balanced_row_split(G, 0)
    assert len(b) == G + 1 and b[0] == 0 and b[-1] == m and all(x <= y for x, y in zip(b, b[1:]))
    per = [int(E.nnz[b[g]:b[g + 1]].sum()) for g in range(G)]
    share = E.nnz_total / G
    assert max(per) <= share + E.nnz.max()                 # never more than one row over the share
    equal = [int(E.nnz[g * 500:(g + 1) * 500].sum()) for g in range(G)]
    assert max(equal) > 3 * max(per)                       # what the equal split would have given
    # shards are the parent's rows, r kept
    S = E.shard_range(b[1], b[2], upload=False)
    assert (S.m, S.n, S.r) == (b[2] - b[1], n, E.r)
    assert np.array_equal(S.idx, E.idx[b[1]:b[2]]) and np.array_equal(S.nnz, E.nnz[b[1]:b[2]])
    # with a per-row cost, empty rows are spread too
    Z = backend.encode_host(np.zeros((10, 4), np.float32))
    assert Z.balanced_row_split(5) == [0, 2, 4, 6, 8, 10]
    assert backend.encode_host(np.ones((2, 3), np.float32)).balanced_row_split(4)[-1] == 2
    with pytest.raises(RuntimeError):
        E.shard_range(5, 4, upload=False)
    with pytest.raises(RuntimeError):
        E.balanced_row_split(0)
