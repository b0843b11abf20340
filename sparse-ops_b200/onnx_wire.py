"""Minimal ONNX protobuf wire-format writer and reader (no `onnx` / protobuf package needed).

Produces the small subset of ONNX graphs that `SparseOnnxModel` loads: Gemm / MatMul / Conv /
Relu / Sigmoid / Tanh / Identity nodes, float32 initialisers, one static-shape input and
output.  Field numbers are those of the public ONNX schema (onnx.proto): ModelProto.graph=7,
GraphProto.node=1 / initializer=5 / input=11 / output=12, NodeProto.input=1 / output=2 /
op_type=4 / attribute=5, AttributeProto.name=1 / i=3 / ints=8 / type=20,
TensorProto.dims=1 / data_type=2 / float_data=4 / name=8 / raw_data=9.
"""
from __future__ import annotations

import numpy as np


def _varint(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire_type: int) -> bytes:
    return _varint((field << 3) | wire_type)


def _ld(field: int, payload: bytes) -> bytes:
    return _key(field, 2) + _varint(len(payload)) + payload


def _s(field: int, text: str) -> bytes:
    return _ld(field, text.encode())


def _i64(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(v)


def tensor(name: str, arr, packed_float_data: bool = False) -> bytes:
    """TensorProto with float32 data in raw_data (default) or packed float_data."""
    arr = np.ascontiguousarray(arr, dtype=np.float32)
    head = b"".join(_i64(1, d) for d in arr.shape) + _i64(2, 1)
    if packed_float_data:
        return head + _ld(4, arr.tobytes()) + _s(8, name)
    return head + _s(8, name) + _ld(9, arr.tobytes())


def value_info(name: str, shape) -> bytes:
    dims = b"".join(_ld(1, _i64(1, d)) for d in shape)
    return _s(1, name) + _ld(2, _ld(1, _i64(1, 1) + _ld(2, dims)))


def attr_int(name: str, v: int) -> bytes:
    return _s(1, name) + _i64(3, v) + _i64(20, 2)


def attr_ints(name: str, vs) -> bytes:
    return _s(1, name) + b"".join(_i64(8, v) for v in vs) + _i64(20, 7)


def node(op: str, inputs, outputs, attrs=()) -> bytes:
    return (b"".join(_s(1, x) for x in inputs) + b"".join(_s(2, x) for x in outputs)
            + _s(4, op) + b"".join(_ld(5, a) for a in attrs))


def model(nodes, initializers, graph_input, graph_output, opset: int = 14) -> bytes:
    """graph_input / graph_output are (name, shape) tuples."""
    g = (b"".join(_ld(1, n) for n in nodes) + _s(2, "g")
         + b"".join(_ld(5, t) for t in initializers)
         + _ld(11, value_info(*graph_input)) + _ld(12, value_info(*graph_output)))
    return _i64(1, 8) + _ld(8, _s(1, "") + _i64(2, opset)) + _ld(7, g)


def mlp_model(weights, biases, acts, batch: int) -> bytes:
    """Gemm(transB=1, with bias) layers, each followed by acts[l] in {None,'Relu','Sigmoid','Tanh'}.

    weights[l] is (out_features, in_features)."""
    nodes, inits = [], []
    cur = "input"
    for l, (W, b) in enumerate(zip(weights, biases)):
        inits.append(tensor(f"W{l}", W))
        ins = [cur, f"W{l}"]
        if b is not None:
            inits.append(tensor(f"b{l}", b))
            ins.append(f"b{l}")
        out = f"fc{l}"
        nodes.append(node("Gemm", ins, [out], [attr_int("transB", 1)]))
        cur = out
        if acts[l]:
            out = f"act{l}"
            nodes.append(node(acts[l], [cur], [out]))
            cur = out
    n_in = weights[0].shape[1]
    n_out = weights[-1].shape[0]
    # the last tensor name becomes the graph output
    return model(nodes, inits, ("input", (batch, n_in)), (cur, (batch, n_out)))


def conv_model(weights, biases, relus, batch: int, H: int, W: int, stride=1, pad=1, dil=1) -> bytes:
    """Chain of Conv (+ optional Relu) layers; weights[l] is (Cout, Cin, kH, kW)."""
    nodes, inits = [], []
    cur = "input"
    h, w = H, W
    for l, (Wt, b) in enumerate(zip(weights, biases)):
        inits.append(tensor(f"W{l}", Wt))
        ins = [cur, f"W{l}"]
        if b is not None:
            inits.append(tensor(f"b{l}", b))
            ins.append(f"b{l}")
        kH, kW = Wt.shape[2], Wt.shape[3]
        out = f"conv{l}"
        nodes.append(node("Conv", ins, [out], [
            attr_ints("kernel_shape", [kH, kW]), attr_ints("strides", [stride, stride]),
            attr_ints("pads", [pad, pad, pad, pad]), attr_ints("dilations", [dil, dil]),
            attr_int("group", 1)]))
        h = (h + 2 * pad - (dil * (kH - 1) + 1)) // stride + 1
        w = (w + 2 * pad - (dil * (kW - 1) + 1)) // stride + 1
        cur = out
        if relus[l]:
            out = f"relu{l}"
            nodes.append(node("Relu", [cur], [out]))
            cur = out
    cin = weights[0].shape[1]
    cout = weights[-1].shape[0]
    return model(nodes, inits, ("input", (batch, cin, H, W)), (cur, (batch, cout, h, w)))


# ---- reader (the subset the pure-Python runtime sparse_onnx.OnnxSparseModel needs) --------------
def _fields(buf: bytes):
    """Yields (field number, wire type, value) of one message; value is an int (varint, fixed) or bytes."""
    i, n = 0, len(buf)
    while i < n:
        key = shift = 0
        while True:
            b = buf[i]; i += 1
            key |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                break
        field, wt = key >> 3, key & 7
        if wt == 0:
            v = shift = 0
            while True:
                b = buf[i]; i += 1
                v |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            yield field, wt, v
        elif wt == 1:
            yield field, wt, int.from_bytes(buf[i:i + 8], "little"); i += 8
        elif wt == 5:
            yield field, wt, int.from_bytes(buf[i:i + 4], "little"); i += 4
        elif wt == 2:
            ln = shift = 0
            while True:
                b = buf[i]; i += 1
                ln |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            if i + ln > n:
                raise ValueError("truncated ONNX file")
            yield field, wt, bytes(buf[i:i + ln]); i += ln
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")


def _varints(payload: bytes):
    out, v, shift = [], 0, 0
    for b in payload:
        v |= (b & 0x7F) << shift
        shift += 7
        if not b & 0x80:
            out.append(v); v = shift = 0
    return out


def _read_tensor(buf: bytes):
    dims, dtype, name, raw, floats = [], 1, "", None, []
    for f, wt, v in _fields(buf):
        if f == 1:
            dims += _varints(v) if wt == 2 else [v]
        elif f == 2:
            dtype = v
        elif f == 4:                                   # float_data, packed or one fixed32 each
            floats.append(v if wt == 2 else int(v).to_bytes(4, "little"))
        elif f == 8:
            name = v.decode()
        elif f == 9:
            raw = v
    if dtype != 1:
        return name, None                              # only float32 initialisers carry weights here
    data = raw if raw is not None else b"".join(floats)
    return name, np.frombuffer(data, dtype="<f4").reshape(dims).copy()


def _read_node(buf: bytes):
    nd = dict(op_type="", input=[], output=[], attrs={})
    for f, wt, v in _fields(buf):
        if f == 1:
            nd["input"].append(v.decode())
        elif f == 2:
            nd["output"].append(v.decode())
        elif f == 4:
            nd["op_type"] = v.decode()
        elif f == 5:
            name, val, ints = "", None, []
            for af, awt, av in _fields(v):
                if af == 1:
                    name = av.decode()
                elif af == 3:
                    val = av - (1 << 64) if av >> 63 else av
                elif af == 8:
                    ints += _varints(av) if awt == 2 else [av]
            nd["attrs"][name] = ints if ints else val
    return nd


def read_model(data: bytes):
    """Parses ModelProto bytes into {'nodes': [...], 'initializers': {name: float32 array}}."""
    graph = None
    for f, wt, v in _fields(data):
        if f == 7 and wt == 2:
            graph = v
    if graph is None:
        raise ValueError("no graph in ONNX file")
    nodes, inits = [], {}
    for f, wt, v in _fields(graph):
        if f == 1 and wt == 2:
            nodes.append(_read_node(v))
        elif f == 5 and wt == 2:
            name, arr = _read_tensor(v)
            if arr is not None:
                inits[name] = arr
    return dict(nodes=nodes, initializers=inits)
