// onnx_reader.hpp -- minimal reader for the ONNX protobuf wire format.
//
// The reference parses models with libprotobuf and the generated onnx.pb.h
// (src/sparse_onnx.cpp:5,101-107).  This reader decodes only the fields that loader touches,
// straight from the wire format, so the library has no protobuf dependency.  Field numbers are
// those of the public ONNX schema: ModelProto.graph=7; GraphProto.node=1, initializer=5,
// input=11, output=12; NodeProto.input=1, output=2, op_type=4, attribute=5;
// AttributeProto.name=1, i=3, ints=8; TensorProto.dims=1, data_type=2, float_data=4, name=8,
// raw_data=9; ValueInfoProto.name=1, type=2; TypeProto.tensor_type=1; Tensor.shape=2;
// TensorShapeProto.dim=1; Dimension.dim_value=1.  Packed and unpacked repeated scalars are
// both accepted.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace spx {
namespace onnx {

struct Attribute {
    std::string name;
    int64_t i = 0;
    std::vector<int64_t> ints;
};

struct Node {
    std::string op_type;
    std::vector<std::string> inputs, outputs;
    std::vector<Attribute> attributes;
    const Attribute* find(const std::string& name) const {
        for (const auto& a : attributes) if (a.name == name) return &a;
        return nullptr;
    }
};

struct Tensor {
    std::string name;
    std::vector<int64_t> dims;
    int32_t data_type = 0;
    std::string raw_data;
    bool has_raw = false;
    std::vector<float> float_data;
    // Flattened float32 contents (raw_data first, else float_data) -- the order of
    // parseTensor, src/sparse_onnx.cpp:55-78.  Throws std::runtime_error when empty.
    std::vector<float> floats() const;
};

struct Dim {
    bool has_value = false;
    int64_t value = 0;
};

struct ValueInfo {
    std::string name;
    std::vector<Dim> shape;
};

struct Graph {
    std::vector<Node> nodes;
    std::vector<Tensor> initializers;
    std::vector<ValueInfo> inputs, outputs;
};

// Throws std::runtime_error("Failed to open/parse ONNX file: <path>") like the reference.
Graph load_graph(const std::string& path);
Graph parse_model(const uint8_t* data, size_t size);

}  // namespace onnx
}  // namespace spx
