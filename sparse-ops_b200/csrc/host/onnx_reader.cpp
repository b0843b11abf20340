// onnx_reader.cpp -- see onnx_reader.hpp.
#include "onnx_reader.hpp"

#include <cstring>
#include <fstream>
#include <iterator>
#include <stdexcept>

namespace spx {
namespace onnx {
namespace {

struct ParseError : std::runtime_error {
    ParseError() : std::runtime_error("malformed protobuf") {}
};

// Cursor over one length-delimited region.
struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    bool more() const { return p < end; }
    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 70; shift += 7) {
            if (p >= end) throw ParseError();
            const uint8_t b = *p++;
            v |= uint64_t(b & 0x7f) << (shift < 64 ? shift : 63);
            if (!(b & 0x80)) return v;
        }
        throw ParseError();
    }
    Cursor sub() {
        const uint64_t n = varint();
        if (n > uint64_t(end - p)) throw ParseError();
        Cursor c{p, p + n};
        p += n;
        return c;
    }
    std::string bytes() {
        Cursor c = sub();
        return std::string(reinterpret_cast<const char*>(c.p), size_t(c.end - c.p));
    }
    void skip(int wire_type) {
        switch (wire_type) {
        case 0: varint(); break;
        case 1: if (end - p < 8) throw ParseError(); p += 8; break;
        case 2: sub(); break;
        case 5: if (end - p < 4) throw ParseError(); p += 4; break;
        default: throw ParseError();
        }
    }
    float fixed32f() {
        if (end - p < 4) throw ParseError();
        float f;
        std::memcpy(&f, p, 4);
        p += 4;
        return f;
    }
};

#define SPX_FIELDS(cur) while ((cur).more()) { const uint64_t key_ = (cur).varint(); \
    const int field = int(key_ >> 3); const int wt = int(key_ & 7); (void)field; (void)wt;
#define SPX_END_FIELDS }

void repeated_i64(Cursor& c, int wt, std::vector<int64_t>& out) {
    if (wt == 0) out.push_back(int64_t(c.varint()));
    else if (wt == 2) { Cursor s = c.sub(); while (s.more()) out.push_back(int64_t(s.varint())); }
    else c.skip(wt);
}

Attribute parse_attribute(Cursor c) {
    Attribute a;
    SPX_FIELDS(c)
        if (field == 1 && wt == 2) a.name = c.bytes();
        else if (field == 3 && wt == 0) a.i = int64_t(c.varint());
        else if (field == 8) repeated_i64(c, wt, a.ints);
        else c.skip(wt);
    SPX_END_FIELDS
    return a;
}

Node parse_node(Cursor c) {
    Node n;
    SPX_FIELDS(c)
        if (field == 1 && wt == 2) n.inputs.push_back(c.bytes());
        else if (field == 2 && wt == 2) n.outputs.push_back(c.bytes());
        else if (field == 4 && wt == 2) n.op_type = c.bytes();
        else if (field == 5 && wt == 2) n.attributes.push_back(parse_attribute(c.sub()));
        else c.skip(wt);
    SPX_END_FIELDS
    return n;
}

Tensor parse_tensor(Cursor c) {
    Tensor t;
    SPX_FIELDS(c)
        if (field == 1) repeated_i64(c, wt, t.dims);
        else if (field == 2 && wt == 0) t.data_type = int32_t(c.varint());
        else if (field == 4 && wt == 2) { Cursor s = c.sub(); while (s.more()) t.float_data.push_back(s.fixed32f()); }
        else if (field == 4 && wt == 5) t.float_data.push_back(c.fixed32f());
        else if (field == 8 && wt == 2) t.name = c.bytes();
        else if (field == 9 && wt == 2) { t.raw_data = c.bytes(); t.has_raw = true; }
        else c.skip(wt);
    SPX_END_FIELDS
    return t;
}

Dim parse_dim(Cursor c) {
    Dim d;
    SPX_FIELDS(c)
        if (field == 1 && wt == 0) { d.has_value = true; d.value = int64_t(c.varint()); }
        else c.skip(wt);
    SPX_END_FIELDS
    return d;
}

void parse_shape(Cursor c, std::vector<Dim>& out) {
    SPX_FIELDS(c)
        if (field == 1 && wt == 2) out.push_back(parse_dim(c.sub()));
        else c.skip(wt);
    SPX_END_FIELDS
}

void parse_tensor_type(Cursor c, std::vector<Dim>& out) {
    SPX_FIELDS(c)
        if (field == 2 && wt == 2) parse_shape(c.sub(), out);
        else c.skip(wt);
    SPX_END_FIELDS
}

void parse_type(Cursor c, std::vector<Dim>& out) {
    SPX_FIELDS(c)
        if (field == 1 && wt == 2) parse_tensor_type(c.sub(), out);
        else c.skip(wt);
    SPX_END_FIELDS
}

ValueInfo parse_value_info(Cursor c) {
    ValueInfo v;
    SPX_FIELDS(c)
        if (field == 1 && wt == 2) v.name = c.bytes();
        else if (field == 2 && wt == 2) parse_type(c.sub(), v.shape);
        else c.skip(wt);
    SPX_END_FIELDS
    return v;
}

Graph parse_graph(Cursor c) {
    Graph g;
    SPX_FIELDS(c)
        if (field == 1 && wt == 2) g.nodes.push_back(parse_node(c.sub()));
        else if (field == 5 && wt == 2) g.initializers.push_back(parse_tensor(c.sub()));
        else if (field == 11 && wt == 2) g.inputs.push_back(parse_value_info(c.sub()));
        else if (field == 12 && wt == 2) g.outputs.push_back(parse_value_info(c.sub()));
        else c.skip(wt);
    SPX_END_FIELDS
    return g;
}

}  // namespace

std::vector<float> Tensor::floats() const {
    size_t size = 1;
    for (int64_t d : dims) size *= size_t(d);
    std::vector<float> out(size);
    if (has_raw && !raw_data.empty()) {
        if (raw_data.size() < size * sizeof(float)) throw std::runtime_error("ONNX tensor raw_data shorter than its shape");
        std::memcpy(out.data(), raw_data.data(), size * sizeof(float));
    } else if (!float_data.empty()) {
        if (float_data.size() > size) throw std::runtime_error("ONNX tensor float_data longer than its shape");
        std::memcpy(out.data(), float_data.data(), float_data.size() * sizeof(float));
    } else {
        throw std::runtime_error("ONNX tensor has no weight data");
    }
    return out;
}

Graph parse_model(const uint8_t* data, size_t size) {
    Cursor c{data, data + size};
    Graph g;
    SPX_FIELDS(c)
        if (field == 7 && wt == 2) g = parse_graph(c.sub());
        else c.skip(wt);
    SPX_END_FIELDS
    return g;
}

Graph load_graph(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open/parse ONNX file: " + path);
    std::string buf((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    try {
        return parse_model(reinterpret_cast<const uint8_t*>(buf.data()), buf.size());
    } catch (const ParseError&) {
        throw std::runtime_error("Failed to open/parse ONNX file: " + path);
    }
}

}  // namespace onnx
}  // namespace spx
