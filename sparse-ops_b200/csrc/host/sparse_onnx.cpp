// sparse_onnx.cpp -- loader / planner and the GPU layer loop of SparseOnnxModel.
#include "sparse_onnx.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>

#include "onnx_reader.hpp"

namespace spx {

namespace {

void transpose_rc(const std::vector<float>& A, uint32_t R, uint32_t C, std::vector<float>& AT)
{
    AT.resize(size_t(R) * C);
    for (uint32_t r = 0; r < R; ++r)
        for (uint32_t c = 0; c < C; ++c) AT[size_t(c) * R + r] = A[size_t(r) * C + c];
}

}  // namespace

// Device-side execution state for one batch size.
struct SparseOnnxModel::Exec {
    uint32_t B = 0;
    void* stream = nullptr;
    void* graph = nullptr;
    float* d_bias = nullptr;
    std::unordered_map<std::string, float*> buf;      // tensor name -> device buffer
    std::unordered_map<std::string, uint64_t> rows;   // tensor name -> rows (elements per column)
    std::vector<void*> owned;
    size_t distinct_buffers = 0;       // activation buffers actually allocated (fewer than tensors when reused)
    // Small results leave the device through a pinned staging buffer: a device -> host copy into
    // the caller's pageable array goes through the driver's bounce buffer in serialised chunks.
    float* h_out = nullptr;
    size_t h_out_bytes = 0;
    // Row-sharded mode with the exchange fused into the SpMM epilogue: for every MatMul output the
    // full buffer of each rank (own pointer + peers' buffers opened over IPC), indexed by rank.
    bool fused = false;
    std::unordered_map<std::string, std::vector<float*>> peers;
    std::vector<void*> opened;
    spx_comm* comm = nullptr;          // not owned
    ~Exec() {
        if (graph) spx_graph_destroy(graph);
        for (void* p : opened) spx_ipc_close(p);
        if (fused && comm && stream) {
            // every rank has unmapped the others' buffers before anybody frees its own
            if (spx_comm_barrier(comm, stream) == SPX_OK) spx_stream_sync(stream);
        }
        for (void* p : owned) spx_free(p);
        spx_free(d_bias);
        spx_host_free(h_out);
        if (stream) spx_stream_destroy(stream);
    }
};

SparseOnnxModel::~SparseOnnxModel()
{
    exec_.reset();
    spx_comm_destroy(comm_);
}

SparseOnnxModel::SparseOnnxModel(const std::string& onnx_path, bool upload_weights)
{
    auto resolve = [this](const std::string& nm) -> std::string {
        std::string cur = nm;
        for (auto it = name_alias_.find(cur); it != name_alias_.end(); it = name_alias_.find(cur)) cur = it->second;
        return cur;
    };

    const onnx::Graph graph = onnx::load_graph(onnx_path);

    std::unordered_map<std::string, const onnx::Tensor*> init_map;
    for (const auto& t : graph.initializers) init_map[t.name] = &t;

    // Model input = first graph input that is not an initializer (src/sparse_onnx.cpp:118-129).
    const onnx::ValueInfo* in_vi = nullptr;
    for (const auto& vi : graph.inputs)
        if (!init_map.count(vi.name)) { in_vi = &vi; break; }
    if (!in_vi) throw std::runtime_error("No non-initializer input found in ONNX graph");
    input_name_ = resolve(in_vi->name);
    if (graph.outputs.size() != 1) throw std::runtime_error("Expected exactly one graph output");
    output_name_ = resolve(graph.outputs[0].name);

    // Static input shape; batch = dim 0, features = product of the rest (:138-167).
    for (const auto& d : in_vi->shape) {
        if (!d.has_value) throw std::runtime_error("Dynamic dims not supported");
        input_shape_.push_back(int(d.value));
    }
    if (input_shape_.size() < 2) throw std::runtime_error("Input tensor must have rank \xE2\x89\xA5 2");
    uint32_t prod = 1;
    for (size_t d = 1; d < input_shape_.size(); ++d) prod *= uint32_t(input_shape_[d]);
    in_features_ = prod;
    batch_dim_ = uint32_t(input_shape_[0]);
    shape_map_[input_name_] = input_shape_;

    auto bias_of = [&](const onnx::Node& node) {
        std::vector<float> b;
        if (node.inputs.size() > 2) {
            auto it = init_map.find(resolve(node.inputs[2]));
            if (it != init_map.end()) b = it->second->floats();
        }
        return b;
    };

    for (const auto& node : graph.nodes) {
        const std::string& op = node.op_type;
        if (node.outputs.empty()) throw std::runtime_error("ONNX node without output: " + op);
        const std::string& out = node.outputs[0];

        if (op == "MatMul" || op == "Gemm") {
            if (node.inputs.size() < 2) throw std::runtime_error(op + " needs two inputs");
            const std::string wname = resolve(node.inputs[1]);
            auto itW = init_map.find(wname);
            if (itW == init_map.end()) throw std::runtime_error("Weight '" + wname + "' not found");
            const onnx::Tensor& W = *itW->second;
            if (W.dims.size() != 2) throw std::runtime_error("FC weight must be 2D");
            std::vector<float> raw = W.floats();
            const uint32_t d0 = uint32_t(W.dims[0]), d1 = uint32_t(W.dims[1]);
            uint32_t M, N;
            std::vector<float> W_MxN;
            if (op == "MatMul") {                 // (B x N) * (N x M): transpose to M x N (:198-201)
                N = d0; M = d1;
                transpose_rc(raw, N, M, W_MxN);
            } else {                              // Gemm: a missing transB means 1, alpha/beta ignored (:204-217)
                int64_t transB = 1;
                if (const auto* a = node.find("transB")) transB = a->i;
                if (transB == 1) { M = d0; N = d1; W_MxN = std::move(raw); }
                else { N = d0; M = d1; transpose_rc(raw, N, M, W_MxN); }
            }
            Layer L;
            L.op = LayerOp::MatMul;
            L.E = std::make_unique<Ellpack>(encode_host(W_MxN.data(), M, N));
            if (op == "Gemm") L.bias = bias_of(node);     // bias only from Gemm's third input (:240-245)
            if (!L.bias.empty() && L.bias.size() != M) throw std::runtime_error("Gemm bias length must equal the output features");
            L.inputs = { resolve(node.inputs[0]) };
            L.outputs = { out };
            L.out_features = M;
            layers_.push_back(std::move(L));
            shape_map_[out] = { int(batch_dim_), int(M) };
            continue;
        }

        if (op == "Add") {
            if (node.inputs.size() != 2) throw std::runtime_error("Add needs two inputs");
            Layer L;
            L.op = LayerOp::Add;
            L.inputs = { resolve(node.inputs[0]), resolve(node.inputs[1]) };
            L.outputs = { out };
            shape_map_[out] = shape_map_.at(L.inputs[0]);
            layers_.push_back(std::move(L));
            continue;
        }

        if (op == "Relu" || op == "Sigmoid" || op == "Tanh") {
            Layer L;
            L.op = op == "Relu" ? LayerOp::Relu : op == "Sigmoid" ? LayerOp::Sigmoid : LayerOp::Tanh;
            L.inputs = { resolve(node.inputs.at(0)) };
            L.outputs = { out };
            shape_map_[out] = shape_map_.at(L.inputs[0]);
            layers_.push_back(std::move(L));
            continue;
        }

        if (op == "Conv") {
            if (node.inputs.size() < 2) throw std::runtime_error("Conv needs two inputs");
            auto itW = init_map.find(resolve(node.inputs[1]));
            if (itW == init_map.end()) throw std::runtime_error("Conv weight initializer not found");
            const onnx::Tensor& W = *itW->second;
            if (W.dims.size() != 4) throw std::runtime_error("Conv weight must be 4D");
            const std::vector<float> kernel = W.floats();
            spx_conv_geom g{};
            g.Cout = uint32_t(W.dims[0]); g.Cin = uint32_t(W.dims[1]);
            g.kH = uint32_t(W.dims[2]);   g.kW = uint32_t(W.dims[3]);
            g.sH = g.sW = g.dH = g.dW = 1;
            uint32_t group = 1;
            // Attributes as the reference reads them (:408-416): begin pads only.
            for (const auto& a : node.attributes) {
                if (a.name == "pads" && a.ints.size() == 4) { g.pH = uint32_t(a.ints[0]); g.pW = uint32_t(a.ints[1]); }
                else if (a.name == "strides" && a.ints.size() == 2) { g.sH = uint32_t(a.ints[0]); g.sW = uint32_t(a.ints[1]); }
                else if (a.name == "dilations" && a.ints.size() == 2) { g.dH = uint32_t(a.ints[0]); g.dW = uint32_t(a.ints[1]); }
                else if (a.name == "group") group = uint32_t(a.i);
            }
            if (group != 1) throw std::runtime_error("Grouped conv not supported (yet)");
            const std::string x_name = resolve(node.inputs[0]);
            const auto in_shape = shape_map_.at(x_name);
            if (in_shape.size() != 4) throw std::runtime_error("Conv input must be 4D");
            if (uint32_t(in_shape[1]) != g.Cin) throw std::runtime_error("Conv Cin mismatch");
            g.H = uint32_t(in_shape[2]); g.W = uint32_t(in_shape[3]);
            g.Ho = (g.H + 2 * g.pH - (g.dH * (g.kH - 1) + 1)) / g.sH + 1;     // (:428-429)
            g.Wo = (g.W + 2 * g.pW - (g.dW * (g.kW - 1) + 1)) / g.sW + 1;
            Layer L;
            L.op = LayerOp::Conv;
            // [Cout][Cin][kH][kW] is already the row-major [Cout x K] matrix, k = (cin, kh, kw) (:394-405).
            L.E = std::make_unique<Ellpack>(encode_host(kernel.data(), g.Cout, g.Cin * g.kH * g.kW));
            L.bias = bias_of(node);
            if (!L.bias.empty() && L.bias.size() != g.Cout) throw std::runtime_error("Conv bias length must equal Cout");
            L.geom = g;
            L.inputs = { x_name };
            L.outputs = { out };
            L.out_features = uint64_t(g.Cout) * g.Ho * g.Wo;
            layers_.push_back(std::move(L));
            shape_map_[out] = { in_shape[0], int(g.Cout), int(g.Ho), int(g.Wo) };
            continue;
        }

        if (op == "MaxPool" || op == "GlobalAveragePool") {     // attributes as the reference reads them (:304-350)
            const std::string x_name = resolve(node.inputs.at(0));
            const auto in_shape = shape_map_.at(x_name);
            if (in_shape.size() != 4) throw std::runtime_error("Pool input must be 4D");
            Layer L;
            PoolGeom& g = L.pool;
            g.C = uint32_t(in_shape[1]); g.H = uint32_t(in_shape[2]); g.W = uint32_t(in_shape[3]);
            if (op == "GlobalAveragePool") {
                L.op = LayerOp::GlobalAveragePool;
                L.out_features = g.C;
                shape_map_[out] = { in_shape[0], int(g.C) };
            } else {
                L.op = LayerOp::MaxPool;
                for (const auto& a : node.attributes) {
                    if (a.name == "kernel_shape" && a.ints.size() == 2) { g.kH = uint32_t(a.ints[0]); g.kW = uint32_t(a.ints[1]); }
                    else if (a.name == "strides" && a.ints.size() == 2) { g.sH = uint32_t(a.ints[0]); g.sW = uint32_t(a.ints[1]); }
                    else if (a.name == "pads" && a.ints.size() == 4) {
                        g.pH0 = uint32_t(a.ints[0]); g.pW0 = uint32_t(a.ints[1]);
                        g.pH1 = uint32_t(a.ints[2]); g.pW1 = uint32_t(a.ints[3]);
                    }
                }
                if (g.kH == 0 || g.kW == 0 || g.sH == 0 || g.sW == 0 || g.H + g.pH0 + g.pH1 < g.kH || g.W + g.pW0 + g.pW1 < g.kW)
                    throw std::runtime_error("MaxPool: bad kernel / stride / padding");
                g.Ho = (g.H + g.pH0 + g.pH1 - g.kH) / g.sH + 1;
                g.Wo = (g.W + g.pW0 + g.pW1 - g.kW) / g.sW + 1;
                L.out_features = uint64_t(g.C) * g.Ho * g.Wo;
                shape_map_[out] = { in_shape[0], int(g.C), int(g.Ho), int(g.Wo) };
            }
            L.inputs = { x_name };
            L.outputs = { out };
            layers_.push_back(std::move(L));
            continue;
        }

        if (op == "Flatten") {                    // [C,H,W,B] is already [features x B]: alias (:353-378)
            int64_t axis = 1;
            if (const auto* a = node.find("axis")) axis = a->i;
            const std::string in = resolve(node.inputs.at(0));
            const auto in_shape = shape_map_.at(in);
            if (axis != 1) throw std::runtime_error("Flatten: only axis=1 is supported");
            int prod = 1;
            for (size_t d = 1; d < in_shape.size(); ++d) prod *= in_shape[d];
            name_alias_[out] = in;
            shape_map_[out] = { in_shape[0], prod };
            continue;
        }

        if (op == "Identity") {                   // alias, no layer (:522-534)
            const std::string in = resolve(node.inputs.at(0));
            name_alias_[out] = in;
            auto it = shape_map_.find(in);
            if (it != shape_map_.end()) shape_map_[out] = it->second;
            continue;
        }

        throw std::runtime_error("Unsupported ONNX op: " + op);
    }
    const std::string labelled_output = graph.outputs[0].name;
    output_name_ = resolve(output_name_);
    if (shape_map_.count(labelled_output)) output_label_shape_ = shape_map_.at(labelled_output);

    // Fuse an activation that directly follows a MatMul / Conv and is its only consumer
    // (reference: Relu only, src/sparse_onnx.cpp:573-620).
    std::unordered_map<std::string, int> use;
    for (const auto& L : layers_) for (const auto& in : L.inputs) use[in]++;
    for (size_t i = 0; i + 1 < layers_.size(); ++i) {
        Layer& A = layers_[i];
        Layer& Bn = layers_[i + 1];
        if (!(A.op == LayerOp::MatMul || A.op == LayerOp::Conv) || A.act != SPX_ACT_NONE) continue;
        if (!(Bn.op == LayerOp::Relu || Bn.op == LayerOp::Sigmoid || Bn.op == LayerOp::Tanh)) continue;
        if (Bn.inputs.size() != 1 || Bn.outputs.size() != 1 || Bn.inputs[0] != A.outputs[0]) continue;
        if (use[A.outputs[0]] != 1 || A.outputs[0] == output_name_) continue;
        A.act = Bn.op == LayerOp::Relu ? SPX_ACT_RELU : Bn.op == LayerOp::Sigmoid ? SPX_ACT_SIGMOID : SPX_ACT_TANH;
        shape_map_[Bn.outputs[0]] = shape_map_.at(A.outputs[0]);
        A.outputs[0] = Bn.outputs[0];
        layers_.erase(layers_.begin() + (i + 1));
    }

    if (!shape_map_.count(output_name_)) throw std::runtime_error("Graph output '" + output_name_ + "' is not produced by any node");
    const auto& os = shape_map_.at(output_name_);
    out_features_ = 1;
    for (size_t d = 1; d < os.size(); ++d) out_features_ *= uint64_t(os[d]);

    // Weights become device-resident now; activation buffers on the first run / resize_buffers.
    if (upload_weights)
        for (auto& L : layers_) if (L.E) L.E->upload();
}

std::vector<size_t> SparseOnnxModel::output_shape() const
{
    std::vector<size_t> dims;
    for (int d : output_label_shape_.empty() ? shape_map_.at(output_name_) : output_label_shape_) dims.push_back(size_t(d));
    return dims;
}

double SparseOnnxModel::flops_per_run(uint32_t B) const
{
    double f = 0.0;
    for (const auto& L : layers_) {
        if (L.op == LayerOp::MatMul) f += 2.0 * double(L.E->nnz_total()) * B;
        else if (L.op == LayerOp::Conv) f += 2.0 * double(L.E->nnz_total()) * double(L.geom.Ho) * L.geom.Wo * B;
    }
    return f;
}

void SparseOnnxModel::shard_rows(int rank, int world, const char* unique_id)
{
    if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("shard_rows: bad rank / world");
    exec_.reset();
    spx_comm_destroy(comm_);
    comm_ = nullptr;
    rank_ = rank;
    world_ = world;
    for (auto& L : layers_) {
        L.shard.reset();
        if (!L.E) continue;
        if (world > 1) L.shard = std::make_unique<Ellpack>(L.E->shard_rows(uint32_t(rank), uint32_t(world)));
    }
    if (world > 1) {
        if (!unique_id) throw std::runtime_error("shard_rows: unique_id is null");
        check(spx_comm_create(rank, world, unique_id, &comm_), "communicator");
    }
}

void SparseOnnxModel::resize_buffers(uint32_t B) { build_exec(B); }

// Every rank exports its full-size output buffers, the 64-byte handles travel through one
// all-gather, and each rank maps its peers' buffers.  Any failure leaves the NCCL route in place.
bool SparseOnnxModel::exchange_peer_buffers(Exec& ex, const std::vector<std::string>& names) const
{
    // Every rank runs the same two collectives whatever happens locally, so that a local failure
    // can never leave the ranks in different modes: the handles travel in the first all-gather, a
    // success flag per rank in the second; the fused route is taken only if every rank succeeded.
    const size_t L = names.size(), hfloats = SPX_IPC_HANDLE_BYTES / sizeof(float), per = L * hfloats + 1;
    std::vector<float> mine(per, 0.0f);
    bool ok = true;
    for (size_t i = 0; i < L && ok; ++i)
        ok = spx_ipc_export(ex.buf.at(names[i]), reinterpret_cast<char*>(mine.data() + i * hfloats)) == SPX_OK;
    float* d_all = nullptr;
    check(spx_malloc(reinterpret_cast<void**>(&d_all), size_t(world_) * per * sizeof(float)), "handle exchange buffer");
    std::vector<float> all(size_t(world_) * per, 0.0f);
    auto gather = [&]() {
        mine[per - 1] = ok ? 1.0f : 0.0f;
        check(spx_memcpy_h2d(d_all + size_t(rank_) * per, mine.data(), per * sizeof(float), ex.stream), "handle exchange");
        check(spx_allgather_rows(comm_, d_all, 1, per, ex.stream), "handle exchange");
        check(spx_memcpy_d2h(all.data(), d_all, all.size() * sizeof(float), ex.stream), "handle exchange");
        check(spx_stream_sync(ex.stream), "handle exchange");
        for (int g = 0; g < world_; ++g) ok = ok && all[size_t(g) * per + per - 1] == 1.0f;
    };
    gather();                                       // handles + "export worked" flags
    if (ok) {
        for (size_t i = 0; i < L && ok; ++i) {
            std::vector<float*> ptrs(world_, nullptr);
            for (int g = 0; g < world_ && ok; ++g) {
                if (g == rank_) { ptrs[g] = ex.buf.at(names[i]); continue; }
                void* p = nullptr;
                ok = spx_ipc_open(reinterpret_cast<const char*>(all.data() + size_t(g) * per + i * hfloats), &p) == SPX_OK;
                if (ok) { ex.opened.push_back(p); ptrs[g] = static_cast<float*>(p); }
            }
            if (ok) ex.peers[names[i]] = std::move(ptrs);
        }
    }
    gather();                                       // "mapping worked" flags
    spx_free(d_all);
    if (!ok) {
        for (void* p : ex.opened) spx_ipc_close(p);
        ex.opened.clear();
        ex.peers.clear();
    }
    return ok;
}

void SparseOnnxModel::build_exec(uint32_t B) const
{
    exec_.reset();
    auto ex = std::make_unique<Exec>();
    ex->B = B;
    check(spx_stream_create(&ex->stream), "stream");

    // All biases packed into one device array (reference: one host array, src/sparse_onnx.cpp:541-571).
    size_t total_bias = 0;
    for (const auto& L : layers_) total_bias += L.bias.size();
    if (total_bias) {
        std::vector<float> packed;
        packed.reserve(total_bias);
        for (auto& L : const_cast<std::vector<Layer>&>(layers_)) {
            L.bias_offset = packed.size();
            packed.insert(packed.end(), L.bias.begin(), L.bias.end());
        }
        check(spx_malloc(reinterpret_cast<void**>(&ex->d_bias), total_bias * sizeof(float)), "bias buffer");
        check(spx_memcpy_h2d(ex->d_bias, packed.data(), total_bias * sizeof(float), nullptr), "bias upload");
        check(spx_stream_sync(nullptr), "bias upload");
    }

    // Activation buffers are planned by liveness, as the reference frees an intermediate once its
    // last reader has run (src/model_run.cpp:14-19, :116-127): a tensor's buffer returns to a free
    // list after the last layer that reads it and is handed to a later output that fits, so a deep
    // graph holds a few activations at a time, not one per layer.  The graph's input and output
    // keep buffers of their own (callers address them), and a layer's output never shares a buffer
    // with that layer's inputs (the inputs are released after the output is placed).  Row-sharded
    // models keep one buffer per tensor: peers store into them between barriers.
    std::unordered_map<std::string, size_t> last_use;
    for (size_t i = 0; i < layers_.size(); ++i)
        for (const auto& in : layers_[i].inputs) last_use[in] = i;
    const bool reuse = world_ == 1 && !std::getenv("SPX_NO_BUFFER_REUSE");
    std::multimap<size_t, void*> free_list;                 // capacity in bytes -> buffer
    std::unordered_map<std::string, size_t> capacity;
    auto alloc = [&](const std::string& name, uint64_t rows, uint64_t padded_rows) {
        const size_t bytes = size_t(padded_rows) * B * sizeof(float);
        void* p = nullptr;
        size_t cap = bytes;
        auto it = (reuse && name != output_name_) ? free_list.lower_bound(bytes) : free_list.end();
        if (it != free_list.end()) {
            cap = it->first;
            p = it->second;
            free_list.erase(it);
        } else {
            check(spx_malloc(&p, bytes), "activation buffer");
            ex->owned.push_back(p);
        }
        ex->buf[name] = static_cast<float*>(p);
        ex->rows[name] = rows;
        capacity[name] = cap;
    };
    alloc(input_name_, in_features_, in_features_);
    for (size_t li = 0; li < layers_.size(); ++li) {
        const auto& L = layers_[li];
        uint64_t rows, padded;
        if (L.op == LayerOp::MatMul || L.op == LayerOp::Conv) {
            rows = L.out_features;
            // row-sharded: room for world slabs of ceil(m/world) rows each
            const uint64_t per_row = L.op == LayerOp::Conv ? uint64_t(L.geom.Ho) * L.geom.Wo : 1;
            const uint64_t m = L.E->m;
            padded = world_ > 1 ? ((m + world_ - 1) / world_) * world_ * per_row : rows;
        } else if (L.op == LayerOp::MaxPool || L.op == LayerOp::GlobalAveragePool) {
            rows = padded = L.out_features;
        } else {
            rows = padded = ex->rows.at(L.inputs[0]);
        }
        alloc(L.outputs[0], rows, padded);
        if (reuse)
            for (const auto& in : L.inputs) {
                auto lu = last_use.find(in);
                if (in == input_name_ || in == output_name_ || lu == last_use.end() || lu->second != li) continue;
                auto c = capacity.find(in);
                if (c == capacity.end()) continue;          // already returned (a layer may name an input twice)
                free_list.emplace(c->second, ex->buf.at(in));
                capacity.erase(c);
            }
    }
    ex->distinct_buffers = ex->owned.size();
    const size_t out_bytes = size_t(out_features_) * B * sizeof(float);
    if (out_bytes && out_bytes <= (size_t(8) << 20) &&
        spx_host_alloc(reinterpret_cast<void**>(&ex->h_out), out_bytes) == SPX_OK)
        ex->h_out_bytes = out_bytes;        // without it run() copies straight into the caller's array
    if (world_ > 1 && comm_) {
        ex->comm = comm_;
        const char* off = std::getenv("SPX_TP_FUSED");
        if (!(off && off[0] == '0')) {
            std::vector<std::string> names;
            for (const auto& L : layers_)
                if (L.op == LayerOp::MatMul && L.shard) names.push_back(L.outputs[0]);
            if (!names.empty()) ex->fused = exchange_peer_buffers(*ex, names);
        }
    }
    exec_ = std::move(ex);

    // One eager pass (lets kernels make their lazy, per-handle allocations outside a capture),
    // then capture the same launches as a graph for the host-buffer run().
    float* d_in = exec_->buf.at(input_name_);
    float* d_out = exec_->buf.at(output_name_);
    check(spx_memset(d_in, 0, size_t(in_features_) * B * sizeof(float), exec_->stream), "memset");
    launch_layers(d_in, d_out, B, exec_->stream);
    check(spx_stream_sync(exec_->stream), "warm-up pass");
    const char* no_graph = std::getenv("SPX_NO_GRAPH");
    if (!(no_graph && no_graph[0] == '1')) {
        if (spx_graph_capture_begin(exec_->stream) == SPX_OK) {
            bool ok = true;
            try { launch_layers(d_in, d_out, B, exec_->stream); } catch (...) { ok = false; }
            void* g = nullptr;
            if (spx_graph_capture_end(exec_->stream, &g) == SPX_OK && ok) exec_->graph = g;
            else if (g) spx_graph_destroy(g);
        }
    }
}

// The layer loop (reference: src/model_run.cpp:28-127).  Buffers were planned in build_exec;
// d_in / d_out replace the planned input / output buffers so callers can run in place on their
// own device memory.
void SparseOnnxModel::launch_layers(const float* d_in, float* d_out, uint32_t B, void* stream) const
{
    const Exec& ex = *exec_;
    auto src_of = [&](const std::string& name) -> const float* {
        return name == input_name_ ? d_in : ex.buf.at(name);
    };
    // Fused exchange: a rank may store into a peer's buffer only after that peer has finished
    // reading it in the previous pass, hence one barrier up front (all later layers are ordered by
    // the barriers that follow each exchange).
    if (ex.fused) check(spx_comm_barrier(comm_, stream), "barrier");
    for (const auto& L : layers_) {
        float* dst = L.outputs[0] == output_name_ ? d_out : ex.buf.at(L.outputs[0]);
        const float* src = src_of(L.inputs[0]);
        switch (L.op) {
        case LayerOp::MatMul: {
            const Ellpack& E = L.shard ? *L.shard : *L.E;
            const uint64_t per = L.shard ? (L.E->m + world_ - 1) / world_ : 0;
            const uint64_t row0 = per * uint64_t(rank_);
            const float* bias = L.bias.empty() ? nullptr : ex.d_bias + L.bias_offset + (L.shard ? row0 : 0);
            auto pit = ex.fused && L.shard ? ex.peers.find(L.outputs[0]) : ex.peers.end();
            if (pit != ex.peers.end() && dst == ex.buf.at(L.outputs[0])) {
                // epilogue stores this rank's rows into every rank's full buffer over NVLink
                check(spx_spmm_bcast(E.dev, src, B, B, bias, L.act, pit->second.data(), uint32_t(world_), row0, B, stream),
                      "MatMul layer (fused exchange)");
                check(spx_comm_barrier(comm_, stream), "barrier");
                break;
            }
            check(spx_spmm(E.dev, src, B, B, bias, L.act, dst + row0 * B, B, stream), "MatMul layer");
            if (L.shard) check(spx_allgather_rows(comm_, dst, per, B, stream), "all-gather");
            break;
        }
        case LayerOp::Conv: {
            const Ellpack& E = L.shard ? *L.shard : *L.E;
            const uint64_t per = L.shard ? (L.E->m + world_ - 1) / world_ : 0;
            const uint64_t row0 = per * uint64_t(rank_);
            const uint64_t row_elems = uint64_t(L.geom.Ho) * L.geom.Wo * B;
            spx_conv_geom g = L.geom;
            g.Cout = E.m;
            const float* bias = L.bias.empty() ? nullptr : ex.d_bias + L.bias_offset + (L.shard ? row0 : 0);
            check(spx_conv2d(E.dev, &g, SPX_LAYOUT_PF, src, B, bias, L.act, dst + row0 * row_elems, stream), "Conv layer");
            if (L.shard) check(spx_allgather_rows(comm_, dst, per, row_elems, stream), "all-gather");
            break;
        }
        case LayerOp::Relu:
        case LayerOp::Sigmoid:
        case LayerOp::Tanh: {
            const int op = L.op == LayerOp::Relu ? SPX_OP_RELU : L.op == LayerOp::Sigmoid ? SPX_OP_SIGMOID : SPX_OP_TANH;
            check(spx_eltwise(op, src, nullptr, dst, ex.rows.at(L.inputs[0]) * B, stream), "activation layer");
            break;
        }
        case LayerOp::MaxPool: {
            const PoolGeom& g = L.pool;
            check(spx_maxpool2d(src, g.C, g.H, g.W, B, g.kH, g.kW, g.sH, g.sW, g.pH0, g.pW0, g.pH1, g.pW1, dst, stream),
                  "MaxPool layer");
            break;
        }
        case LayerOp::GlobalAveragePool: {
            const PoolGeom& g = L.pool;
            check(spx_global_avgpool(src, g.C, g.H, g.W, B, dst, stream), "GlobalAveragePool layer");
            break;
        }
        case LayerOp::Add: {
            const uint64_t ra = ex.rows.at(L.inputs[0]), rb = ex.rows.at(L.inputs[1]);
            if (ra != rb) throw std::runtime_error("Add: operand shapes differ");
            check(spx_eltwise(SPX_OP_ADD, src, src_of(L.inputs[1]), dst, ra * B, stream), "Add layer");
            break;
        }
        }
    }
    if (layers_.empty() || output_name_ == input_name_) {
        // degenerate graph (only Identity nodes): output = input
        check(spx_memcpy_d2d(d_out, d_in, size_t(in_features_) * B * sizeof(float), stream), "copy");
    }
}

void SparseOnnxModel::run(const float* input, uint32_t B, float* output) const
{
    if (!exec_ || exec_->B != B) build_exec(B);
    Exec& ex = *exec_;
    float* d_in = ex.buf.at(input_name_);
    float* d_out = ex.buf.at(output_name_);
    check(spx_memcpy_h2d(d_in, input, size_t(in_features_) * B * sizeof(float), ex.stream), "input copy");
    if (ex.graph) check(spx_graph_launch(ex.graph, ex.stream), "graph launch");
    else launch_layers(d_in, d_out, B, ex.stream);
    const size_t out_bytes = size_t(out_features_) * B * sizeof(float);
    if (ex.h_out && ex.h_out_bytes == out_bytes) {
        check(spx_memcpy_d2h(ex.h_out, d_out, out_bytes, ex.stream), "output copy");
        check(spx_stream_sync(ex.stream), "run");
        std::memcpy(output, ex.h_out, out_bytes);
        return;
    }
    check(spx_memcpy_d2h(output, d_out, out_bytes, ex.stream), "output copy");
    check(spx_stream_sync(ex.stream), "run");
}

size_t SparseOnnxModel::activation_buffers() const
{
    if (!exec_) throw std::runtime_error("activation_buffers: call resize_buffers(B) first");
    return exec_->distinct_buffers;
}

float* SparseOnnxModel::device_input() const
{
    if (!exec_) throw std::runtime_error("device_input: call resize_buffers(B) first");
    return exec_->buf.at(input_name_);
}

float* SparseOnnxModel::device_output() const
{
    if (!exec_) throw std::runtime_error("device_output: call resize_buffers(B) first");
    return exec_->buf.at(output_name_);
}

void SparseOnnxModel::run_resident(void* stream) const
{
    if (!exec_) throw std::runtime_error("run_resident: call resize_buffers(B) first");
    if (exec_->graph) check(spx_graph_launch(exec_->graph, stream), "graph launch");
    else launch_layers(device_input(), device_output(), exec_->B, stream);
}

void SparseOnnxModel::run_device(const float* d_input, uint32_t B, float* d_output, void* stream) const
{
    if (!exec_ || exec_->B != B) build_exec(B);
    launch_layers(d_input, d_output, B, stream);
}

}  // namespace spx
