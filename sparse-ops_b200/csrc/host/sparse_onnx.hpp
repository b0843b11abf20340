// sparse_onnx.hpp -- SparseOnnxModel: ONNX-driven sparse inference whose layer loop runs on the
// GPU.  Interface of the reference class (include/sparse_onnx.hpp:139-163): construct from a
// path, run(input, B, output), output_shape(); plus resize_buffers(B), which the reference's
// README documents (README.md:144-148).
//
// Load time (constructor) follows the reference planner (src/sparse_onnx.cpp:82-636): Gemm /
// MatMul / Conv weights are ELLPACK-encoded once and kept device-resident, biases are packed
// into one device array, MatMul/Conv + Relu pairs are fused (:573-620; Sigmoid and Tanh are
// fused into the producing kernel's epilogue as well -- same values, one pass less).
//
// Beyond the reference: MaxPool, GlobalAveragePool and Flatten also work on [C,H,W,B] tensors
// (the reference indexes those three in an older layout that its own convolution no longer
// produces, so conv -> pool / flatten graphs are wrong there).  In [C,H,W,B] a Flatten is a pure
// alias whose feature order (c, h, w) equals the flatten order of an NCHW tensor, so fully
// connected weights need no column permutation.
//
// Memory contract of run(), identical to the reference (src/model_run.cpp, src/layers/matmul.cpp:
// activations are feature-major): the input bytes are read as [in_features x B] for dense
// models or [Cin, H, W, B] for convolutional ones, B fastest; the output bytes are [M x B] /
// [Cout, Ho, Wo, B], regardless of the labelled ONNX shape.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "ellpack.hpp"

namespace spx {

enum class LayerOp { MatMul, Relu, Sigmoid, Tanh, Add, Conv, MaxPool, GlobalAveragePool };

/// MaxPool / GlobalAveragePool geometry (reference: PoolAttr, include/sparse_onnx.hpp:95-105).
struct PoolGeom {
    uint32_t C = 0, H = 0, W = 0;
    uint32_t kH = 1, kW = 1, sH = 1, sW = 1;
    uint32_t pH0 = 0, pW0 = 0, pH1 = 0, pW1 = 0;
    uint32_t Ho = 1, Wo = 1;
};

struct Layer {
    LayerOp op;
    std::unique_ptr<Ellpack> E;        ///< full matrix, host arrays (+ device copy when unsharded)
    std::unique_ptr<Ellpack> shard;    ///< this rank's rows when row-sharded
    std::vector<float> bias;           ///< empty = no bias
    size_t bias_offset = 0;            ///< into the packed device bias array
    int act = SPX_ACT_NONE;            ///< activation fused into the epilogue
    spx_conv_geom geom{};              ///< Conv only
    PoolGeom pool{};                   ///< MaxPool / GlobalAveragePool only
    std::vector<std::string> inputs, outputs;
    uint64_t out_features = 0;         ///< output elements per batch column
};

class SparseOnnxModel {
public:
    /// upload_weights = false only parses and plans (no CUDA call is made): for inspecting the
    /// plan on a machine without a GPU; such a model cannot run.
    explicit SparseOnnxModel(const std::string& onnx_path, bool upload_weights = true);
    ~SparseOnnxModel();
    SparseOnnxModel(const SparseOnnxModel&) = delete;
    SparseOnnxModel& operator=(const SparseOnnxModel&) = delete;

    /// Host buffers in, host buffers out (see the memory contract above).  Re-plans the device
    /// buffers when B differs from the current batch.
    void run(const float* input, uint32_t B, float* output) const;
    /// Device buffers in and out; launches the layer loop on `stream` without synchronising.
    void run_device(const float* d_input, uint32_t B, float* d_output, void* stream) const;
    /// The model's own device buffers for the current batch (valid after resize_buffers / run):
    /// fill device_input(), call run_resident(), read device_output().  run_resident replays the
    /// captured CUDA graph on `stream` (or launches the layers when no graph was captured) and does
    /// not synchronise.
    float* device_input() const;
    float* device_output() const;
    void run_resident(void* stream) const;
    /// Number of distinct activation buffers the current plan holds; buffers are reused by
    /// liveness, so this stays small for deep graphs (reference: src/model_run.cpp:116-127).
    size_t activation_buffers() const;
    /// Output dims as labelled in the ONNX graph (static shape recorded at load).
    std::vector<size_t> output_shape() const;
    /// (Re)allocate the activation buffers for batch B and capture the layer loop as a CUDA graph.
    void resize_buffers(uint32_t B);
    /// Tensor-parallel mode: every MatMul / Conv keeps only rows [rank*ceil(m/world), ...) on this
    /// process's GPU.  MatMul layers store their rows straight into every rank's full output buffer
    /// (peers' buffers mapped over IPC, plain stores over NVLink, then a barrier); Conv layers, and
    /// MatMul layers when the buffers cannot be shared (or SPX_TP_FUSED=0), end with an in-place NCCL
    /// all-gather of the row slabs.
    /// unique_id: SPX_UNIQUE_ID_BYTES bytes from spx_comm_unique_id, identical on all ranks.
    void shard_rows(int rank, int world, const char* unique_id);

    uint32_t batch() const { return batch_dim_; }
    uint32_t in_features() const { return in_features_; }
    uint64_t out_features() const { return out_features_; }
    size_t num_layers() const { return layers_.size(); }
    const Layer& layer(size_t i) const { return layers_[i]; }
    /// Algorithmic work of one forward pass at batch B: 2 * nnz * columns summed over layers.
    double flops_per_run(uint32_t B) const;

private:
    struct Exec;                                   // device buffers, stream, graph (mutable state)
    void build_exec(uint32_t B) const;
    bool exchange_peer_buffers(Exec& ex, const std::vector<std::string>& names) const;
    void launch_layers(const float* d_in, float* d_out, uint32_t B, void* stream) const;

    std::vector<Layer> layers_;
    uint32_t batch_dim_ = 1;
    uint32_t in_features_ = 0;
    uint64_t out_features_ = 0;
    std::vector<int> input_shape_;
    std::unordered_map<std::string, std::vector<int>> shape_map_;
    std::unordered_map<std::string, std::string> name_alias_;
    std::vector<int> output_label_shape_;
    std::string input_name_, output_name_;
    int rank_ = 0, world_ = 1;
    spx_comm* comm_ = nullptr;
    mutable std::unique_ptr<Exec> exec_;
};

}  // namespace spx

#ifndef SPX_NO_GLOBAL_NAMES
using spx::SparseOnnxModel;
#endif
