// eltwise.cu -- standalone activations and same-shape add for graphs whose activation cannot be
// fused into the producing kernel's epilogue.  Replaces applyRelu / applySigmoid / applyTanh
// (src/layers/activation.cpp:3-62), relu/sigmoid/tanh_inplace (src/activations.cpp:20-68) and
// applyAdd (src/layers/add.cpp:9-76) of the reference.  Pure streaming: 8 (12 for add) bytes
// per element, grid-stride, 16-byte vectors when the pointers allow.
#include "common.cuh"

namespace {

__device__ __forceinline__ float op1(float a, float b, int op) {
    switch (op) {
    case SPX_OP_RELU:    return a > 0.0f ? a : 0.0f;
    case SPX_OP_SIGMOID: return 1.0f / (1.0f + expf(-a));
    case SPX_OP_TANH:    return tanhf(a);
    default:             return a + b;   // SPX_OP_ADD
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
eltwise_kernel(int op, const float* a, const float* b, float* out, uint64_t count)   // out may alias a
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const uint64_t n4 = count >> 2;
        for (uint64_t q = i; q < n4; q += stride) {
            const float4 va = reinterpret_cast<const float4*>(a)[q];
            float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
            if (op == SPX_OP_ADD) vb = reinterpret_cast<const float4*>(b)[q];
            float4 o;
            o.x = op1(va.x, vb.x, op); o.y = op1(va.y, vb.y, op);
            o.z = op1(va.z, vb.z, op); o.w = op1(va.w, vb.w, op);
            reinterpret_cast<float4*>(out)[q] = o;
        }
        for (uint64_t q = (n4 << 2) + i; q < count; q += stride)
            out[q] = op1(a[q], op == SPX_OP_ADD ? b[q] : 0.0f, op);
    } else {
        for (; i < count; i += stride) out[i] = op1(a[i], op == SPX_OP_ADD ? b[i] : 0.0f, op);
    }
}

}  // namespace

namespace spx {

int launch_eltwise(int op, const float* a, const float* b, float* out, uint64_t count, cudaStream_t s)
{
    if (count == 0) return SPX_OK;
    int dev = 0;
    SPX_CUDA(cudaGetDevice(&dev));
    const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out) |
                       (b ? reinterpret_cast<uintptr_t>(b) : 0)) & 15) == 0;
    uint64_t want = (count / (vec ? 4 : 1) + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count(dev) * 8;
    if (want > cap) want = cap;
    if (want == 0) want = 1;
    if (vec) eltwise_kernel<true><<<(unsigned)want, 256, 0, s>>>(op, a, b, out, count);
    else     eltwise_kernel<false><<<(unsigned)want, 256, 0, s>>>(op, a, b, out, count);
    SPX_LAUNCH_CHECK("eltwise_kernel");
    return SPX_OK;
}

}  // namespace spx
