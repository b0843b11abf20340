// pool.cu -- MaxPool and GlobalAveragePool on [C,H,W,B] activations (batch fastest).
//
// Replaces applyMaxPool / applyGlobalAveragePool of the reference (src/layers/pool.cpp:28-154)
// with the same arithmetic: max over the in-image taps of the window starting from -inf
// (:44,60-70); mean = (sequential sum over h then w, starting from 0) * (1.0f / (H*W)) (:121-137).
// The reference indexes these two layers as b + B*(c + C*(h + H*w)), which does not match the
// [C,H,W,B] tensors its own convolution produces; here every layer of the model uses [C,H,W,B],
// so conv -> pool -> flatten -> fc graphs are consistent.  Both kernels are pure streaming.
#include "common.cuh"

namespace {

struct PoolParams {
    uint32_t C, H, W, B, Ho, Wo, kH, kW, sH, sW, pH, pW;
};

__global__ void __launch_bounds__(256)
maxpool_pf_kernel(const float* __restrict__ in, float* __restrict__ out, PoolParams p)
{
    const uint64_t total = (uint64_t)p.C * p.Ho * p.Wo * p.B;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += stride) {
        const uint32_t b = (uint32_t)(o % p.B);
        uint64_t t = o / p.B;
        const uint32_t ow = (uint32_t)(t % p.Wo); t /= p.Wo;
        const uint32_t oh = (uint32_t)(t % p.Ho);
        const uint32_t c = (uint32_t)(t / p.Ho);
        const int h0 = (int)(oh * p.sH) - (int)p.pH, w0 = (int)(ow * p.sW) - (int)p.pW;
        float v = -INFINITY;
        for (uint32_t kh = 0; kh < p.kH; ++kh) {
            const int ih = h0 + (int)kh;
            if ((unsigned)ih >= p.H) continue;
            for (uint32_t kw = 0; kw < p.kW; ++kw) {
                const int iw = w0 + (int)kw;
                if ((unsigned)iw >= p.W) continue;
                v = fmaxf(v, __ldg(in + (((size_t)c * p.H + ih) * p.W + iw) * p.B + b));
            }
        }
        out[o] = v;
    }
}

__global__ void __launch_bounds__(256)
gap_pf_kernel(const float* __restrict__ in, float* __restrict__ out, uint32_t C, uint32_t HW, uint32_t B, float scale)
{
    const uint64_t total = (uint64_t)C * B;
    const uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= total) return;
    const uint32_t b = (uint32_t)(o % B), c = (uint32_t)(o / B);
    const float* src = in + (size_t)c * HW * B + b;
    float s = 0.0f;
    for (uint32_t i = 0; i < HW; ++i) s += __ldg(src + (size_t)i * B);   // h outer, w inner: storage order
    out[o] = s * scale;
}

}  // namespace

extern "C" {

int spx_maxpool2d(const float* in, uint32_t C, uint32_t H, uint32_t W, uint32_t B, uint32_t kH, uint32_t kW,
                  uint32_t sH, uint32_t sW, uint32_t pH0, uint32_t pW0, uint32_t pH1, uint32_t pW1, float* out,
                  void* stream)
{
    if (kH == 0 || kW == 0 || sH == 0 || sW == 0) return spx::fail(SPX_ERR_ARG, "maxpool: kernel and stride must be positive");
    if (H + pH0 + pH1 < kH || W + pW0 + pW1 < kW) return spx::fail(SPX_ERR_ARG, "maxpool: window larger than padded input");
    PoolParams p{C, H, W, B, (H + pH0 + pH1 - kH) / sH + 1, (W + pW0 + pW1 - kW) / sW + 1, kH, kW, sH, sW, pH0, pW0};
    const uint64_t total = (uint64_t)C * p.Ho * p.Wo * B;
    if (total == 0) return SPX_OK;
    if (!in || !out) return spx::fail(SPX_ERR_ARG, "maxpool: null operand");
    int dev = 0;
    SPX_CUDA(cudaGetDevice(&dev));
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = (uint64_t)spx::sm_count(dev) * 16;
    if (blocks > cap) blocks = cap;
    maxpool_pf_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(in, out, p);
    SPX_LAUNCH_CHECK("maxpool_pf_kernel");
    return SPX_OK;
}

int spx_global_avgpool(const float* in, uint32_t C, uint32_t H, uint32_t W, uint32_t B, float* out, void* stream)
{
    const uint64_t total = (uint64_t)C * B;
    if (total == 0) return SPX_OK;
    if (H == 0 || W == 0) return spx::fail(SPX_ERR_ARG, "global average pool: empty image");
    if (!in || !out) return spx::fail(SPX_ERR_ARG, "global average pool: null operand");
    const uint64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffull) return spx::fail(SPX_ERR_LIMIT, "global average pool: too many outputs");
    gap_pf_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(in, out, C, H * W, B, 1.0f / (float)(H * W));
    SPX_LAUNCH_CHECK("gap_pf_kernel");
    return SPX_OK;
}

}  // extern "C"
