// probe.cu -- a measured denominator for the SpMM operand path.
//
// The SpMM kernels are bound by gathering rows of X from L2 into the SMs (one 4-byte operand
// per FMA), not by HBM.  spx_probe_l2_gather issues the same kind of traffic with no arithmetic
// to speak of: every warp reads 512-byte segments (32 lanes x float4, like one NV slice of an X
// row) at pseudo-random segment positions of a buffer that fits L2, bypassing L1, eight loads in
// flight per lane.  bytes / time of this kernel is the L2 -> SM gather bandwidth the SpMM's
// operand traffic can be compared with.
#include "common.cuh"

namespace {

__device__ __forceinline__ float4 ld_l2(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

constexpr int kProbeInFlight = 8;

__global__ void __launch_bounds__(256)
l2_gather_probe_kernel(const float4* __restrict__ buf, uint32_t seg_mask, uint32_t rounds, float* __restrict__ sink)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    uint32_t state = warp * 2654435761u + 12345u;
    float acc = 0.0f;
    for (uint32_t r = 0; r < rounds; ++r) {
        float4 v[kProbeInFlight];
#pragma unroll
        for (int u = 0; u < kProbeInFlight; ++u) {
            state = state * 1664525u + 1013904223u;              // same value in every lane of the warp
            const uint32_t seg = (state >> 8) & seg_mask;
            v[u] = ld_l2(buf + (size_t)seg * 32 + lane);
        }
#pragma unroll
        for (int u = 0; u < kProbeInFlight; ++u) acc += v[u].x + v[u].y + v[u].z + v[u].w;
    }
    if (acc == 123.456f) sink[0] = acc;                          // keeps the loads alive; practically never true
}

}  // namespace

extern "C" int spx_probe_l2_gather(const void* buf, size_t bytes, uint32_t rounds, float* sink, void* stream,
                                   uint64_t* bytes_read)
{
    using spx::fail;
    if (!buf || !sink || !bytes_read) return fail(SPX_ERR_ARG, "probe: null argument");
    if ((reinterpret_cast<uintptr_t>(buf) & 15) != 0) return fail(SPX_ERR_ARG, "probe: buffer must be 16-byte aligned");
    uint64_t segs = bytes / 512;
    if (segs < 2 || rounds == 0) return fail(SPX_ERR_ARG, "probe: need at least 1 KiB and one round");
    uint32_t pow2 = 1;
    while ((uint64_t)pow2 * 2 <= segs && pow2 < (1u << 30)) pow2 <<= 1;      // largest power of two that fits
    int dev = 0;
    SPX_CUDA(cudaGetDevice(&dev));
    const uint32_t blocks = (uint32_t)spx::sm_count(dev) * 8;               // 2048 threads per SM
    l2_gather_probe_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const float4*>(buf), pow2 - 1, rounds, sink);
    SPX_LAUNCH_CHECK("l2_gather_probe_kernel");
    *bytes_read = (uint64_t)blocks * 8 /* warps */ * rounds * kProbeInFlight * 512ull;
    return SPX_OK;
}
