// l2_gather_probe.cu -- a measured denominator for the SpMM operand path.  Bench equipment: built
// into its own small library (libspx_bench_probe.so) that only the benchmark loads; it is not part
// of the product library or of its C ABI.
//
// The SpMM kernels are bound by gathering rows of X from L2 into the SMs (one 4-byte operand
// per FMA), not by HBM.  bench_l2_gather_probe issues the same kind of traffic with no arithmetic
// to speak of: every warp reads 512-byte segments (32 lanes x float4, like one NV slice of an X
// row) at pseudo-random segment positions of a buffer that fits L2, bypassing L1, eight loads in
// flight per lane.  bytes / time of this kernel is the L2 -> SM gather bandwidth the SpMM's
// operand traffic can be compared with.
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

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

// Gathers 512-byte segments at pseudo-random positions of buf (the largest power-of-two number of
// segments within `bytes`; choose a size that fits L2), `rounds` x 8 loads per lane on a grid of 8
// CTAs per SM, and reports how many bytes the launch reads.  sink: one writable float on the device.
// Returns 0, -1 for a bad argument, or the cudaError_t of a failed call.
extern "C" int bench_l2_gather_probe(const void* buf, size_t bytes, uint32_t rounds, float* sink, void* stream,
                                     uint64_t* bytes_read)
{
    if (!buf || !sink || !bytes_read) return -1;
    if ((reinterpret_cast<uintptr_t>(buf) & 15) != 0) return -1;
    uint64_t segs = bytes / 512;
    if (segs < 2 || rounds == 0) return -1;
    uint32_t pow2 = 1;
    while ((uint64_t)pow2 * 2 <= segs && pow2 < (1u << 30)) pow2 <<= 1;      // largest power of two that fits
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return (int)err;
    const uint32_t blocks = (uint32_t)sms * 8;                              // 2048 threads per SM
    l2_gather_probe_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const float4*>(buf), pow2 - 1, rounds, sink);
    err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
    *bytes_read = (uint64_t)blocks * 8 /* warps */ * rounds * kProbeInFlight * 512ull;
    return 0;
}
