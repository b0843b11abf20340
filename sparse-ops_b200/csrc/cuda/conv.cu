// conv.cu -- sparse 2-D convolution by implicit im2col for sm_100a.
//
// Replaces the reference's conv2d_* family (src/layers/conv_kernels.cpp:66-470), all of which
// compute  out[m, p] = act(bias[m] + sum_j Wd[m,j] * patch[idx[m,j], p])  where the weight
// [Cout][Cin][kH][kW] is flattened to an ELLPACK of Cout rows over K = Cin*kH*kW columns with
// k = (cin*kH + kh)*kW + kw (src/sparse_onnx.cpp:394-405) and patch[k, p] is the input value
// under tap k of output position p, zero outside the image.  The reference materialises patch
// tiles (explicit im2col) and calls its SpMM; here the patch value is gathered on the fly.
//
// Arithmetic contract (same as the SpMM): per output element, start from bias, one FMA per
// stored nonzero of row m in storage order; a tap outside the image contributes the operand
// 0.0f exactly as the reference's zero-filled tile does.  Results are bit-identical to the
// reference for stride 1 (the reference mis-indexes stride_w > 1, :305-306 and :438-439; this
// kernel implements the mathematically correct stride).
#include "common.cuh"

namespace {

// Per-nonzero tap table: idx k decoded once per kernel shape to cin<<16 | kh<<8 | kw.
__global__ void build_taps_kernel(const uint32_t* __restrict__ idx, const uint32_t* __restrict__ nnz,
                                  uint32_t m, uint32_t pitch, uint32_t kH, uint32_t kW,
                                  uint32_t* __restrict__ taps)
{
    const uint32_t row = blockIdx.x;
    if (row >= m) return;
    const uint32_t nn = nnz[row];
    for (uint32_t j = threadIdx.x; j < nn; j += blockDim.x) {
        const uint32_t k = idx[(size_t)row * pitch + j];
        const uint32_t kw = k % kW;
        const uint32_t kh = (k / kW) % kH;
        const uint32_t cin = k / (kW * kH);
        taps[(size_t)row * pitch + j] = (cin << 16) | (kh << 8) | kw;
    }
}

struct ConvParams {
    uint32_t Cin, Cout, kH, kW, sH, sW, pH, pW, dH, dW, H, W, Ho, Wo, B;
};

// General kernel: one thread per output element, any layout, any geometry.  Threads of a warp
// are adjacent along the fastest output dimension (batch for PF, width for NCHW), so input
// reads of a tap are coalesced and the row's (w, tap) reads are warp-uniform.
template <int LAYOUT>
__global__ void __launch_bounds__(256)
conv_direct_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ taps,
                   const uint32_t* __restrict__ nnz, uint32_t pitch, ConvParams p,
                   const float* __restrict__ in, const float* __restrict__ bias, int act,
                   float* __restrict__ out)
{
    const uint64_t per_m = (uint64_t)p.Ho * p.Wo * p.B;
    const uint64_t col = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t mo = blockIdx.y;
    if (col >= per_m) return;
    uint32_t b, oh, ow;
    if (LAYOUT == SPX_LAYOUT_PF) {
        b = (uint32_t)(col % p.B);
        const uint64_t px = col / p.B;
        ow = (uint32_t)(px % p.Wo);
        oh = (uint32_t)(px / p.Wo);
    } else {
        ow = (uint32_t)(col % p.Wo);
        const uint64_t t = col / p.Wo;
        oh = (uint32_t)(t % p.Ho);
        b = (uint32_t)(t / p.Ho);
    }
    const int ih0 = (int)(oh * p.sH) - (int)p.pH;
    const int iw0 = (int)(ow * p.sW) - (int)p.pW;
    const float* __restrict__ w = Wd + (size_t)mo * pitch;
    const uint32_t* __restrict__ tp = taps + (size_t)mo * pitch;
    const uint32_t nn = __ldg(nnz + mo);
    float acc = bias ? __ldg(bias + mo) : 0.0f;
    for (uint32_t j = 0; j < nn; ++j) {
        const uint32_t t = __ldg(tp + j);
        const uint32_t cin = t >> 16;
        const int ih = ih0 + (int)(((t >> 8) & 0xffu) * p.dH);
        const int iw = iw0 + (int)((t & 0xffu) * p.dW);
        float xv = 0.0f;
        if ((unsigned)ih < p.H && (unsigned)iw < p.W) {
            const size_t off = LAYOUT == SPX_LAYOUT_PF
                ? (((size_t)cin * p.H + ih) * p.W + iw) * p.B + b
                : (((size_t)b * p.Cin + cin) * p.H + ih) * p.W + iw;
            xv = __ldg(in + off);
        }
        acc = fmaf(__ldg(w + j), xv, acc);
    }
    acc = spx::apply_act(acc, act);
    const size_t o = LAYOUT == SPX_LAYOUT_PF
        ? (((size_t)mo * p.Ho + oh) * p.Wo + ow) * p.B + b
        : (((size_t)b * p.Cout + mo) * p.Ho + oh) * p.Wo + ow;
    out[o] = acc;
}

}  // namespace

namespace spx {

static int ensure_taps(spx_ell* e, uint32_t kH, uint32_t kW, cudaStream_t s)
{
    if (e->taps && e->taps_kH == kH && e->taps_kW == kW) return SPX_OK;
    if (e->r == 0) return SPX_OK;
    if (!e->taps) SPX_CUDA(cudaMalloc(&e->taps, (size_t)e->m * e->pitch * sizeof(uint32_t)));
    build_taps_kernel<<<e->m, 128, 0, s>>>(e->idx, e->nnz, e->m, e->pitch, kH, kW, e->taps);
    SPX_LAUNCH_CHECK("build_taps_kernel");
    e->taps_kH = kH;
    e->taps_kW = kW;
    return SPX_OK;
}

int launch_conv2d(spx_ell* e, const spx_conv_geom* g, int layout, const float* in, uint32_t B,
                  const float* bias, int act, float* out, cudaStream_t s)
{
    if (e->m == 0 || B == 0 || g->Ho == 0 || g->Wo == 0) return SPX_OK;
    if (g->kH > 255 || g->kW > 255 || g->Cin > 65535)
        return fail(SPX_ERR_LIMIT, "conv2d: kernel extent > 255 or Cin > 65535 not supported");
    int rc = ensure_taps(e, g->kH, g->kW, s);
    if (rc != SPX_OK) return rc;
    ConvParams p{g->Cin, g->Cout, g->kH, g->kW, g->sH, g->sW, g->pH, g->pW, g->dH, g->dW,
                 g->H, g->W, g->Ho, g->Wo, B};
    const uint64_t per_m = (uint64_t)g->Ho * g->Wo * B;
    const uint64_t gx = (per_m + 255) / 256;
    if (gx > 0x7fffffffull || e->m > 65535)
        return fail(SPX_ERR_LIMIT, "conv2d: output too large for one launch");
    dim3 grid((unsigned)gx, e->m);
    if (layout == SPX_LAYOUT_PF)
        conv_direct_kernel<SPX_LAYOUT_PF><<<grid, 256, 0, s>>>(e->Wd, e->taps, e->nnz, e->pitch, p, in, bias, act, out);
    else
        conv_direct_kernel<SPX_LAYOUT_NCHW><<<grid, 256, 0, s>>>(e->Wd, e->taps, e->nnz, e->pitch, p, in, bias, act, out);
    SPX_LAUNCH_CHECK("conv_direct_kernel");
    return SPX_OK;
}

}  // namespace spx

// ---------------------------------------------------------------------------------------------
// spx_conv2d_static: the same convolution for callers that must not allocate device memory.
//
// Who cannot allocate: a host program that gives the whole device memory to its own pool at
// start-up (typical for inference servers) has nothing left for a later cudaMalloc, and a
// latency-bound serving loop cannot afford the device-wide synchronisation an allocation or a
// free may imply.  spx_conv2d allocates once per handle (its tap table).  This variant keeps
// the tap table in a fixed array that is part of the library image instead, so the call
// itself never allocates or frees anything: no cudaMalloc / cudaFree, no allocating library
// routine.  The price: every GPU that loads the library holds the array (4 MiB) until the
// process exits, and a weight matrix whose padded slab (Cout * pitch) has more slots than the
// array is rejected with SPX_ERR_LIMIT.
//
// The array is shared by all calls and keeps the previous call's contents.  Each call first
// rewrites the slots its own convolution reads (nothing has to start at zero), but two calls
// that overlap on the GPU (different streams or threads) would overwrite each other's table:
// serialise them.  The first call on a device looks the array's device address up
// (cudaGetSymbolAddress); make that first call before any stream capture begins.
// ---------------------------------------------------------------------------------------------
#include <mutex>

constexpr uint32_t kStaticTapSlots = 1u << 20;          // 4 MiB of uint32 slots
static __device__ __align__(256) uint32_t spx_static_taps[kStaticTapSlots];

// In host code `spx_static_taps` is only a handle for the runtime, not a device address.  The
// address is fetched once per device, with that device current, and cached.
static int static_taps_address(int device, uint32_t** out)
{
    static std::mutex mu;
    static uint32_t* cached[64] = {};
    if (device < 0 || device >= 64) return spx::fail(SPX_ERR_LIMIT, "conv2d_static: device ordinal %d not supported", device);
    std::lock_guard<std::mutex> lk(mu);
    if (!cached[device]) {
        void* p = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&p, spx_static_taps);
        if (err != cudaSuccess || !p)
            return spx::fail(SPX_ERR_CUDA, "conv2d_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
        cached[device] = static_cast<uint32_t*>(p);
    }
    *out = cached[device];
    return SPX_OK;
}

extern "C" int spx_conv2d_static(const spx_ell* e, const spx_conv_geom* g, int layout, const float* in, uint32_t B,
                                 const float* bias, int act, float* out, void* stream)
{
    using spx::fail;
    if (!e || !g) return fail(SPX_ERR_ARG, "handle / geometry is null");
    if (layout != SPX_LAYOUT_PF && layout != SPX_LAYOUT_NCHW) return fail(SPX_ERR_ARG, "unknown layout %d", layout);
    if (act < SPX_ACT_NONE || act > SPX_ACT_TANH) return fail(SPX_ERR_ARG, "unknown activation %d", act);
    if (g->sH == 0 || g->sW == 0 || g->dH == 0 || g->dW == 0 || g->kH == 0 || g->kW == 0)
        return fail(SPX_ERR_ARG, "stride, dilation and kernel extent must be positive");
    if (e->m != g->Cout) return fail(SPX_ERR_ARG, "ELLPACK rows (%u) != Cout (%u)", e->m, g->Cout);
    if ((uint64_t)g->Cin * g->kH * g->kW != e->n) return fail(SPX_ERR_ARG, "ELLPACK columns (%u) != Cin*kH*kW", e->n);
    const uint32_t eh = g->dH * (g->kH - 1) + 1, ew = g->dW * (g->kW - 1) + 1;
    if (g->H + 2 * g->pH < eh || g->W + 2 * g->pW < ew) return fail(SPX_ERR_ARG, "kernel larger than padded input");
    if (g->Ho != (g->H + 2 * g->pH - eh) / g->sH + 1 || g->Wo != (g->W + 2 * g->pW - ew) / g->sW + 1)
        return fail(SPX_ERR_ARG, "Ho / Wo inconsistent with the geometry");
    if (g->kH > 255 || g->kW > 255 || g->Cin > 65535)
        return fail(SPX_ERR_LIMIT, "conv2d_static: kernel extent > 255 or Cin > 65535 not supported");
    if (B == 0 || e->m == 0 || g->Ho == 0 || g->Wo == 0) return SPX_OK;
    if (!in || !out) return fail(SPX_ERR_ARG, "in / out is null");
    const uint64_t slots = (uint64_t)e->m * e->pitch;
    if (slots > kStaticTapSlots)
        return fail(SPX_ERR_LIMIT, "conv2d_static: weight slab has %llu slots (Cout * padded row length), the fixed "
                    "tap table holds %u; use spx_conv2d", (unsigned long long)slots, kStaticTapSlots);
    int cur = -1;
    SPX_CUDA(cudaGetDevice(&cur));
    if (cur != e->device)
        return fail(SPX_ERR_ARG, "conv2d_static: the handle's device (%d) must be current (current: %d)", e->device, cur);
    uint32_t* taps = nullptr;
    int rc = static_taps_address(cur, &taps);
    if (rc != SPX_OK) return rc;

    cudaStream_t s = (cudaStream_t)stream;
    if (e->r) {
        build_taps_kernel<<<e->m, 128, 0, s>>>(e->idx, e->nnz, e->m, e->pitch, g->kH, g->kW, taps);
        SPX_LAUNCH_CHECK("build_taps_kernel");
    }
    ConvParams p{g->Cin, g->Cout, g->kH, g->kW, g->sH, g->sW, g->pH, g->pW, g->dH, g->dW, g->H, g->W, g->Ho, g->Wo, B};
    const uint64_t per_m = (uint64_t)g->Ho * g->Wo * B;
    const uint64_t gx = (per_m + 255) / 256;
    if (gx > 0x7fffffffull || e->m > 65535) return fail(SPX_ERR_LIMIT, "conv2d_static: output too large for one launch");
    dim3 grid((unsigned)gx, e->m);
    if (layout == SPX_LAYOUT_PF)
        conv_direct_kernel<SPX_LAYOUT_PF><<<grid, 256, 0, s>>>(e->Wd, taps, e->nnz, e->pitch, p, in, bias, act, out);
    else
        conv_direct_kernel<SPX_LAYOUT_NCHW><<<grid, 256, 0, s>>>(e->Wd, taps, e->nnz, e->pitch, p, in, bias, act, out);
    SPX_LAUNCH_CHECK("conv_direct_kernel");
    return SPX_OK;
}
