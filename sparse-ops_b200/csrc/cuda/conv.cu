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
