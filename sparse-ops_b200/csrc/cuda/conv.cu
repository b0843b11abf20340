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

#include <cuda.h>            // CUtensorMap and its enums only; the encoder is looked up at run time
#include <cudaTypedefs.h>

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

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
    } else if (LAYOUT == SPX_LAYOUT_FMAJOR) {
        b = (uint32_t)(col % p.B);
        const uint64_t px = col / p.B;
        oh = (uint32_t)(px % p.Ho);
        ow = (uint32_t)(px / p.Ho);
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
                : LAYOUT == SPX_LAYOUT_FMAJOR
                ? (((size_t)iw * p.H + ih) * p.Cin + cin) * p.B + b
                : (((size_t)b * p.Cin + cin) * p.H + ih) * p.W + iw;
            xv = __ldg(in + off);
        }
        acc = fmaf(__ldg(w + j), xv, acc);
    }
    acc = spx::apply_act(acc, act);
    const size_t o = LAYOUT == SPX_LAYOUT_PF
        ? (((size_t)mo * p.Ho + oh) * p.Wo + ow) * p.B + b
        : LAYOUT == SPX_LAYOUT_FMAJOR
        ? (((size_t)ow * p.Ho + oh) * p.Cout + mo) * p.B + b
        : (((size_t)b * p.Cout + mo) * p.Ho + oh) * p.Wo + ow;
    out[o] = acc;
}


// dst[c * rows + r] = src[r * cols + c]: used to run NCHW tensors ([B][C*H*W]) through the
// [C,H,W,B] kernel ([C*H*W][B]) and back.  32 x 32 tiles through padded shared memory, both
// sides coalesced.
template <bool ROWS_ON_X>   // which dimension is the long one and therefore rides on gridDim.x
__global__ void __launch_bounds__(256)
transpose2d_kernel(const float* __restrict__ src, uint64_t rows, uint64_t cols, float* __restrict__ dst)
{
    __shared__ float t[32][33];
    const uint64_t c0 = (uint64_t)(ROWS_ON_X ? blockIdx.y : blockIdx.x) * 32;
    const uint64_t r0 = (uint64_t)(ROWS_ON_X ? blockIdx.x : blockIdx.y) * 32;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;     // 32 x 8
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        const uint64_t r = r0 + ty + i;
        const uint64_t c = c0 + tx;
        if (r < rows && c < cols) t[ty + i][tx] = src[(size_t)r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        const uint64_t c = c0 + ty + i;
        const uint64_t r = r0 + tx;
        if (r < rows && c < cols) dst[(size_t)c * rows + r] = t[tx][ty + i];
    }
}

// dst[r * dst_pitch + c] = c < src_cols ? src[r * src_pitch + c] : 0  for c < dst_cols: widens the
// batch dimension of a [C,H,W,B] tensor to a multiple of 4 (zeros in the added entries) or narrows
// it back.
__global__ void __launch_bounds__(256)
repitch_kernel(const float* __restrict__ src, uint32_t src_pitch, uint32_t src_cols,
               float* __restrict__ dst, uint32_t dst_pitch, uint32_t dst_cols, uint64_t rows)
{
    const uint64_t total = rows * dst_cols;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / dst_cols;
        const uint32_t c = (uint32_t)(i - r * dst_cols);
        dst[r * dst_pitch + c] = c < src_cols ? src[r * src_pitch + c] : 0.0f;
    }
}

// dst[k][j][i][b] = src[i][j][k][b]: reverses the three outer dimensions (D0, D1, D2) of a tensor whose
// innermost dimension B stays contiguous -- F-major [W,H,C,B] to [C,H,W,B] and back.
__global__ void __launch_bounds__(256)
reverse3_kernel(const float* __restrict__ src, uint32_t D0, uint32_t D1, uint32_t D2, uint32_t B,
                float* __restrict__ dst)
{
    const uint64_t total = (uint64_t)D0 * D1 * D2 * B;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t b = (uint32_t)(t % B);
        uint64_t r = t / B;
        const uint32_t i = (uint32_t)(r % D0);
        r /= D0;
        const uint32_t j = (uint32_t)(r % D1);
        const uint32_t k = (uint32_t)(r / D1);
        dst[t] = __ldg(src + ((((uint64_t)i * D1 + j) * D2 + k) * B + b));
    }
}

// ---------------------------------------------------------------------------------------------
// conv_pf_tile_kernel: the fast path for the [C,H,W,B] layout with B % 4 == 0.
//
// A CTA owns a tile of 4 x 8 (2 x 8 at a full batch tile of 32) output positions x BT batch entries
// x 16 (32) output channels: one warp per output channel, accumulators in registers for the whole
// kernel.  It walks the input channels in chunks: the chunk's input patch (CC channels x the tile's receptive field x BT) is
// staged in shared memory with 16-byte cp.async copies, positions outside the image are stored as
// zeros (so a tap there contributes the operand 0.0f exactly like the reference's zero-filled
// im2col tile), and every warp then consumes the nonzeros of its weight row whose input channel
// lies in the chunk -- they are contiguous because rows are sorted by k = (cin, kh, kw).
// Per nonzero: (w, tap offset) are read coalesced 32 at a time and broadcast with two shuffles,
// then G float4 shared-memory loads feed 4*G FMAs per lane.  A quarter-warp always reads 128
// contiguous bytes, so the loads are bank-conflict free for stride 1.
//
// Bound: one 4-byte operand per FMA from shared memory = 128 B/clk/SM = 32 FMA/clk/SM, a quarter
// of the FP32 peak; HBM / L2 traffic is the input patch once per CTA (16 or 32 output channels)
// plus the output once.
// ---------------------------------------------------------------------------------------------
#ifndef SPX_CONV_FMA2
#define SPX_CONV_FMA2 1         // packed fma.rn.f32x2 in the tiled kernels (same rounding per element)
#endif
constexpr int kTileH = 4, kTileW = 8, kTileWarps = 16;

struct TileParams {
    ConvParams c;
    uint32_t BT;        // batch entries per CTA (multiple of 4, <= 32)
    uint32_t CC;        // input channels per staged chunk
    uint32_t THin, TWin;
    uint32_t tilesX;
    uint32_t stage;     // floats between the two staging buffers of the bulk-copy path (0: one buffer)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// ---- bulk tensor copies (TMA) for the staged input patch -----------------------------------------
// One thread asks the copy unit for the whole [channels][rows][columns][batch] box of a chunk; the
// unit writes it into shared memory (zeros where the box leaves the image) and signals an mbarrier
// with the byte count.  No multicast, the tensor map covers this GPU's own input tensor only.
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
                   "r"((uint32_t)__cvta_generic_to_shared(bar)) : "memory");
}
// Waits for the phase with the given parity; gives up one second (of the GPU's wall clock) after
// its 256th unsuccessful poll and returns false, so a copy that never completes cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(bar);
    uint64_t t0 = 0;
    for (uint32_t i = 1;; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(a), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 255u) == 0) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 1000000000ull) return false;
        }
    }
}

// Stages input channels [c0, c1) of a CTA's receptive field in shared memory as
// [channel][row][column][BT batch entries]: one warp per (channel, row), 16-byte cp.async copies,
// zeros where the row or column lies outside the image.  Ends with the copies landed and the CTA
// synchronised.
template <int QB, int WARPS>
__device__ __forceinline__ void stage_chunk(float* tile, const TileParams& tp, const float* __restrict__ in,
                                            uint32_t c0, uint32_t c1, int ih0, int iw0, uint32_t b0,
                                            int warp, int lane)
{
    const ConvParams& p = tp.c;
    const uint32_t rowUnits = tp.TWin * QB;             // float4 units per staged row
    const uint32_t rows = (c1 - c0) * tp.THin;
    for (uint32_t r = warp; r < rows; r += WARPS) {
        const uint32_t c = r / tp.THin, y = r % tp.THin;
        const int ih = ih0 + (int)y;
        const bool rowok = (unsigned)ih < p.H;
        float* srow = tile + (size_t)r * rowUnits * 4;
        const float* grow = in + (((size_t)(c0 + c) * p.H + (rowok ? ih : 0)) * p.W) * p.B + b0;
        for (uint32_t u = lane; u < rowUnits; u += 32) {
            const uint32_t x = u / QB, q = u % QB;
            const int iw = iw0 + (int)x;
            if (rowok && (unsigned)iw < p.W) cp_async16(srow + u * 4, grow + (size_t)iw * p.B + q * 4);
            else *reinterpret_cast<float4*>(srow + u * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    cp_async_wait_all();
    __syncthreads();
}

// QB: batch quads per output position (= BT / 4); G: float4 groups per lane, so a warp covers
// 32*G/QB positions (kTileW wide); WARPS: output channels per CTA; MINB: CTAs per SM aimed for.
template <int QB, int G, int WARPS, int MINB>
__global__ void __launch_bounds__(WARPS * 32, MINB)
conv_pf_tile_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ taps,
                    const uint32_t* __restrict__ nnz, uint32_t pitch, TileParams tp,
                    const float* __restrict__ in, const float* __restrict__ bias, int act,
                    float* __restrict__ out)
{
    extern __shared__ __align__(128) float tile[];
    const ConvParams& p = tp.c;
    const uint32_t BT = QB * 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t ty = blockIdx.x / tp.tilesX, tx = blockIdx.x % tp.tilesX;
    constexpr uint32_t TH = 32u * G / QB / kTileW;       // tile height in output positions
    const uint32_t oh0 = ty * TH, ow0 = tx * kTileW;
    const uint32_t b0 = blockIdx.z * BT;
    const uint32_t mo = blockIdx.y * WARPS + warp;
    const bool active = mo < p.Cout;
    const int ih0 = (int)(oh0 * p.sH) - (int)p.pH;      // image row of staged row 0
    const int iw0 = (int)(ow0 * p.sW) - (int)p.pW;

    // this lane's G output units: unit q = lane + 32 g -> (position, batch quad)
    uint32_t off[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint32_t q = lane + 32u * g;
        const uint32_t pix = q / QB, quad = q % QB;
        const uint32_t py = pix / kTileW, px = pix % kTileW;
        off[g] = ((py * p.sH) * tp.TWin + px * p.sW) * BT + quad * 4;
    }
    const float bv = (active && bias) ? __ldg(bias + mo) : 0.0f;
    float4 acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g] = make_float4(bv, bv, bv, bv);

    const uint32_t nn = active ? __ldg(nnz + mo) : 0u;
    const float* __restrict__ wrow = Wd + (size_t)(active ? mo : 0) * pitch;
    const uint32_t* __restrict__ trow = taps + (size_t)(active ? mo : 0) * pitch;
    uint32_t pos = 0;

    for (uint32_t c0 = 0; c0 < p.Cin; c0 += tp.CC) {
        const uint32_t c1 = min(p.Cin, c0 + tp.CC);
        stage_chunk<QB, WARPS>(tile, tp, in, c0, c1, ih0, iw0, b0, warp, lane);
        // ---- consume this row's nonzeros whose input channel is in [c0, c1) ----
        if (active) {
            for (;;) {
                float wl = 0.0f;
                uint32_t tl = 0, cin = 0xffffffffu;
                if (pos + lane < nn) {
                    wl = __ldg(wrow + pos + lane);
                    const uint32_t t = __ldg(trow + pos + lane);
                    cin = t >> 16;
                    tl = (((cin - c0) * tp.THin + ((t >> 8) & 0xffu) * p.dH) * tp.TWin + (t & 0xffu) * p.dW) * BT;
                }
                const uint32_t cnt = __popc(__ballot_sync(0xffffffffu, cin < c1));   // a prefix: rows are sorted by k
                for (uint32_t t = 0; t < cnt; ++t) {
                    const float wt = __shfl_sync(0xffffffffu, wl, t);
                    const float* xs = tile + __shfl_sync(0xffffffffu, tl, t);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 xv = *reinterpret_cast<const float4*>(xs + off[g]);
#if SPX_CONV_FMA2
                        spx::fma_pair(acc[g].x, acc[g].y, wt, xv.x, xv.y);
                        spx::fma_pair(acc[g].z, acc[g].w, wt, xv.z, xv.w);
#else
                        acc[g].x = fmaf(wt, xv.x, acc[g].x);
                        acc[g].y = fmaf(wt, xv.y, acc[g].y);
                        acc[g].z = fmaf(wt, xv.z, acc[g].z);
                        acc[g].w = fmaf(wt, xv.w, acc[g].w);
#endif
                    }
                }
                pos += cnt;
                if (cnt < 32) break;
            }
        }
        __syncthreads();
    }
    if (!active) return;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint32_t q = lane + 32u * g;
        const uint32_t pix = q / QB, quad = q % QB;
        const uint32_t oh = oh0 + pix / kTileW, ow = ow0 + pix % kTileW;
        if (oh < p.Ho && ow < p.Wo) {
            float4 o = acc[g];
            if (act != SPX_ACT_NONE) {
                o.x = spx::apply_act(o.x, act); o.y = spx::apply_act(o.y, act);
                o.z = spx::apply_act(o.z, act); o.w = spx::apply_act(o.w, act);
            }
            *reinterpret_cast<float4*>(out + (((size_t)mo * p.Ho + oh) * p.Wo + ow) * p.B + b0 + quad * 4) = o;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Row-block-merged weights.  The reference's build_rbm_from_ellpack (src/layers/rbm_conv.cpp:7-73)
// merges the column ids of consecutive weight rows into one ascending list so that a patch
// operand is fetched once per block of rows instead of once per row; its consumer
// (conv2d_rbm_fmajor_implicit, src/layers/conv_kernels.cpp:66-147) is not called at its HEAD.
// Here the same merge feeds the tiled kernel below, with blocks of 4 rows (8 rows, the
// reference's block, measured slower at every density: twice the mask tests per union column).
// Device form, per block b of 4 rows:
//   hdr[b*cap + c] = (packed tap cin<<16 | kh<<8 | kw of union column c,  bit r set when row
//                     4b + r stores that column)
//   w[(b*cap + c)*4 + r] = that row's weight, 0.0f where the bit is clear (never multiplied)
//   ncols[b] = number of union columns.
// One CTA per block: a K-bit set in shared memory collects the columns, a scan over its words
// ranks them, a second pass over the rows scatters taps, masks and weights.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kRbmRows = 4;
constexpr uint32_t kRbmMaxK = 1u << 17;         // 2 x 16 KB of shared memory for the set and its ranks

__global__ void __launch_bounds__(256)
build_rbm_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ idx, const uint32_t* __restrict__ nnz,
                 uint32_t m, uint32_t K, uint32_t pitch, uint32_t kH, uint32_t kW, uint32_t cap,
                 uint2* __restrict__ hdr, float* __restrict__ w4, uint32_t* __restrict__ ncols)
{
    extern __shared__ uint32_t rbm_sm[];
    const uint32_t words = (K + 31) / 32;
    uint32_t* set = rbm_sm;
    uint32_t* rank = rbm_sm + words;
    __shared__ uint32_t total_s;
    const uint32_t blk = blockIdx.x, r0 = blk * kRbmRows;
    for (uint32_t i = threadIdx.x; i < words; i += blockDim.x) set[i] = 0;
    __syncthreads();
    for (uint32_t r = 0; r < kRbmRows && r0 + r < m; ++r) {
        const uint32_t row = r0 + r, nn = nnz[row];
        for (uint32_t j = threadIdx.x; j < nn; j += blockDim.x) {
            const uint32_t k = idx[(size_t)row * pitch + j];
            atomicOr(&set[k >> 5], 1u << (k & 31));
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) {                     // exclusive scan of the words' popcounts, 32 at a time
        uint32_t run = 0;
        for (uint32_t w0 = 0; w0 < words; w0 += 32) {
            const uint32_t i = w0 + threadIdx.x;
            const uint32_t c = i < words ? __popc(set[i]) : 0u;
            uint32_t inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, inc, o);
                if ((int)threadIdx.x >= o) inc += v;
            }
            if (i < words) rank[i] = run + inc - c;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (threadIdx.x == 0) { total_s = run; ncols[blk] = run; }
    }
    __syncthreads();
    const uint32_t total = total_s;
    const size_t base = (size_t)blk * cap;
    for (uint32_t c = threadIdx.x; c < total; c += blockDim.x) hdr[base + c] = make_uint2(0u, 0u);
    for (uint32_t c = threadIdx.x; c < total * kRbmRows; c += blockDim.x) w4[base * kRbmRows + c] = 0.0f;
    __syncthreads();
    for (uint32_t r = 0; r < kRbmRows && r0 + r < m; ++r) {
        const uint32_t row = r0 + r, nn = nnz[row];
        for (uint32_t j = threadIdx.x; j < nn; j += blockDim.x) {
            const uint32_t k = idx[(size_t)row * pitch + j];
            const uint32_t c = rank[k >> 5] + __popc(set[k >> 5] & ((1u << (k & 31)) - 1u));
            const uint32_t kw = k % kW, kh = (k / kW) % kH, cin = k / (kW * kH);
            hdr[base + c].x = (cin << 16) | (kh << 8) | kw;      // the same value from every row
            atomicOr(&hdr[base + c].y, 1u << r);
            w4[(base + c) * kRbmRows + r] = Wd[(size_t)row * pitch + j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// conv_rbm_tile_kernel: the tiled kernel over row-block-merged weights.
//
// Same CTA structure as conv_pf_tile_kernel (input chunk staged in shared memory, accumulators
// in registers for the whole kernel), but a warp owns a block of 4 output channels x 128/QB
// positions: per union column it loads its 4 float4 patch operands ONCE and applies them to
// every row of the block that stores the column (mask bits tested with warp-uniform branches;
// the row's weight is broadcast from the lane that preloaded the column).  Shared-memory loads
// per FMA drop by the mean number of rows per union column (1.36 at 80 % sparsity, 2.1 at
// 50 %, 4 for a dense weight), which is what bounds conv_pf_tile_kernel; the price is the mask
// tests, so the kernel is issue-bound rather than shared-memory-bound.  A row still sees its
// nonzeros in ascending k with one FMA each: results are bit-identical to the per-row kernels.
// The CTA's NB warps are NB row blocks on one tile of positions.
// ---------------------------------------------------------------------------------------------
constexpr int kRbmG = 4;                                 // float4 groups per lane: 4 rows x 4 groups = 64 accumulators

// One row of the block: when the union column holds an entry of row R, fetch its weight from the
// lane that preloaded the column and run the row's 16 FMAs.  The test is warp-uniform.
template <int R, int G>
__device__ __forceinline__ void rbm_row(float4 (&acc)[kRbmRows][G], uint32_t hm, float wsrc, uint32_t t,
                                        const float4 (&x)[G])
{
    if (hm & (1u << R)) {
        const float wt = __shfl_sync(0xffffffffu, wsrc, t);
#pragma unroll
        for (int g = 0; g < G; ++g) {
#if SPX_CONV_FMA2
            spx::fma_pair(acc[R][g].x, acc[R][g].y, wt, x[g].x, x[g].y);
            spx::fma_pair(acc[R][g].z, acc[R][g].w, wt, x[g].z, x[g].w);
#else
            acc[R][g].x = fmaf(wt, x[g].x, acc[R][g].x);
            acc[R][g].y = fmaf(wt, x[g].y, acc[R][g].y);
            acc[R][g].z = fmaf(wt, x[g].z, acc[R][g].z);
            acc[R][g].w = fmaf(wt, x[g].w, acc[R][g].w);
#endif
        }
    }
}

// Work units are (tile of positions, group of NB row blocks, batch tile), numbered tile-fastest.
// G = kRbmG: the CTA takes unit `unit0 + blockIdx.x`.  G = kRbmG / 2 (half-height tiles): CTAs
// 2u and 2u + 1 take the upper and lower half of unit `unit0 + u`; used for the last, partly
// filled wave of a launch so that its work spreads over twice as many SMs.
struct RbmUnits {
    uint32_t unit0, tiles, groups;     // first unit of this launch; tiles per image; row-block groups
};

template <int QB, int NB, int G>
__global__ void __launch_bounds__(NB * 32, 1)
conv_rbm_tile_kernel(const uint2* __restrict__ hdr, const float4* __restrict__ w4,
                     const uint32_t* __restrict__ ncols, uint32_t cap, TileParams tp, RbmUnits un,
                     const float* __restrict__ in, const float* __restrict__ bias, int act,
                     float* __restrict__ out, const __grid_constant__ CUtensorMap tmap, uint32_t use_tma,
                     int* __restrict__ tma_failed, int* __restrict__ tma_failed_host)
{
    extern __shared__ __align__(128) float tile[];
    __shared__ __align__(8) uint64_t tile_bar[2];
    __shared__ uint32_t buf_done[2];      // warps that have finished the chunk held by buffer 0 / 1
    __shared__ uint32_t copies_asked;     // bulk copies this CTA has asked for
    constexpr int RB = (int)kRbmRows;
    constexpr uint32_t BT = QB * 4;
    constexpr uint32_t TH = 32u * G / QB / kTileW;       // rows of output positions per tile
    constexpr bool kHalf = G != kRbmG;
    const ConvParams& p = tp.c;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t unit = un.unit0 + (kHalf ? blockIdx.x >> 1 : blockIdx.x);
    const uint32_t t_id = unit % un.tiles, by = (unit / un.tiles) % un.groups, bz = unit / un.tiles / un.groups;
    const uint32_t ty = kHalf ? (t_id / tp.tilesX) * 2 + (blockIdx.x & 1) : t_id / tp.tilesX, tx = t_id % tp.tilesX;
    const uint32_t oh0 = ty * TH, ow0 = tx * kTileW;
    if (oh0 >= p.Ho) return;                             // lower half of a tile that ends above it
    const uint32_t b0 = bz * BT;
    const uint32_t blk = by * NB + warp;
    const uint32_t mo0 = blk * RB;
    const bool active = mo0 < p.Cout;
    const int ih0 = (int)(oh0 * p.sH) - (int)p.pH;
    const int iw0 = (int)(ow0 * p.sW) - (int)p.pW;

    uint32_t off[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint32_t q = lane + 32u * g;
        const uint32_t pix = q / QB, quad = q % QB;
        off[g] = (((pix / kTileW) * p.sH) * tp.TWin + (pix % kTileW) * p.sW) * BT + quad * 4;
    }
    float4 acc[RB][G];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const float bv = (bias && mo0 + r < p.Cout) ? __ldg(bias + mo0 + r) : 0.0f;
#pragma unroll
        for (int g = 0; g < G; ++g) acc[r][g] = make_float4(bv, bv, bv, bv);
    }
    const uint32_t nn = active ? __ldg(ncols + blk) : 0u;
    const uint2* __restrict__ hrow = hdr + (size_t)(active ? blk : 0) * cap;
    const float4* __restrict__ wrow = w4 + (size_t)(active ? blk : 0) * cap;
    uint32_t pos = 0;
    // Bulk-copy staging: two buffers of tp.CC channels each, filled by the copy unit (no load / store
    // slots of the 16 warps; the halo is the unit's zero fill; a box always has tp.CC channels, past
    // the last channel it reads zeros).  Chunks 0 and 1 are asked for at once.  A warp waits on the
    // buffer's mbarrier, multiplies, and counts itself out of the buffer; the warp that counts out
    // last asks for the chunk after next into that buffer.  So the warps of a CTA never meet at a
    // barrier: a warp with few columns in a chunk runs ahead into the next one.  Every wait is
    // bounded: after a wait that ran out the warp stops waiting, finishes on whatever the buffers
    // hold and raises *tma_failed (the host then reports the call as failed); no more copies are
    // asked for and CTAs that start later leave at once.
    // use_tma bit 1 (a test switch): the barrier is told to expect 16 bytes more than the copy
    // delivers, so the wait runs out and the failure report can be exercised without any fault.
    const uint32_t box_bytes = tp.CC * tp.THin * tp.TWin * BT * (uint32_t)sizeof(float) + ((use_tma & 2u) ? 16u : 0u);
    const uint32_t nchunks = (p.Cin + tp.CC - 1) / tp.CC;
    const uint32_t blocks_left = (p.Cout - min(p.Cout, by * NB * RB) + RB - 1) / RB;
    const uint32_t nactive = min((uint32_t)NB, blocks_left);       // warps of this CTA with rows
    bool landed = true;
    if (use_tma) {
        if (threadIdx.x == 0) {
            mbar_init(&tile_bar[0], 1);
            mbar_init(&tile_bar[1], 1);
            buf_done[0] = 0;
            buf_done[1] = 0;
            copies_asked = min(2u, nchunks);
        }
        if (__syncthreads_or(*reinterpret_cast<volatile int*>(tma_failed) != 0)) return;
        if (threadIdx.x == 0) {
            mbar_expect_tx(&tile_bar[0], box_bytes);
            tma_load_4d(tile, &tmap, (int)b0, iw0, ih0, 0, &tile_bar[0]);
            if (nchunks > 1) {
                mbar_expect_tx(&tile_bar[1], box_bytes);
                tma_load_4d(tile + tp.stage, &tmap, (int)b0, iw0, ih0, (int)tp.CC, &tile_bar[1]);
            }
        }
        if (!active) return;        // warps without rows take no part in the counting below
    }

    uint32_t chunk = 0;
    for (uint32_t c0 = 0; c0 < p.Cin; c0 += tp.CC, ++chunk) {
        const uint32_t c1 = min(p.Cin, c0 + tp.CC);
        const float* cur = tile;
        if (use_tma) {
            if (landed) landed = mbar_wait(&tile_bar[chunk & 1u], (chunk >> 1) & 1u);
            cur = tile + (chunk & 1u) * tp.stage;
        } else {
            stage_chunk<QB, NB>(tile, tp, in, c0, c1, ih0, iw0, b0, warp, lane);
        }
        if (active) {
            // lane l holds union column pos + l: header (packed tap, row mask) and its 4 weights.  The
            // operands of the next batch of 32 columns are asked for before this batch's FMAs, so the
            // round trip to L2 runs behind them.
            bool have = pos + lane < nn;
            uint2 h = make_uint2(0u, 0u);
            float4 wl = make_float4(0.f, 0.f, 0.f, 0.f);
            if (have) {
                h = __ldg(hrow + pos + lane);
                wl = __ldg(wrow + pos + lane);
            }
            for (;;) {
                const uint32_t cin = have ? (h.x >> 16) : 0xffffffffu;
                const uint32_t tl = (((cin - c0) * tp.THin + ((h.x >> 8) & 0xffu) * p.dH) * tp.TWin + (h.x & 0xffu) * p.dW) * BT;
                const uint32_t hl = (tl << 8) | h.y;      // shared-memory offset << 8 | row mask (unused beyond cnt)
                const uint32_t cnt = __popc(__ballot_sync(0xffffffffu, cin < c1));   // a prefix: columns ascend
                const uint32_t npos = pos + cnt;
                bool nhave = false;
                uint2 nh = make_uint2(0u, 0u);
                float4 nw = make_float4(0.f, 0.f, 0.f, 0.f);
                if (cnt == 32) {
                    nhave = npos + lane < nn;
                    if (nhave) {
                        nh = __ldg(hrow + npos + lane);
                        nw = __ldg(wrow + npos + lane);
                    }
                }
                for (uint32_t t = 0; t < cnt; ++t) {
                    const uint32_t hm = __shfl_sync(0xffffffffu, hl, t);
                    const float* xs = cur + (hm >> 8);
                    float4 x[G];
#pragma unroll
                    for (int g = 0; g < G; ++g) x[g] = *reinterpret_cast<const float4*>(xs + off[g]);
                    rbm_row<0, G>(acc, hm, wl.x, t, x);
                    rbm_row<1, G>(acc, hm, wl.y, t, x);
                    rbm_row<2, G>(acc, hm, wl.z, t, x);
                    rbm_row<3, G>(acc, hm, wl.w, t, x);
                }
                pos = npos;
                if (cnt < 32) break;
                have = nhave; h = nh; wl = nw;
            }
        }
        if (!use_tma) {
            __syncthreads();
            continue;
        }
        __syncwarp();
        if (lane == 0) {
            const uint32_t b = chunk & 1u;
            __threadfence_block();                                  // this warp's reads of the buffer, then the count
            if (atomicAdd(&buf_done[b], 1u) + 1u == nactive) {      // last warp out of the buffer
                buf_done[b] = 0;                                    // next counted out after the refill has landed
                if (landed && chunk + 2 < nchunks) {
                    __threadfence_block();
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // all warps' reads, then the unit's writes
                    mbar_expect_tx(&tile_bar[b], box_bytes);
                    tma_load_4d(tile + b * tp.stage, &tmap, (int)b0, iw0, ih0, (int)((chunk + 2) * tp.CC), &tile_bar[b]);
                    atomicAdd(&copies_asked, 1u);
                }
            }
        }
    }
    if (use_tma && !landed) {
        *tma_failed = 1;
        *tma_failed_host = 1;
        // the last two copies asked for may still be writing this CTA's shared memory: one more
        // bounded wait for each before this warp leaves (the memory stays until the last warp has)
        if (lane == 0) {
            const uint32_t asked = *reinterpret_cast<volatile uint32_t*>(&copies_asked);
            for (uint32_t j = asked > 2 ? asked - 2 : 0; j < asked; ++j)
                (void)mbar_wait(&tile_bar[j & 1u], (j >> 1) & 1u);
        }
    }
    if (!active) return;
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const uint32_t mo = mo0 + r;
        if (mo >= p.Cout) break;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint32_t q = lane + 32u * g;
            const uint32_t pix = q / QB, quad = q % QB;
            const uint32_t oh = oh0 + pix / kTileW, ow = ow0 + pix % kTileW;
            if (oh < p.Ho && ow < p.Wo) {
                float4 o = acc[r][g];
                if (act != SPX_ACT_NONE) {
                    o.x = spx::apply_act(o.x, act); o.y = spx::apply_act(o.y, act);
                    o.z = spx::apply_act(o.z, act); o.w = spx::apply_act(o.w, act);
                }
                *reinterpret_cast<float4*>(out + (((size_t)mo * p.Ho + oh) * p.Wo + ow) * p.B + b0 + quad * 4) = o;
            }
        }
    }
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

template <int QB, int G, int WARPS, int MINB>
static int launch_tile_qb(const spx_ell* e, const TileParams& tp, dim3 grid, size_t smem, const float* in,
                          const float* bias, int act, float* out, cudaStream_t s)
{
    auto kfn = conv_pf_tile_kernel<QB, G, WARPS, MINB>;
    cudaError_t err = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return fail(SPX_ERR_CUDA, "conv2d: shared memory opt-in failed: %s", cudaGetErrorString(err));
    kfn<<<grid, WARPS * 32, smem, s>>>(e->Wd, e->taps, e->nnz, e->pitch, tp, in, bias, act, out);
    SPX_LAUNCH_CHECK("conv_pf_tile_kernel");
    return SPX_OK;
}

// Shapes the tiled kernel covers: batch a multiple of 4, one channel of the tile's receptive field
// within the shared-memory budget, grid within limits.
static bool pf_tile_covers(const ConvParams& p)
{
    static const bool disabled = [] { const char* v = getenv("SPX_CONV_DIRECT"); return v && v[0] == '1'; }();
    if (disabled || p.B % 4 != 0) return false;
    const size_t THin = (kTileH - 1) * p.sH + (p.kH - 1) * p.dH + 1, TWin = (kTileW - 1) * p.sW + (p.kW - 1) * p.dW + 1;
    uint32_t BT = 0;
    for (uint32_t c = 32; c >= 4; c -= 4) if (p.B % c == 0) { BT = c; break; }
    if (!BT || THin * TWin * BT * sizeof(float) > 100 * 1024) return false;
    const uint64_t tiles = (uint64_t)((p.Wo + kTileW - 1) / kTileW) * ((p.Ho + kTileH - 1) / kTileH);
    return tiles <= 0x7fffffffull && (p.Cout + kTileWarps - 1) / kTileWarps <= 65535 && p.B / BT <= 65535;
}

static int transpose2d(const float* src, uint64_t rows, uint64_t cols, float* dst, cudaStream_t s)
{
    const uint64_t rt = (rows + 31) / 32, ct = (cols + 31) / 32;
    const bool rows_on_x = rows >= cols;
    const uint64_t gx = rows_on_x ? rt : ct, gy = rows_on_x ? ct : rt;
    if (gx > 0x7fffffffull || gy > 65535) return fail(SPX_ERR_LIMIT, "conv2d: tensor too large to transpose");
    if (rows_on_x) transpose2d_kernel<true><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, s>>>(src, rows, cols, dst);
    else           transpose2d_kernel<false><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, s>>>(src, rows, cols, dst);
    SPX_LAUNCH_CHECK("transpose2d_kernel");
    return SPX_OK;
}

// Builds (once per handle and kernel shape) the row-block-merged weights.
static int ensure_rbm(spx_ell* e, uint32_t kH, uint32_t kW, cudaStream_t s)
{
    if (e->rbm_hdr && e->rbm_kH == kH && e->rbm_kW == kW) return SPX_OK;
    const uint32_t nblocks = (e->m + kRbmRows - 1) / kRbmRows;
    if (!e->rbm_hdr) {
        // Up to three times the ELLPACK slab (24 bytes per union column, at most 4 * max_nnz columns
        // per block of 4 rows).  Without room for it the per-row kernel is used instead.
        if (e->rbm_cap == UINT32_MAX) return -1;        // an earlier attempt ran out of memory
        const uint32_t cap = (uint32_t)std::min<uint64_t>((uint64_t)kRbmRows * e->max_nnz, e->n);
        if (cudaMalloc(&e->rbm_ncols, (size_t)nblocks * sizeof(uint32_t)) != cudaSuccess ||
            cudaMalloc(&e->rbm_w, (size_t)nblocks * cap * kRbmRows * sizeof(float)) != cudaSuccess ||
            cudaMalloc(&e->rbm_hdr, (size_t)nblocks * cap * sizeof(uint2)) != cudaSuccess) {
            (void)cudaGetLastError();
            cudaFree(e->rbm_ncols); cudaFree(e->rbm_w); cudaFree(e->rbm_hdr);
            e->rbm_ncols = nullptr; e->rbm_w = nullptr; e->rbm_hdr = nullptr;
            e->rbm_cap = UINT32_MAX;
            return -1;
        }
        e->rbm_cap = cap;
        // Two words for a kernel whose bounded wait for a bulk tensor copy runs out: one in device
        // memory, which CTAs that start later read and leave on, and one in pinned host memory
        // (only ever written by the kernel: a read of host memory costs an SM about a microsecond),
        // which the next convolution call on the handle reports.
        if (!e->tma_failed_host && cudaHostAlloc(reinterpret_cast<void**>(&e->tma_failed_host), sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
            *e->tma_failed_host = 0;
            if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&e->tma_failed_mapped), e->tma_failed_host, 0) != cudaSuccess ||
                cudaMalloc(reinterpret_cast<void**>(&e->tma_failed_dev), sizeof(int)) != cudaSuccess ||
                cudaMemset(e->tma_failed_dev, 0, sizeof(int)) != cudaSuccess) {
                e->tma_failed_mapped = nullptr;
                if (e->tma_failed_dev) cudaFree(e->tma_failed_dev);
                e->tma_failed_dev = nullptr;
            }
        }
        (void)cudaGetLastError();
    }
    const size_t smem = (size_t)((e->n + 31) / 32) * 2 * sizeof(uint32_t);
    build_rbm_kernel<<<nblocks, 256, smem, s>>>(e->Wd, e->idx, e->nnz, e->m, e->n, e->pitch, kH, kW, e->rbm_cap,
                                                e->rbm_hdr, e->rbm_w, e->rbm_ncols);
    SPX_LAUNCH_CHECK("build_rbm_kernel");
    e->rbm_kH = kH;
    e->rbm_kW = kW;
    return SPX_OK;
}

// cuTensorMapEncodeTiled, looked up through the runtime (the library does not link libcuda).
static PFN_cuTensorMapEncodeTiled tensor_map_encoder()
{
    static const PFN_cuTensorMapEncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            p = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }();
    return fn;
}

template <int QB, int G>
static int launch_rbm_units(const spx_ell* e, TileParams tp, RbmUnits un, uint32_t ctas, const float* in, const float* bias,
                            int act, float* out, cudaStream_t s, uint32_t b_avail)
{
    constexpr int NB = 16;
    const ConvParams& p = tp.c;
    constexpr uint32_t TH = 32u * G / QB / kTileW;
    tp.BT = QB * 4;
    tp.THin = (TH - 1) * p.sH + (p.kH - 1) * p.dH + 1;
    tp.TWin = (kTileW - 1) * p.sW + (p.kW - 1) * p.dW + 1;
    const size_t chanBytes = (size_t)tp.THin * tp.TWin * tp.BT * sizeof(float);
    const size_t budget = 200 * 1024;
    tp.CC = (uint32_t)std::min<size_t>(p.Cin, budget / chanBytes);
    // The chunk's patch as one bulk tensor copy (TMA) where a map of the input tensor can be made:
    // dimensions, innermost first, [B][W][H][Cin]; box [BT][TWin][THin][CC] (each extent at most
    // 256); positions outside the tensor read as zero, which is the halo.  The innermost
    // coordinate of every copy is a multiple of BT floats, i.e. of 16 bytes, as the copy unit
    // requires.  SPX_CONV_TMA=0 keeps the per-thread cp.async staging.
    static const int tma_env = [] { const char* v = getenv("SPX_CONV_TMA"); return v ? atoi(v) : 1; }();
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    uint32_t use_tma = 0;
    const PFN_cuTensorMapEncodeTiled encode = tensor_map_encoder();
    if (tma_env && !e->tma_off && encode && e->tma_failed_dev && e->tma_failed_mapped && tp.TWin <= 256 && tp.THin <= 256 &&
        p.B % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
        // two buffers: half the channels of the single-buffer chunk each
        const uint32_t cc = std::min<uint32_t>(std::max<uint32_t>(1u, (uint32_t)(budget / 2 / chanBytes)), std::min<uint32_t>(p.Cin, 256));
        const cuuint64_t gdim[4] = {b_avail, p.W, p.H, p.Cin};    // `in` may point into the batch row (a segment)
        const cuuint64_t gstr[3] = {(cuuint64_t)p.B * 4, (cuuint64_t)p.W * p.B * 4, (cuuint64_t)p.H * p.W * p.B * 4};
        const cuuint32_t box[4] = {tp.BT, tp.TWin, tp.THin, cc};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(in), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
            static const int short_env = [] { const char* v = getenv("SPX_CONV_TMA_TEST_TIMEOUT"); return v ? atoi(v) : 0; }();
            use_tma = short_env ? 3u : 1u;
            tp.CC = cc;
            tp.stage = (uint32_t)((chanBytes * cc + 127) / 128 * 32);     // buffers start on 128-byte boundaries
        }
    }
    const size_t smem = use_tma ? (size_t)tp.stage * (p.Cin > tp.CC ? 2 : 1) * sizeof(float) : chanBytes * tp.CC;
    auto kfn = conv_rbm_tile_kernel<QB, NB, G>;
    cudaError_t err = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return fail(SPX_ERR_CUDA, "conv2d: shared memory opt-in failed: %s", cudaGetErrorString(err));
    kfn<<<ctas, NB * 32, smem, s>>>(e->rbm_hdr, reinterpret_cast<const float4*>(e->rbm_w), e->rbm_ncols, e->rbm_cap,
                                    tp, un, in, bias, act, out, map, use_tma, e->tma_failed_dev, e->tma_failed_mapped);
    SPX_LAUNCH_CHECK("conv_rbm_tile_kernel");
    return SPX_OK;
}

template <int QB>
static int launch_rbm_qb(spx_ell* e, TileParams tp, const float* in, const float* bias, int act, float* out,
                         cudaStream_t s, uint32_t b_base, uint32_t b_len)
{
    // a batch segment [b_base, b_base + b_len): the batch is the innermost dimension of both tensors,
    // so the segment is the same kernel on pointers moved by b_base entries
    in += b_base;
    out += b_base;
    const uint32_t b_avail = tp.c.B - b_base;       // batch entries from the moved pointer to the end of a row
    constexpr int NB = 16;
    const ConvParams& p = tp.c;
    constexpr uint32_t TH = 32u * kRbmG / QB / kTileW;
    const uint32_t THin = (TH - 1) * p.sH + (p.kH - 1) * p.dH + 1, TWin = (kTileW - 1) * p.sW + (p.kW - 1) * p.dW + 1;
    if ((size_t)THin * TWin * QB * 4 * sizeof(float) > 200 * 1024) return -1;
    tp.tilesX = (p.Wo + kTileW - 1) / kTileW;
    const uint64_t tiles = (uint64_t)tp.tilesX * ((p.Ho + TH - 1) / TH);
    const uint32_t nblocks = (p.Cout + kRbmRows - 1) / kRbmRows;
    const uint32_t groups = (nblocks + NB - 1) / NB;
    const uint64_t units = tiles * groups * (b_len / (QB * 4));
    if (units > 0x3fffffffull) return -1;
    const int rc = ensure_rbm(e, p.kH, p.kW, s);
    if (rc != SPX_OK) return rc;                        // -1: no memory for the merged weights
    // One CTA per SM, all units equally long: the launch runs in waves of sm_count units.  A last
    // wave that fills less than half of the SMs is issued as a second launch of half-height tiles
    // (twice the CTAs, each about 0.6 of a full unit's time): 784 units on 148 SMs are 5 full waves
    // + 44 units -> 5 waves + 88 half units.  SPX_CONV_RBM_SPLIT_TAIL=0 keeps one launch.
    static const int split_tail = [] { const char* v = getenv("SPX_CONV_RBM_SPLIT_TAIL"); return v ? atoi(v) : 1; }();
    const uint32_t sms = (uint32_t)sm_count(e->device);
    const uint32_t rem = (uint32_t)(units % sms);
    RbmUnits un{0u, (uint32_t)tiles, groups};
    if (split_tail && units > sms && rem && rem * 2 <= sms) {
        const int rc1 = launch_rbm_units<QB, kRbmG>(e, tp, un, (uint32_t)(units - rem), in, bias, act, out, s, b_avail);
        if (rc1 != SPX_OK) return rc1;
        un.unit0 = (uint32_t)(units - rem);
        return launch_rbm_units<QB, kRbmG / 2>(e, tp, un, rem * 2, in, bias, act, out, s, b_avail);
    }
    return launch_rbm_units<QB, kRbmG>(e, tp, un, (uint32_t)units, in, bias, act, out, s, b_avail);
}

// Row-block-merged path.  Taken whenever K fits the builder's set and the batch is a multiple of 4:
// multiples of 16 on tiles of 16 entries, the rest on a tile of 8 and / or of 4, each segment a
// launch of its own on pointers moved along the (innermost) batch dimension (batch 20 / 24 / 12:
// 1.00 / 1.16 / 0.68 ms against 1.39 / 1.59 / 0.76 ms on the per-row kernel's tiles of 20 / 24 /
// 12).  Measured against conv_pf_tile_kernel on 256 -> 256
// channels, 3 x 3, 56 x 56 (ms, merged vs per-row):
//   batch 32 (tiles of 16; faster than tiles of 32: twice the channels per staged chunk):
//     dense 4.1 vs 7.9, 50 % sparse 2.77 vs 4.15, 80 % 1.69 vs 1.89, 90 % 1.07 vs 1.13,
//     95 % 0.69 vs 0.75, 99 % 0.35 vs 0.44;
//   batch 8: 80 % 0.51 vs 0.57, 90 % 0.33 vs 0.40, 99 % 0.12 vs 0.25;   batch 4: 90 % 0.26 vs 0.37.
// The fewer operand loads pay at high density; at low density the win comes from a CTA covering 64
// output channels per staged chunk instead of 16 or 32.  SPX_CONV_RBM=0 turns the path off;
// SPX_CONV_RBM_MIN_SHARE=x requires an expected 4 d / (1 - (1 - d)^4) >= x rows per union column
// (density d).  Returns -1 when not taken.
static int launch_conv_rbm_tile(spx_ell* e, const ConvParams& p, uint32_t BT, const float* in, const float* bias,
                                int act, float* out, cudaStream_t s)
{
    static const int enabled = [] { const char* v = getenv("SPX_CONV_RBM"); return v ? atoi(v) : 1; }();
    static const double share_env = [] { const char* v = getenv("SPX_CONV_RBM_MIN_SHARE"); return v ? atof(v) : -1.0; }();
    if (e->tma_failed_host && *e->tma_failed_host) {
        // reported once; the handle stages with per-thread copies from here on
        *e->tma_failed_host = 0;
        e->tma_off = true;
        return fail(SPX_ERR_CUDA, "conv2d: a bulk tensor copy of an earlier call on this handle did not complete; its output is invalid");
    }
    // fewer than 8 row blocks would leave most of the CTA's 16 warps without work
    if (!enabled || e->n > kRbmMaxK || e->m < 8 * kRbmRows - 3 || e->max_nnz == 0) return -1;
    (void)BT;
    if (p.B % 4) return -1;
    const double d = (double)e->nnz_total / ((double)e->m * e->n);
    const double share = d >= 1.0 ? (double)kRbmRows : kRbmRows * d / (1.0 - std::pow(1.0 - d, (double)kRbmRows));
    if (share_env >= 0.0 && share < share_env) return -1;
    // The batch in segments: all multiples of 16 on tiles of 16 entries, then a tile of 8 and / or
    // of 4 for the rest, one launch (or two, with the tail split) per segment.  Batch 8 keeps its
    // single tile of 8.  SPX_CONV_RBM_SEGMENTS=0: only batches that are one tile of 4 / 8 or a
    // multiple of 16, the others on the per-row kernel.
    static const int segments = [] { const char* v = getenv("SPX_CONV_RBM_SEGMENTS"); return v ? atoi(v) : 1; }();
    const uint32_t n16 = p.B / 16 * 16, rest = p.B - n16;
    if (!segments && n16 && rest) return -1;
    if (!segments && !n16 && rest == 12) return -1;
    // every segment's staged patch must fit shared memory (checked before any launch)
    const auto fits = [&](uint32_t qb) {
        const uint32_t TH = 32u * kRbmG / qb / kTileW;
        const size_t THin = (size_t)(TH - 1) * p.sH + (size_t)(p.kH - 1) * p.dH + 1;
        const size_t TWin = (size_t)(kTileW - 1) * p.sW + (size_t)(p.kW - 1) * p.dW + 1;
        return THin * TWin * qb * 4 * sizeof(float) <= 200 * 1024;
    };
    if ((n16 && !fits(4)) || (rest >= 8 && !fits(2)) || (rest % 8 == 4 && !fits(1))) return -1;
    TileParams tp{};
    tp.c = p;
    uint32_t at = 0;
    if (n16) {
        const int rc = launch_rbm_qb<4>(e, tp, in, bias, act, out, s, 0, n16);
        if (rc != SPX_OK) return rc;
        at = n16;
    }
    if (rest >= 8) {
        const int rc = launch_rbm_qb<2>(e, tp, in, bias, act, out, s, at, 8);
        if (rc != SPX_OK) return at ? fail(SPX_ERR_CUDA, "conv2d: a batch segment could not be launched") : rc;
        at += 8;
    }
    if (p.B - at == 4) {
        const int rc = launch_rbm_qb<1>(e, tp, in, bias, act, out, s, at, 4);
        if (rc != SPX_OK) return at ? fail(SPX_ERR_CUDA, "conv2d: a batch segment could not be launched") : rc;
    }
    return SPX_OK;
}

// Returns -1 when the shape is not covered (caller falls back to the direct kernel).
static int launch_conv_pf_tile(spx_ell* e, const ConvParams& p, const float* in, const float* bias, int act,
                               float* out, cudaStream_t s)
{
    if (!e->cols_ascending || !pf_tile_covers(p)) return -1;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
    // batch entries per CTA: the largest multiple of 4 that divides B and is <= 32
    uint32_t BT = 0;
    for (uint32_t c = 32; c >= 4; c -= 4) if (p.B % c == 0) { BT = c; break; }
    if (!BT) return -1;
    {
        const int rc = launch_conv_rbm_tile(e, p, BT, in, bias, act, out, s);
        if (rc != -1) return rc;
    }
    static const int ctas = [] { const char* v = getenv("SPX_CONV_CTAS"); return v ? atoi(v) : 0; }();
    static const int small_tile = [] { const char* v = getenv("SPX_CONV_SMALL_TILE"); return v ? atoi(v) : -1; }();
    // Full batch tile (32 entries): 2 x 8 positions per warp and 32 warps (= output channels) per
    // CTA instead of 4 x 8 positions and 16 warps: 64 registers per thread, twice the warps to hide
    // the shared-memory latency, half the staging traffic per output channel.  Measured on
    // 256 -> 256 channels, 56 x 56, batch 32: 1.89 ms against 2.03 ms.  SPX_CONV_SMALL_TILE=0 selects
    // the larger tile.
    const bool small = BT == 32 && small_tile != 0;
    // Batch tile of 8 entries: a 4 x 8 tile would leave a lane two float4 per nonzero, so the warp
    // takes 8 x 8 positions instead and the two broadcast shuffles per nonzero are amortised over 4
    // shared-memory loads (0.571 ms against 0.593 ms on 256 -> 256 channels, 56 x 56, batch 8; a
    // 16 x 8 tile for 4 entries measured slower than 4 x 8).  SPX_CONV_WIDE_TILE=0 turns it off.
    static const int wide_env = [] { const char* v = getenv("SPX_CONV_WIDE_TILE"); return v ? atoi(v) : 1; }();
    const uint32_t QBv = BT / 4;
    const uint32_t Gv = (wide_env && QBv == 2) ? 4 : (small ? 4 : QBv);
    const uint32_t TH = 32 * Gv / QBv / kTileW;
    const uint32_t warps = small ? 32 : kTileWarps;
    TileParams tp{};
    tp.c = p;
    tp.BT = BT;
    tp.THin = (TH - 1) * p.sH + (p.kH - 1) * p.dH + 1;
    tp.TWin = (kTileW - 1) * p.sW + (p.kW - 1) * p.dW + 1;
    const size_t chanBytes = (size_t)tp.THin * tp.TWin * BT * sizeof(float);
    // Two CTAs per SM overlap one CTA's staging with the other's FMAs; with 8 float4 groups per
    // lane (batch 32) the accumulators need more than the 64 registers that allows.
    const int per_sm = small ? 1 : (ctas == 1 || ctas == 2 ? ctas : (BT / 4 > 4 ? 1 : 2));
    const size_t budget = per_sm == 2 ? 100 * 1024 : 200 * 1024;
    if (chanBytes > budget) return -1;
    tp.CC = (uint32_t)std::min<size_t>(p.Cin, budget / chanBytes);
    // the per-nonzero shared-memory offset must fit 32 bits (it does: <= budget / 4)
    tp.tilesX = (p.Wo + kTileW - 1) / kTileW;
    const uint32_t tilesY = (p.Ho + TH - 1) / TH;
    const uint64_t tiles = (uint64_t)tp.tilesX * tilesY;
    const uint32_t gy = (p.Cout + warps - 1) / warps, gz = p.B / BT;
    if (tiles > 0x7fffffffull || gy > 65535 || gz > 65535) return -1;
    dim3 grid((unsigned)tiles, gy, gz);
    const size_t smem = chanBytes * tp.CC;
    if (small) return launch_tile_qb<8, 4, 32, 1>(e, tp, grid, smem, in, bias, act, out, s);
    if (Gv != QBv) return launch_tile_qb<2, 4, kTileWarps, 2>(e, tp, grid, smem, in, bias, act, out, s);
#define SPX_TILE_CASE(Q)                                                                                           \
    case Q: return per_sm == 2 ? launch_tile_qb<Q, Q, kTileWarps, 2>(e, tp, grid, smem, in, bias, act, out, s)     \
                               : launch_tile_qb<Q, Q, kTileWarps, 1>(e, tp, grid, smem, in, bias, act, out, s);
    switch (BT / 4) {
        SPX_TILE_CASE(1) SPX_TILE_CASE(2) SPX_TILE_CASE(3) SPX_TILE_CASE(4)
        SPX_TILE_CASE(5) SPX_TILE_CASE(6) SPX_TILE_CASE(7) SPX_TILE_CASE(8)
    }
#undef SPX_TILE_CASE
    return -1;
}

// Batch size the tiled kernels run at: B rounded up to a multiple of 4, or further up to a multiple
// of 16 when that is cheaper.  Cost per batch entry on 256 -> 256 channels, 3 x 3, 56 x 56, 80 %
// sparse (ms per entry).  Merged kernel, which takes any multiple of 4 in segments of 16 / 8 / 4:
// 0.0436 / 0.0516 / 0.0645 - rounding up to 16 never pays (28 as 16 + 8 + 4: 1.37 ms, as 32 with
// the widening passes: 1.53 ms).  Per-row kernel (matrices the merged one does not take) with its
// tiles of 4 .. 32: 0.094, 0.064, 0.064, 0.056, 0.069, 0.066, 0.068, 0.056 - there 28 runs as 32
// and 44 as 48, while 12, 20, 24 and 36 stay as they are.
static uint32_t padded_batch(uint32_t B, bool merged)
{
    const uint32_t b4 = round_up(B, 4u), b16 = round_up(B, 16u);
    if (b4 == b16 || merged) return b4;
    uint32_t tile = 0;
    for (uint32_t c = 32; c >= 4; c -= 4) if (b4 % c == 0) { tile = c; break; }
    static const double per_entry[9] = {0, 0.094, 0.064, 0.064, 0.056, 0.069, 0.066, 0.068, 0.056};
    const double as_is = b4 * per_entry[tile / 4], widened = b16 * 0.056 * 1.03;
    return widened < as_is ? b16 : b4;
}

// Whether launch_conv_rbm_tile will take this handle (the part of its test that does not depend on
// the geometry): the merged kernel is on, K fits its builder, and there are at least 8 row blocks.
static bool merged_kernel_takes(const spx_ell* e)
{
    static const int enabled = [] { const char* v = getenv("SPX_CONV_RBM"); return v ? atoi(v) : 1; }();
    static const int segments = [] { const char* v = getenv("SPX_CONV_RBM_SEGMENTS"); return v ? atoi(v) : 1; }();
    static const bool share_set = getenv("SPX_CONV_RBM_MIN_SHARE") != nullptr;
    return enabled && segments && !share_set && e->cols_ascending && e->n <= kRbmMaxK && e->m >= 8 * kRbmRows - 3 && e->max_nnz != 0;
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
    // The tiled kernels want [C,H,W,B] with B a multiple of 4.  Other inputs are brought into that
    // form in per-handle scratch and the result is converted back:
    //   NCHW (B > 1; one NCHW image already is [C,H,W,1]): transpose in, transpose out - two extra
    //     streaming passes over input and output (about 5 % of the kernel's time at 256 channels);
    //   B not a multiple of 4 (or cheaper at the next multiple of 16, see padded_batch): the batch
    //     dimension is widened with zero entries and narrowed again
    //     (256 -> 256 channels, 56 x 56: batch 3 takes 0.4 ms this way against 1.2 ms with the general
    //     kernel, batch 1 0.4 against 0.43 ms).
    // Arithmetic per output element is unchanged in both cases.
    const uint32_t B4 = padded_batch(B, merged_kernel_takes(e));
    ConvParams p4 = p;
    p4.B = B4;
    // F-major tensors, b + B*(c + C*(h + H*w)): [W,H,C,B] is [C,H,W,B] with the three outer
    // dimensions reversed, so the tiled kernels are reached through two more streaming passes
    // (reverse in, reverse out) in scratch of their own; shapes the tiled kernels do not cover
    // gather straight from the F-major tensor in the general kernel below.
    if (layout == SPX_LAYOUT_FMAJOR && e->r && e->cols_ascending && pf_tile_covers(p4)) {
        const uint64_t n_in = (uint64_t)g->Cin * g->H * g->W * B, n_out = (uint64_t)g->Cout * g->Ho * g->Wo * B;
        const uint64_t in_slab = (n_in + 63) / 64 * 64;
        const size_t need = (size_t)(in_slab + n_out) * sizeof(float);
        if (e->fm_scratch_bytes < need) {
            if (e->fm_scratch) cudaFree(e->fm_scratch);
            e->fm_scratch = nullptr;
            e->fm_scratch_bytes = 0;
            SPX_CUDA(cudaMalloc(&e->fm_scratch, need));
            e->fm_scratch_bytes = need;
        }
        float* in_pf = static_cast<float*>(e->fm_scratch);
        float* out_pf = in_pf + in_slab;
        auto reverse3 = [&](const float* src, uint32_t D0, uint32_t D1, uint32_t D2, float* dst, uint64_t total) {
            const unsigned blocks = (unsigned)std::min<uint64_t>((total + 255) / 256, (uint64_t)sm_count(e->device) * 32);
            reverse3_kernel<<<blocks, 256, 0, s>>>(src, D0, D1, D2, B, dst);
            SPX_LAUNCH_CHECK("reverse3_kernel");
            return SPX_OK;
        };
        rc = reverse3(in, g->W, g->H, g->Cin, in_pf, n_in);                   // [W,H,C,B] -> [C,H,W,B]
        if (rc != SPX_OK) return rc;
        rc = launch_conv2d(e, g, SPX_LAYOUT_PF, in_pf, B, bias, act, out_pf, s);
        if (rc != SPX_OK) return rc;
        return reverse3(out_pf, g->Cout, g->Ho, g->Wo, out, n_out);           // [C,Ho,Wo,B] -> [Wo,Ho,C,B]
    }
    if (layout != SPX_LAYOUT_FMAJOR && e->r && e->cols_ascending && pf_tile_covers(p4)) {
        const bool nchw = layout == SPX_LAYOUT_NCHW && B > 1;
        const bool pad = B4 != B;
        if (!nchw && !pad) {
            rc = launch_conv_pf_tile(e, p, in, bias, act, out, s);
            if (rc != -1) return rc;             // -1: shape not covered by the tiled kernels
        } else {
            const uint64_t in_rows = (uint64_t)g->Cin * g->H * g->W, out_rows = (uint64_t)g->Cout * g->Ho * g->Wo;
            auto slab = [](uint64_t floats) { return (floats + 63) / 64 * 64; };
            const uint64_t n_in4 = slab(in_rows * B4), n_out4 = slab(out_rows * B4);
            const uint64_t n_in = (nchw && pad) ? slab(in_rows * B) : 0, n_out = (nchw && pad) ? slab(out_rows * B) : 0;
            const size_t need = (size_t)(n_in4 + n_out4 + n_in + n_out) * sizeof(float);
            if (e->conv_scratch_bytes < need) {
                if (e->conv_scratch) cudaFree(e->conv_scratch);
                e->conv_scratch = nullptr;
                e->conv_scratch_bytes = 0;
                SPX_CUDA(cudaMalloc(&e->conv_scratch, need));
                e->conv_scratch_bytes = need;
            }
            float* in4 = static_cast<float*>(e->conv_scratch);
            float* out4 = in4 + n_in4;
            float* in_t = out4 + n_out4;          // [C,H,W,B] before widening (NCHW and widening only)
            float* out_t = in_t + n_in;
            auto repitch = [&](const float* src, uint32_t sp, uint32_t sc, float* dst, uint32_t dp, uint32_t dc, uint64_t rows) {
                const uint64_t total = rows * dc;
                const unsigned blocks = (unsigned)std::min<uint64_t>((total + 255) / 256, (uint64_t)sm_count(e->device) * 32);
                repitch_kernel<<<blocks, 256, 0, s>>>(src, sp, sc, dst, dp, dc, rows);
                SPX_LAUNCH_CHECK("repitch_kernel");
                return SPX_OK;
            };
            const float* src_pf = in;
            if (nchw) {
                rc = transpose2d(in, B, in_rows, pad ? in_t : in4, s);
                if (rc != SPX_OK) return rc;
                src_pf = in_t;
            }
            if (pad) {
                rc = repitch(src_pf, B, B, in4, B4, B4, in_rows);
                if (rc != SPX_OK) return rc;
            }
            rc = launch_conv_pf_tile(e, p4, in4, bias, act, out4, s);
            if (rc == SPX_OK) {
                if (!pad) return transpose2d(out4, out_rows, B, out, s);
                rc = repitch(out4, B4, B, nchw ? out_t : out, B, B, out_rows);
                if (rc != SPX_OK || !nchw) return rc;
                return transpose2d(out_t, out_rows, B, out, s);
            }
            if (rc != -1) return rc;
        }
    }
    const uint64_t per_m = (uint64_t)g->Ho * g->Wo * B;
    const uint64_t gx = (per_m + 255) / 256;
    if (gx > 0x7fffffffull || e->m > 65535)
        return fail(SPX_ERR_LIMIT, "conv2d: output too large for one launch");
    dim3 grid((unsigned)gx, e->m);
    if (layout == SPX_LAYOUT_PF)
        conv_direct_kernel<SPX_LAYOUT_PF><<<grid, 256, 0, s>>>(e->Wd, e->taps, e->nnz, e->pitch, p, in, bias, act, out);
    else if (layout == SPX_LAYOUT_FMAJOR)
        conv_direct_kernel<SPX_LAYOUT_FMAJOR><<<grid, 256, 0, s>>>(e->Wd, e->taps, e->nnz, e->pitch, p, in, bias, act, out);
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

    // every limit is checked before the first launch: a refused call leaves the shared table alone
    const uint64_t per_m = (uint64_t)g->Ho * g->Wo * B;
    const uint64_t gx = (per_m + 255) / 256;
    if (gx > 0x7fffffffull || e->m > 65535) return fail(SPX_ERR_LIMIT, "conv2d_static: output too large for one launch");
    cudaStream_t s = (cudaStream_t)stream;
    if (e->r) {
        build_taps_kernel<<<e->m, 128, 0, s>>>(e->idx, e->nnz, e->m, e->pitch, g->kH, g->kW, taps);
        SPX_LAUNCH_CHECK("build_taps_kernel");
    }
    ConvParams p{g->Cin, g->Cout, g->kH, g->kW, g->sH, g->sW, g->pH, g->pW, g->dH, g->dW, g->H, g->W, g->Ho, g->Wo, B};
    dim3 grid((unsigned)gx, e->m);
    if (layout == SPX_LAYOUT_PF)
        conv_direct_kernel<SPX_LAYOUT_PF><<<grid, 256, 0, s>>>(e->Wd, taps, e->nnz, e->pitch, p, in, bias, act, out);
    else
        conv_direct_kernel<SPX_LAYOUT_NCHW><<<grid, 256, 0, s>>>(e->Wd, taps, e->nnz, e->pitch, p, in, bias, act, out);
    SPX_LAUNCH_CHECK("conv_direct_kernel");
    return SPX_OK;
}
