// spmm.cu -- ELLPACK SpMM  Y = act(bias + E * X)  for sm_100a.
//
// Replaces ellpack_matmul_fused<USE_MASK,FUSE_RELU> of the reference
// (src/ellpack_matmul.cpp:11-92).  Arithmetic contract kept from the reference: every output
// element starts from bias[i] (or 0) and receives ONE fused multiply-add per stored nonzero
// of row i, in storage order (:56-66); the activation follows (:68-70).  A thread owns whole
// output elements, so the result is bit-identical to the reference for every C, and no
// padding slot is ever multiplied.
//
// Kernel: spmm_gather -- warp per row, lanes across dense columns, X rows gathered through L1/L2.
// Column panels are the slow grid dimension so that all CTAs in flight work on the same X panel.
// Rows are taken from the handle's sorted row schedule (longest first), so the warps of a CTA
// and the CTAs of a wave carry equal work.  Because every row walks its column ids in ascending
// order, the warps resident on an SM sweep X roughly in step and share its rows through L1
// (56 % L1 hit rate measured on a 4096 x 4096, 10 % dense matrix) -- staging X in shared memory
// block by block was tried and was slower (staging, barriers and predicated tails cost more than
// the L1 misses they removed).
#include "common.cuh"

#include <algorithm>
#include <cstdlib>

namespace {

constexpr int kGatherWarps = 8;
constexpr int kMaxPeers = 8;

// Linear block id -> (row block, column panel).  Normally panel-major: all row blocks of panel 0,
// then panel 1, ... so that the CTAs in flight share one panel of X in L2.  The first `head` row
// blocks (the longest rows of the sorted schedule) can instead be issued first, for all panels:
// a long row is one dependent chain of gathers, and when the whole kernel is only a few such chains
// long, a chain that starts with the last panel would end well after everything else.
struct BlockMap {
    uint32_t blocks;      // grid size
    uint32_t row_blocks;  // CTAs per panel
    uint32_t panels;
    uint32_t head;        // row blocks issued first, panel-minor
};

__device__ __forceinline__ void decode_block(const BlockMap& bm, uint32_t b, uint32_t& rb, uint32_t& panel) {
    const uint32_t head_blocks = bm.head * bm.panels;
    if (b < head_blocks) {
        rb = b / bm.panels;
        panel = b % bm.panels;
    } else {
        const uint32_t t = b - head_blocks, rest = bm.row_blocks - bm.head;
        panel = t / rest;
        rb = bm.head + t % rest;
    }
}

// Destinations of the epilogue.  Plain SpMM: one pointer (this GPU's Y).  Row-sharded SpMM with
// the all-gather fused in: the full Y buffer of every rank (this GPU's own and its peers' buffers
// mapped over NVLink); each finished output vector is stored to all of them with ordinary 16-byte
// stores, so the exchange overlaps the multiply instead of following it.
struct PeerOut {
    float* p[kMaxPeers];
    int n;
    int mcast;          // p[0] is an NVLink multicast address: one multimem.st reaches every rank's buffer
    uint64_t row0;      // first row of this rank's slab inside the full buffers
};

// One finished vector to every destination.  Peer list: one ordinary 16-byte store per buffer (the
// GPU sends the vector once per peer).  Multicast address: a single multimem.st, replicated to all
// bound GPUs (this one included) by the NVSwitch, so the vector leaves this GPU once.
__device__ __forceinline__ void store_out(const PeerOut& out, size_t at, const float4& o) {
    if (out.mcast) {
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(out.p[0] + at), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
        return;
    }
#pragma unroll
    for (int g = 0; g < kMaxPeers; ++g)
        if (g < out.n) *reinterpret_cast<float4*>(out.p[g] + at) = o;
}
__device__ __forceinline__ void store_out(const PeerOut& out, size_t at, float o) {
    if (out.mcast) {
        asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(out.p[0] + at), "f"(o) : "memory");
        return;
    }
#pragma unroll
    for (int g = 0; g < kMaxPeers; ++g)
        if (g < out.n) out.p[g][at] = o;
}

__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

__device__ __forceinline__ void fma4(float4& a, float w, const float4& x) {
    a.x = fmaf(w, x.x, a.x);
    a.y = fmaf(w, x.y, a.y);
    a.z = fmaf(w, x.z, a.z);
    a.w = fmaf(w, x.w, a.w);
}

// ---------------------------------------------------------------------------------------
// spmm_gather<NV>: lane owns NV float4 groups: columns c0 + v*128 + 4*lane .. +3.
// ---------------------------------------------------------------------------------------
template <int NV, int G, int MINB>
__global__ void __launch_bounds__(kGatherWarps * 32, MINB)
spmm_gather_vec(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                uint32_t m, uint32_t pitch,
                const float* __restrict__ X, uint32_t C, uint64_t ldx,
                const float* __restrict__ bias, int act, PeerOut out, uint64_t ldy, BlockMap bm)
{
    const int lane = threadIdx.x & 31;
    uint32_t rb, panel;
    decode_block(bm, blockIdx.x, rb, panel);
    const uint32_t slot = rb * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (slot >= m) return;                      // whole warp leaves together
    const uint32_t row = __ldg(row_order + slot);   // rows by descending length: equal work per CTA
    const uint32_t c0 = panel * (128u * NV) + 4u * lane;
    bool on[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) on[v] = (c0 + 128u * v) < C;   // C % 4 == 0 on this path

    const float b = bias ? __ldg(bias + row) : 0.0f;
    float4 acc[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[v] = make_float4(b, b, b, b);

    const uint32_t nn = __ldg(nnz + row);
    const float* __restrict__ w = Wd + (size_t)row * pitch;
    const uint32_t* __restrict__ k = idx + (size_t)row * pitch;

    for (uint32_t j0 = 0; j0 < nn; j0 += 32) {
        float wl = 0.0f;
        uint32_t kl = 0;
        if (j0 + lane < nn) {                   // coalesced 128-byte slab reads
            wl = __ldg(w + j0 + lane);
            kl = __ldg(k + j0 + lane);
        }
        const uint32_t cnt = min(32u, nn - j0);
        for (uint32_t t0 = 0; t0 < cnt; t0 += G) {
            float wt[G];
            float4 xv[G][NV];
#pragma unroll
            for (int u = 0; u < G; ++u) {       // issue all gathers of the group first
                wt[u] = __shfl_sync(0xffffffffu, wl, (t0 + u) & 31);
                const uint32_t kt = __shfl_sync(0xffffffffu, kl, (t0 + u) & 31);
                const float* xr = X + (size_t)kt * ldx + c0;
                const bool live = (t0 + u) < cnt;
#pragma unroll
                for (int v = 0; v < NV; ++v)
                    xv[u][v] = (live && on[v]) ? ldg4(xr + 128 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < G; ++u) {       // then the FMA chain, strictly in storage order
                if ((t0 + u) < cnt) {
#pragma unroll
                    for (int v = 0; v < NV; ++v) fma4(acc[v], wt[u], xv[u][v]);
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        if (on[v]) {
            float4 o = acc[v];
            if (act != SPX_ACT_NONE) {
                o.x = spx::apply_act(o.x, act); o.y = spx::apply_act(o.y, act);
                o.z = spx::apply_act(o.z, act); o.w = spx::apply_act(o.w, act);
            }
            const size_t at = (size_t)(out.row0 + row) * ldy + c0 + 128 * v;
            store_out(out, at, o);
        }
    }
}

// ---------------------------------------------------------------------------------------
// spmm_gather_staged: the kernel for matrices whose longest rows decide the duration (few rows
// per GPU, skewed lengths: a row shard of a power-law matrix).  Same chain per output element
// as spmm_gather_vec.  Differences: (1) the first `head` row blocks of the schedule -- the rows
// with 512 and more stored entries -- are issued first, for all their panels, and run on
// 128-column panels with eight rows of X in flight per round trip; all other row blocks follow
// panel-major on 256-column panels with four.  (2) A row's (w, idx) slab travels 32 entries at a
// time, one batch ahead, through a double-buffered 256-byte staging area of the warp in shared
// memory (cp.async) and is handed to the lanes with 16-byte broadcast loads, one per four
// entries, instead of two shuffles per entry: the chain of a long row no longer waits for slab
// reads.  (3) Loads and FMAs carry the predicate "entry exists"; nothing is zero-filled.
// ---------------------------------------------------------------------------------------
struct StagedMap {
    uint32_t blocks;        // grid size
    uint32_t row_blocks;    // row blocks (one row per warp)
    uint32_t head;          // row blocks on the narrow path, issued first, panel-minor
    uint32_t head_panels;   // 128-column panels
    uint32_t panels;        // panels of the other row blocks: 256 columns, or 128 when all_narrow
    uint32_t all_narrow;    // every row on 128-column panels (panel-major, so one 128-column panel of X is in use at a time)
    uint32_t rest_ascending;    // the rows behind the head run shortest first (see launch_spmm_bcast)
};

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One row on one panel of 128 * NV columns, G rows of X per round trip; the lane owns columns
// c0 + 128 * v + 0..3.
template <int NV, int G>
__device__ __forceinline__ void staged_row(const float* __restrict__ w, const uint32_t* __restrict__ k, uint32_t nn,
                                           const float* __restrict__ X, uint32_t c0, uint32_t C, uint32_t ldxb, float b, int act,
                                           const PeerOut& out, size_t out_at, float* sw, uint32_t* sk, int lane)
{
    static_assert(G % 4 == 0 && 32 % G == 0, "groups are made of 16-byte quads");
    bool on[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) on[v] = (c0 + 128u * v) < C;   // C % 4 == 0 on this path
    float4 acc[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[v] = make_float4(b, b, b, b);
    const char* xbase = reinterpret_cast<const char*>(X + c0);

    if ((uint32_t)lane < nn) {
        cp_async4(sw + lane, w + lane);
        cp_async4(sk + lane, k + lane);
    }
    cp_async_commit();
    const uint32_t batches = (nn + 31) >> 5;
    for (uint32_t bt = 0; bt < batches; ++bt) {
        const float* bw = sw + (bt & 1) * 32;
        const uint32_t* bk = sk + (bt & 1) * 32;
        cp_async_wait_all();
        __syncwarp();       // batch bt has landed for all lanes; the other buffer is no longer read
        const uint32_t jn = (bt + 1) * 32 + lane;
        if (jn < nn) {      // next batch in flight while this one is multiplied
            cp_async4(sw + ((bt + 1) & 1) * 32 + lane, w + jn);
            cp_async4(sk + ((bt + 1) & 1) * 32 + lane, k + jn);
        }
        cp_async_commit();
        const uint32_t cnt = min(32u, nn - bt * 32);
        for (uint32_t t = 0; t < cnt; t += G) {
            float wt[G];
            uint32_t kt[G];
#pragma unroll
            for (int q = 0; q < G / 4; ++q) {
                const float4 w4 = *reinterpret_cast<const float4*>(bw + t + 4 * q);
                const uint4 k4 = *reinterpret_cast<const uint4*>(bk + t + 4 * q);
                wt[4 * q] = w4.x; wt[4 * q + 1] = w4.y; wt[4 * q + 2] = w4.z; wt[4 * q + 3] = w4.w;
                kt[4 * q] = k4.x; kt[4 * q + 1] = k4.y; kt[4 * q + 2] = k4.z; kt[4 * q + 3] = k4.w;
            }
            const uint32_t left = cnt - t;
            float4 xv[G][NV];
#pragma unroll
            for (int u = 0; u < G; ++u) {       // issue all gathers of the group first
                if ((uint32_t)u < left) {
                    const char* xr = xbase + (size_t)kt[u] * ldxb;
#pragma unroll
                    for (int v = 0; v < NV; ++v)
                        if (on[v]) xv[u][v] = __ldg(reinterpret_cast<const float4*>(xr + 512 * v));
                }
            }
#pragma unroll
            for (int u = 0; u < G; ++u) {       // then the FMA chain, strictly in storage order
                if ((uint32_t)u < left) {
#pragma unroll
                    for (int v = 0; v < NV; ++v)
                        if (on[v]) fma4(acc[v], wt[u], xv[u][v]);
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        if (on[v]) {
            float4 o = acc[v];
            if (act != SPX_ACT_NONE) {
                o.x = spx::apply_act(o.x, act); o.y = spx::apply_act(o.y, act);
                o.z = spx::apply_act(o.z, act); o.w = spx::apply_act(o.w, act);
            }
            const size_t at = out_at + 128 * v;
            store_out(out, at, o);
        }
    }
}

__global__ void __launch_bounds__(kGatherWarps * 32, 4)
spmm_gather_staged(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                   const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                   uint32_t m, uint32_t pitch,
                   const float* __restrict__ X, uint32_t C, uint32_t ldxb,
                   const float* __restrict__ bias, int act, PeerOut out, uint64_t ldy, StagedMap sm)
{
    extern __shared__ __align__(16) float s_stage[];           // per warp: 64 weights, then 64 column ids
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* s_w = s_stage + warp * 128;
    uint32_t* s_k = reinterpret_cast<uint32_t*>(s_w + 64);
    const uint32_t head_blocks = sm.head * sm.head_panels;
    const bool narrow = blockIdx.x < head_blocks;
    uint32_t rb, panel;
    if (narrow) {
        rb = blockIdx.x / sm.head_panels;
        panel = blockIdx.x % sm.head_panels;
    } else {
        const uint32_t t = blockIdx.x - head_blocks, rest = sm.row_blocks - sm.head;
        panel = t / rest;
        rb = sm.head + t % rest;
    }
    uint32_t slot = rb * (blockDim.x >> 5) + warp;
    if (slot >= m) return;                      // whole warp leaves together
    if (!narrow && sm.rest_ascending) {
        const uint32_t first = sm.head * (blockDim.x >> 5);      // schedule slots [first, m) in reverse
        slot = first + (m - 1 - slot);
    }
    const uint32_t row = __ldg(row_order + slot);
    const float b = bias ? __ldg(bias + row) : 0.0f;
    const uint32_t nn = __ldg(nnz + row);
    const float* __restrict__ w = Wd + (size_t)row * pitch;
    const uint32_t* __restrict__ k = idx + (size_t)row * pitch;
    const size_t out_row = (size_t)(out.row0 + row) * ldy;
    if (narrow || sm.all_narrow) {
        const uint32_t c0 = panel * 128u + 4u * lane;
        staged_row<1, 8>(w, k, nn, X, c0, C, ldxb, b, act, out, out_row + c0, s_w, s_k, lane);
    } else {
        const uint32_t c0 = panel * 256u + 4u * lane;
        staged_row<2, 4>(w, k, nn, X, c0, C, ldxb, b, act, out, out_row + c0, s_w, s_k, lane);
    }
}

// ---------------------------------------------------------------------------------------
// spmm_gather_sub<LPR>: narrow X (C <= 4*LPR, LPR = 8 or 16).  A full warp per row would leave
// most lanes idle, so LPR lanes share a row and a warp carries 32/LPR rows of the sorted schedule
// (neighbours there have near-equal lengths).  Same chain per output element as spmm_gather_vec.
// ---------------------------------------------------------------------------------------
template <int LPR, int BM, int MINB>   // BM: entries loaded per lane and batch (LPR*BM gathers in flight per row)
__global__ void __launch_bounds__(kGatherWarps * 32, MINB)
spmm_gather_sub(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                uint32_t m, uint32_t pitch,
                const float* __restrict__ X, uint32_t C, uint64_t ldx,
                const float* __restrict__ bias, int act, PeerOut out, uint64_t ldy, bool prefetch_slabs)
{
    constexpr int RPW = 32 / LPR;
    const int lane = threadIdx.x & 31;
    const int sl = lane % LPR;
    const uint32_t slot = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + lane / LPR;
    const bool live = slot < m;
    const uint32_t row = live ? __ldg(row_order + slot) : 0u;
    const uint32_t c0 = 4u * sl;
    const bool on = live && c0 < C;

    const float b = (live && bias) ? __ldg(bias + row) : 0.0f;
    float4 acc = make_float4(b, b, b, b);
    const uint32_t nn = live ? __ldg(nnz + row) : 0u;
    const uint32_t nmax = __reduce_max_sync(0xffffffffu, nn);       // the warp runs to its longest row
    const float* __restrict__ w = Wd + (size_t)row * pitch;
    const uint32_t* __restrict__ k = idx + (size_t)row * pitch;

    constexpr int NB = LPR * BM;
    // (w, idx) of the next batch are fetched while this batch's gathers are in flight, so a batch
    // costs one memory round trip, not two (the kernel is bound by this per-row chain).
    float wn[BM];
    uint32_t kn[BM];
    auto fetch = [&](uint32_t j) {
#pragma unroll
        for (int h = 0; h < BM; ++h) {
            wn[h] = 0.0f;
            kn[h] = 0;
            if (j + h * LPR + sl < nn) {
                wn[h] = __ldg(w + j + h * LPR + sl);
                kn[h] = __ldg(k + j + h * LPR + sl);
            }
        }
    };
    fetch(0);
    // The row's slabs are touched 32 entries at a time, one DRAM round trip each when they are not
    // in L2 yet: ask for all of the row's lines now so that the later batches find them in L2.
    // Only when the whole matrix fits L2 with room to spare (the caller decides): otherwise the
    // lines would be evicted again before their batch comes up.
    if (prefetch_slabs) {
        for (uint32_t j = NB + sl * 32; j < nn; j += LPR * 32) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(w + j));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(k + j));
        }
    }
    for (uint32_t j0 = 0; j0 < nmax; j0 += NB) {
        float wl[BM];
        uint32_t kl[BM];
#pragma unroll
        for (int h = 0; h < BM; ++h) { wl[h] = wn[h]; kl[h] = kn[h]; }
        if (j0 + NB < nmax) fetch(j0 + NB);
        const uint32_t cnt = j0 < nn ? min((uint32_t)NB, nn - j0) : 0u;      // entries of this lane's row in the batch
        float wt[NB];
        float4 xv[NB];
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            wt[u] = __shfl_sync(0xffffffffu, wl[u / LPR], u % LPR, LPR);
            const uint32_t kt = __shfl_sync(0xffffffffu, kl[u / LPR], u % LPR, LPR);
            xv[u] = (on && (uint32_t)u < cnt) ? ldg4(X + (size_t)kt * ldx + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < NB; ++u)
            if ((uint32_t)u < cnt) fma4(acc, wt[u], xv[u]);
    }
    if (on) {
        float4 o = acc;
        if (act != SPX_ACT_NONE) {
            o.x = spx::apply_act(o.x, act); o.y = spx::apply_act(o.y, act);
            o.z = spx::apply_act(o.z, act); o.w = spx::apply_act(o.w, act);
        }
        const size_t at = (size_t)(out.row0 + row) * ldy + c0;
        store_out(out, at, o);
    }
}

// ---------------------------------------------------------------------------------------
// spmm_gather_half: 64 < C <= 128.  With a full warp per row a lane would own one float4 and the
// per-entry work that does not scale with the width (two shuffles, the row address, the loop)
// would be spread over 4 FMAs; here 16 lanes share a row and own two float4 each, a warp carries
// two neighbouring rows of the sorted schedule, and every shuffle / address / load instruction
// serves both rows, as in spmm_gather_vec<2> at C = 256.  Same chain per output element.
// ---------------------------------------------------------------------------------------
template <int G, int MINB>
__global__ void __launch_bounds__(kGatherWarps * 32, MINB)
spmm_gather_half(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                 const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                 uint32_t m, uint32_t pitch,
                 const float* __restrict__ X, uint32_t C, uint64_t ldx,
                 const float* __restrict__ bias, int act, PeerOut out, uint64_t ldy)
{
    const int lane = threadIdx.x & 31;
    const int sl = lane & 15;
    const uint32_t slot = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
    const bool live = slot < m;
    const uint32_t row = live ? __ldg(row_order + slot) : 0u;
    const uint32_t c0 = 4u * sl;
    bool on[2];
#pragma unroll
    for (int v = 0; v < 2; ++v) on[v] = live && (c0 + 64u * v) < C;

    const float b = (live && bias) ? __ldg(bias + row) : 0.0f;
    float4 acc[2];
#pragma unroll
    for (int v = 0; v < 2; ++v) acc[v] = make_float4(b, b, b, b);
    const uint32_t nn = live ? __ldg(nnz + row) : 0u;
    const uint32_t nmax = __reduce_max_sync(0xffffffffu, nn);       // the warp runs to its longer row
    const float* __restrict__ w = Wd + (size_t)row * pitch;
    const uint32_t* __restrict__ k = idx + (size_t)row * pitch;

    for (uint32_t j0 = 0; j0 < nmax; j0 += 16) {
        float wl = 0.0f;
        uint32_t kl = 0;
        if (j0 + sl < nn) {                     // 64-byte slab reads per half warp
            wl = __ldg(w + j0 + sl);
            kl = __ldg(k + j0 + sl);
        }
        const uint32_t cnt = j0 < nn ? min(16u, nn - j0) : 0u;      // entries of this lane's row in the batch
        const uint32_t cmax = min(16u, nmax - j0);
        for (uint32_t t0 = 0; t0 < cmax; t0 += G) {
            float wt[G];
            float4 xv[G][2];
#pragma unroll
            for (int u = 0; u < G; ++u) {
                wt[u] = __shfl_sync(0xffffffffu, wl, (t0 + u) & 15, 16);
                const uint32_t kt = __shfl_sync(0xffffffffu, kl, (t0 + u) & 15, 16);
                const float* xr = X + (size_t)kt * ldx + c0;
                const bool have = (t0 + u) < cnt;
#pragma unroll
                for (int v = 0; v < 2; ++v)
                    xv[u][v] = (have && on[v]) ? ldg4(xr + 64 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < G; ++u) {
                if ((t0 + u) < cnt) {
#pragma unroll
                    for (int v = 0; v < 2; ++v) fma4(acc[v], wt[u], xv[u][v]);
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < 2; ++v) {
        if (on[v]) {
            float4 o = acc[v];
            if (act != SPX_ACT_NONE) {
                o.x = spx::apply_act(o.x, act); o.y = spx::apply_act(o.y, act);
                o.z = spx::apply_act(o.z, act); o.w = spx::apply_act(o.w, act);
            }
            const size_t at = (size_t)(out.row0 + row) * ldy + c0 + 64 * v;
            store_out(out, at, o);
        }
    }
}

// Scalar variant for C % 4 != 0 or unaligned operands: lane owns columns c0 + 32*v + lane.
template <int NV>
__global__ void __launch_bounds__(kGatherWarps * 32)
spmm_gather_scalar(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                   const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                   uint32_t m, uint32_t pitch,
                   const float* __restrict__ X, uint32_t C, uint64_t ldx,
                   const float* __restrict__ bias, int act, PeerOut out, uint64_t ldy, BlockMap bm)
{
    const int lane = threadIdx.x & 31;
    uint32_t rb, panel;
    decode_block(bm, blockIdx.x, rb, panel);
    const uint32_t slot = rb * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (slot >= m) return;
    const uint32_t row = __ldg(row_order + slot);
    const uint32_t c0 = panel * (32u * NV) + lane;
    bool on[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) on[v] = (c0 + 32u * v) < C;

    const float b = bias ? __ldg(bias + row) : 0.0f;
    float acc[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[v] = b;

    const uint32_t nn = __ldg(nnz + row);
    const float* __restrict__ w = Wd + (size_t)row * pitch;
    const uint32_t* __restrict__ k = idx + (size_t)row * pitch;

    for (uint32_t j0 = 0; j0 < nn; j0 += 32) {
        float wl = 0.0f;
        uint32_t kl = 0;
        if (j0 + lane < nn) {
            wl = __ldg(w + j0 + lane);
            kl = __ldg(k + j0 + lane);
        }
        const uint32_t cnt = min(32u, nn - j0);
        for (uint32_t t0 = 0; t0 < cnt; t0 += 8) {
            float wt[8];
            float xv[8][NV];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                wt[u] = __shfl_sync(0xffffffffu, wl, (t0 + u) & 31);
                const uint32_t kt = __shfl_sync(0xffffffffu, kl, (t0 + u) & 31);
                const float* xr = X + (size_t)kt * ldx + c0;
                const bool live = (t0 + u) < cnt;
#pragma unroll
                for (int v = 0; v < NV; ++v) xv[u][v] = (live && on[v]) ? __ldg(xr + 32 * v) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if ((t0 + u) < cnt) {
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[v] = fmaf(wt[u], xv[u][v], acc[v]);
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < NV; ++v)
        if (on[v]) {
            const float o = spx::apply_act(acc[v], act);
            const size_t at = (size_t)(out.row0 + row) * ldy + c0 + 32 * v;
            store_out(out, at, o);
        }
}

}  // namespace

namespace spx {

// Column-panel width of the gather kernel.  All CTAs in flight work on one panel of X
// (n rows x 128*NV columns); it must stay L2-resident while every row of E gathers from it.
// SPX_SPMM_NV=1|2 overrides the choice (tuning knob).
static int gather_nv(uint32_t n, uint32_t C)
{
    static const int forced = [] { const char* v = getenv("SPX_SPMM_NV"); return v ? atoi(v) : 0; }();
    if (forced == 1 || forced == 2) return C > 128 ? forced : 1;
    (void)n;
    // Measured on B200 (262144 x 65536, C = 1024): 256-column panels beat 128-column ones
    // (4.5 ms against 5.4 ms) even though the 67 MB panel no longer fits the near L2 partition:
    // the (w, idx) broadcast is amortised over twice the columns.
    return C > 128 ? 2 : 1;
}

// Warps (= rows) per CTA.  Large problems use 8; small ones use fewer so that the grid still has
// several CTAs per SM and the last wave is not mostly empty (a 4096-row matrix with 8 rows per CTA
// left the SMs idle 40 % of the kernel's duration).
static uint32_t gather_wpb(const spx_ell* e, uint32_t panels)
{
    static const int forced = [] { const char* v = getenv("SPX_SPMM_WPB"); return v ? atoi(v) : 0; }();
    if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return (uint32_t)forced;
    const uint64_t want = (uint64_t)sm_count(e->device) * 8;
    for (uint32_t wpb : {8u, 4u, 2u})
        if ((uint64_t)((e->m + wpb - 1) / wpb) * panels >= want) return wpb;
    return 2;
}

// Grid layout (see BlockMap).  Rows with at least 512 stored entries go first for all panels.
// Measured on B200 with power-law rows (mean 64, max 2048), n = 65536, C = 1024: 32768 rows
// 0.75 -> 0.61 ms, 65536 rows 1.11 -> 1.01 ms, 262144 rows unchanged (3.9 ms), so it is always on.
static BlockMap block_map(const spx_ell* e, uint32_t C, uint32_t panels, uint32_t wpb)
{
    static const int forced = [] { const char* v = getenv("SPX_SPMM_HEAD"); return v ? atoi(v) : -1; }();
    BlockMap bm{};
    bm.row_blocks = (e->m + wpb - 1) / wpb;
    bm.panels = panels;
    bm.blocks = bm.row_blocks * panels;
    (void)C;
    const bool head = forced != 0 && panels > 1 && e->long_rows > 0;
    bm.head = head ? std::min<uint32_t>(bm.row_blocks, (e->long_rows + wpb - 1) / wpb) : 0;
    return bm;
}

// Whether the longest row's chain of gathers decides the kernel's duration (see
// spmm_gather_staged).  Estimates: the kernel moves 4*C bytes of X per stored entry at about
// 17 TB/s; the longest row's chain takes max_nnz / 4 round trips of about 1.2 us on the wide path.
// Measured on B200 (power-law rows, mean 64, max 2048, n = 65536, C = 1024), staged kernel against
// spmm_gather_vec: 32768 rows 0.556 against 0.610 ms, 65536 rows 1.00 against 1.00 ms, 262144 rows
// 4.21 against 4.09 ms.  SPX_SPMM_STAGED=0|1 overrides.
static int staged_mode()
{
    static const int forced = [] { const char* v = getenv("SPX_SPMM_STAGED"); return v ? atoi(v) : -1; }();
    return forced;
}

static bool chain_bound(const spx_ell* e, uint32_t C)
{
    const int forced = staged_mode();
    if (C <= 128) return false;
    if (forced == 2) return true;                   // experiment: every row on 128-column panels
    if (e->long_rows == 0) return false;
    if (forced >= 0) return forced != 0;
    const double kernel_us = (double)e->nnz_total * C * 4.0 / 17e6 * (148.0 / sm_count(e->device));
    const double chain_us = e->max_nnz / 4.0 * 1.2;
    return chain_us > 0.4 * kernel_us;
}

int launch_spmm(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias,
                int act, float* Y, uint64_t ldy, cudaStream_t s)
{
    float* one[1] = { Y };
    return launch_spmm_bcast(e, X, C, ldx, bias, act, one, 1, 0, ldy, s);
}

int launch_spmm_bcast(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                      float* const* Ys, uint32_t npeers, uint64_t row0, uint64_t ldy, cudaStream_t s, bool mcast)
{
    if (e->m == 0 || C == 0) return SPX_OK;
    if (npeers == 0 || npeers > (uint32_t)kMaxPeers) return fail(SPX_ERR_LIMIT, "spmm: 1..%d destination buffers supported", kMaxPeers);
    if (mcast && npeers != 1) return fail(SPX_ERR_ARG, "spmm: a multicast destination is one address");
    PeerOut out{};
    out.n = (int)npeers;
    out.mcast = mcast ? 1 : 0;
    out.row0 = row0;
    bool aligned = true;
    for (uint32_t g = 0; g < npeers; ++g) {
        if (!Ys[g]) return fail(SPX_ERR_ARG, "spmm: destination %u is null", g);
        out.p[g] = Ys[g];
        aligned = aligned && (reinterpret_cast<uintptr_t>(Ys[g]) & 15) == 0;
    }
    static const int half_env = [] { const char* v = getenv("SPX_SPMM_HALF"); return v ? atoi(v) : 1; }();
    const bool vec_ok = (C % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) &&
                        ((reinterpret_cast<uintptr_t>(X) & 15) == 0) && aligned;
    if (vec_ok && C <= 64) {
        const int lpr = C <= 32 ? 8 : 16;
        const uint32_t rpw = 32 / lpr;
        const uint32_t warps = (e->m + rpw - 1) / rpw;
        uint32_t wpb = 8;
        while (wpb > 1 && (uint64_t)((warps + wpb - 1) / wpb) < (uint64_t)sm_count(e->device) * 8) wpb >>= 1;
        const uint32_t blocks = (warps + wpb - 1) / wpb;
        // Few rows per SM and 8 lanes per row: the kernel is bound by the per-row chain of gathers,
        // so use the registers the idle warps leave free for twice as many gathers in flight per row
        // (batch 32 forward of a 4096-wide MLP: 0.165 -> 0.106 ms; with 16 lanes per row it was slower).
        static const int deep_env = [] { const char* v = getenv("SPX_SPMM_SUB_DEEP"); return v ? atoi(v) : -1; }();
        const bool deep = deep_env >= 0 ? deep_env != 0 : warps < (uint64_t)sm_count(e->device) * 16;
        // L2 prefetch of each row's slabs at row start: 4096-wide MLP at batch 32, 0.102 -> 0.096 ms;
        // a 134 MB matrix (larger than L2) got 16 % slower with it, hence the size limit.
        const bool pf = e->nnz_total * 8 <= (32ull << 20);
        if (lpr == 8 && deep)
            spmm_gather_sub<8, 4, 1><<<blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                X, C, ldx, bias, act, out, ldy, pf);
        else if (lpr == 8)
            spmm_gather_sub<8, 2, 4><<<blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                X, C, ldx, bias, act, out, ldy, pf);
        else
            spmm_gather_sub<16, 1, 4><<<blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                 X, C, ldx, bias, act, out, ldy, pf);
        SPX_LAUNCH_CHECK("spmm_gather_sub");
    } else if (vec_ok && C <= 128 && half_env) {
        const uint32_t warps = (e->m + 1) / 2;
        uint32_t wpb = 8;
        while (wpb > 1 && (uint64_t)((warps + wpb - 1) / wpb) < (uint64_t)sm_count(e->device) * 8) wpb >>= 1;
        const uint32_t blocks = (warps + wpb - 1) / wpb;
        spmm_gather_half<4, 4><<<blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                          X, C, ldx, bias, act, out, ldy);
        SPX_LAUNCH_CHECK("spmm_gather_half");
    } else if (vec_ok) {
        const int nv = gather_nv(e->n, C);
        // A row is one dependent chain of gathers, G rows of X per round trip to L2 (about a
        // microsecond under load).  When the longest row's chain is a large part of the whole
        // kernel (few rows per GPU, skewed lengths) it becomes the tail: spmm_gather_staged then
        // gives the rows with 512 and more entries 128-column panels with eight rows of X in
        // flight per round trip (half the round trips), issued first.
        if (nv == 2 && ldx < (1ull << 30) && chain_bound(e, C)) {
            const bool all_narrow = staged_mode() == 2;
            const uint32_t wpb = gather_wpb(e, (C + 255) / 256);
            StagedMap sm{};
            sm.all_narrow = all_narrow ? 1u : 0u;
            // With the exchange fused in, every finished row is 4*C bytes to each peer, whatever its
            // length.  In descending order the many short rows all finish at the end and the links
            // idle until then; shortest first behind the head keeps them busy from the start, while
            // the long rows (the head) still start at once.  SPX_SPMM_BCAST_ORDER=0 keeps descending.
            static const int order_env = [] { const char* v = getenv("SPX_SPMM_BCAST_ORDER"); return v ? atoi(v) : 1; }();
            sm.rest_ascending = ((npeers > 1 || mcast) && order_env) ? 1u : 0u;
            sm.row_blocks = (e->m + wpb - 1) / wpb;
            sm.panels = all_narrow ? (C + 127) / 128 : (C + 255) / 256;
            sm.head_panels = (C + 127) / 128;
            sm.head = all_narrow ? 0u : std::min<uint32_t>(sm.row_blocks, (e->long_rows + wpb - 1) / wpb);
            sm.blocks = sm.head * sm.head_panels + (sm.row_blocks - sm.head) * sm.panels;
            spmm_gather_staged<<<sm.blocks, wpb * 32, (size_t)wpb * 512, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                          X, C, (uint32_t)(ldx * 4), bias, act, out, ldy, sm);
            SPX_LAUNCH_CHECK("spmm_gather_staged");
            return SPX_OK;
        }
        const uint32_t panels = (C + 128 * nv - 1) / (128 * nv);
        const uint32_t wpb = gather_wpb(e, panels);
        const BlockMap bm = block_map(e, C, panels, wpb);
        if (nv == 1)
            spmm_gather_vec<1, 8, 4><<<bm.blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                   X, C, ldx, bias, act, out, ldy, bm);
        else
            spmm_gather_vec<2, 4, 4><<<bm.blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                   X, C, ldx, bias, act, out, ldy, bm);
        SPX_LAUNCH_CHECK("spmm_gather_vec");
    } else {
        const int nv = C > 32 ? 2 : 1;
        const uint32_t panels = (C + 32 * nv - 1) / (32 * nv);
        const uint32_t wpb = gather_wpb(e, panels);
        const BlockMap bm = block_map(e, C, panels, wpb);
        if (nv == 2)
            spmm_gather_scalar<2><<<bm.blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                X, C, ldx, bias, act, out, ldy, bm);
        else
            spmm_gather_scalar<1><<<bm.blocks, wpb * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->pitch,
                                                                X, C, ldx, bias, act, out, ldy, bm);
        SPX_LAUNCH_CHECK("spmm_gather_scalar");
    }
    return SPX_OK;
}

}  // namespace spx
