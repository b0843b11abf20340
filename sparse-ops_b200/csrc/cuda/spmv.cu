// spmv.cu -- ELLPACK SpMV  y = bias + E * x  for sm_100a.
//
// Replaces ellpack_matvec of the reference (src/ellpack_matvec.cpp:20-147).  The reference
// gathers x[idx] for all r slots of a row into the Xt scratch, then runs a 16-lane FMA over
// the nnz[i] live entries and a horizontal reduce.  Here the gather goes straight to
// registers: x is staged once per CTA in shared memory (random 4-byte reads cost a few bank
// conflicts there instead of one L1 line each), LPR lanes share a row and stream its Wd / idx
// slab with coalesced 16-byte loads, partial sums are combined with warp shuffles.  The
// summation order differs from the reference's 16-partial-sum order, so results agree within
// the stated tolerance 1e-5 * sum|w||x|, not bit for bit.  Padding slots are never multiplied.
//
// The kernel is HBM-bound: 8 bytes per nonzero streamed once.  The grid is persistent
// (a multiple of the SM count) so x is staged once per CTA.
#include "common.cuh"

#include <algorithm>
#include <climits>
#include <cstdint>
#include <cstdlib>

namespace {

template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int LPR, bool SMEM>
__global__ void __launch_bounds__(1024)
spmv_ell_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                uint32_t m, uint32_t n, uint32_t pitch,
                const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y)
{
    extern __shared__ __align__(16) float xs[];
    if (SMEM) {
        // n floats, 16-byte vectors where alignment allows
        const uint32_t n4 = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? (n >> 2) : 0;
        for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x)
            reinterpret_cast<float4*>(xs)[i] = __ldg(reinterpret_cast<const float4*>(x) + i);
        for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) xs[i] = __ldg(x + i);
        __syncthreads();
    }
    const float* __restrict__ xsrc = SMEM ? xs : x;

    const uint32_t lane = threadIdx.x & (LPR - 1);
    const uint32_t groups_per_block = blockDim.x / LPR;
    const uint32_t group = blockIdx.x * groups_per_block + threadIdx.x / LPR;
    const uint32_t stride = gridDim.x * groups_per_block;
    // All lanes of a warp run the same number of row iterations so that the shuffles below
    // always see the full warp.
    const uint32_t iters = (m + stride - 1) / stride;

    for (uint32_t it = 0; it < iters; ++it) {
        // slots of the sorted row schedule are dealt round-robin: every group gets long and short rows
        const uint32_t slot = group + it * stride;
        const bool live = slot < m;
        const uint32_t row = live ? __ldg(row_order + slot) : 0u;
        const uint32_t nn = live ? __ldg(nnz + row) : 0u;
        const float4* __restrict__ w4 = reinterpret_cast<const float4*>(Wd + (size_t)row * pitch);
        const uint4* __restrict__ k4 = reinterpret_cast<const uint4*>(idx + (size_t)row * pitch);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        // UNR 16-byte vectors of Wd and of idx in flight per lane; entries >= nn are padding and
        // are neither loaded nor multiplied
        constexpr int UNR = 4;
        for (uint32_t j = lane * 4; j < nn; j += LPR * 4 * UNR) {
            float4 wv[UNR];
            uint4 kv[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t ju = j + u * LPR * 4;
                if (ju < nn) {
                    wv[u] = __ldcs(w4 + (ju >> 2));
                    kv[u] = __ldcs(k4 + (ju >> 2));
                } else {
                    wv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    kv[u] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t ju = j + u * LPR * 4;
                if (ju < nn) a0 = fmaf(wv[u].x, xsrc[kv[u].x], a0);
                if (ju + 1 < nn) a1 = fmaf(wv[u].y, xsrc[kv[u].y], a1);
                if (ju + 2 < nn) a2 = fmaf(wv[u].z, xsrc[kv[u].z], a2);
                if (ju + 3 < nn) a3 = fmaf(wv[u].w, xsrc[kv[u].w], a3);
            }
        }
        float acc = (a0 + a1) + (a2 + a3);
        acc = group_sum<LPR>(acc);
        if (live && lane == 0) y[row] = (bias ? __ldg(bias + row) : 0.0f) + acc;
    }
}

// spmv_ell_small_kernel: matrices of a few thousand columns (x up to 32 KB).  They are
// latency-bound: staging x, the row schedule, the row length and the slabs would be four memory
// round trips in a row.  So this kernel is software-pipelined: a group asks
// for its first row's id and length and for that row's first slab vectors BEFORE x is staged (none
// of them depends on x), and while a row is summed the next row's id, length and first vectors
// are already in flight.  row_order may be null (rows of near-equal length): slot == row then, and
// one dependent load goes away.
template <int LPR>
__global__ void __launch_bounds__(1024)
spmv_ell_small_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                uint32_t m, uint32_t n, uint32_t pitch,
                const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y)
{
    extern __shared__ __align__(16) float xs[];
    constexpr int UNR = 4;                       // 16-byte vectors of Wd and of idx in flight per lane
    constexpr uint32_t STEP = LPR * 4 * UNR;     // entries a group consumes per chunk
    const uint32_t lane = threadIdx.x & (LPR - 1);
    const uint32_t groups_per_block = blockDim.x / LPR;
    const uint32_t group = blockIdx.x * groups_per_block + threadIdx.x / LPR;
    const uint32_t stride = gridDim.x * groups_per_block;
    // All lanes of a warp run the same number of row iterations so that the shuffles below
    // always see the full warp.
    const uint32_t iters = (m + stride - 1) / stride;

    float4 wv[UNR];
    uint4 kv[UNR];
    // entries >= nn are padding and are neither loaded nor multiplied
    auto load_chunk = [&](uint32_t row, uint32_t nn, uint32_t j) {
        const float4* __restrict__ w4 = reinterpret_cast<const float4*>(Wd + (size_t)row * pitch);
        const uint4* __restrict__ k4 = reinterpret_cast<const uint4*>(idx + (size_t)row * pitch);
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t ju = j + u * LPR * 4;
            if (ju < nn) {
                wv[u] = __ldcs(w4 + (ju >> 2));
                kv[u] = __ldcs(k4 + (ju >> 2));
            } else {
                wv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                kv[u] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    // slots of the sorted row schedule are dealt round-robin: every group gets long and short rows
    uint32_t slot = group;
    bool live = slot < m;
    uint32_t row = live ? (row_order ? __ldg(row_order + slot) : slot) : 0u;
    uint32_t nn = live ? __ldg(nnz + row) : 0u;
    load_chunk(row, nn, lane * 4);

    {
        // n floats, 16-byte vectors where alignment allows
        const uint32_t n4 = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? (n >> 2) : 0;
        for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x)
            reinterpret_cast<float4*>(xs)[i] = __ldg(reinterpret_cast<const float4*>(x) + i);
        for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) xs[i] = __ldg(x + i);
        __syncthreads();
    }
    const float* __restrict__ xsrc = xs;

    for (uint32_t it = 0; it < iters; ++it) {
        // the next row's id and length travel while this row is summed
        const uint32_t slot_n = slot + stride;
        const bool live_n = (it + 1 < iters) && slot_n < m;
        const uint32_t row_n = live_n ? (row_order ? __ldg(row_order + slot_n) : slot_n) : 0u;
        const uint32_t nn_n = live_n ? __ldg(nnz + row_n) : 0u;
        const float b = (live && bias) ? __ldg(bias + row) : 0.0f;

        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (uint32_t j = lane * 4; j < nn; j += STEP) {
            if (j != lane * 4) load_chunk(row, nn, j);          // the first chunk is already here
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t ju = j + u * LPR * 4;
                if (ju < nn) a0 = fmaf(wv[u].x, xsrc[kv[u].x], a0);
                if (ju + 1 < nn) a1 = fmaf(wv[u].y, xsrc[kv[u].y], a1);
                if (ju + 2 < nn) a2 = fmaf(wv[u].z, xsrc[kv[u].z], a2);
                if (ju + 3 < nn) a3 = fmaf(wv[u].w, xsrc[kv[u].w], a3);
            }
        }
        load_chunk(row_n, nn_n, lane * 4);                      // first vectors of the next row
        float acc = (a0 + a1) + (a2 + a3);
        acc = group_sum<LPR>(acc);
        if (live && lane == 0) y[row] = b + acc;
        slot = slot_n; live = live_n; row = row_n; nn = nn_n;
    }
}

// ---------------------------------------------------------------------------------------------
// x larger than shared memory: the columns are cut into equal windows that do fit, and the kernel
// runs one phase per window: stage x[window], then every row adds the products of its entries
// whose column lies in the window (a contiguous run, rows ascend; the run's ends come from a
// per-row split table built once per handle by binary search).  Each matrix entry is still read
// once; y is written in phase 0 (bias + partial) and updated by the same lane in later phases.
// Against gathering x through L1 / L2 (32-byte sectors for 4 useful bytes) this keeps every gather
// in shared memory.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
spmv_splits_kernel(const uint32_t* __restrict__ idx, const uint32_t* __restrict__ nnz, uint32_t m, uint32_t pitch,
                   uint32_t win, uint32_t bounds, uint32_t* __restrict__ split)
{
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (uint64_t)m * bounds) return;
    const uint32_t row = (uint32_t)(t % m), b = (uint32_t)(t / m);
    const uint32_t bound = (b + 1) * win;
    const uint32_t* __restrict__ k = idx + (size_t)row * pitch;
    uint32_t lo = 0, hi = nnz[row];
    while (lo < hi) {                           // first entry with column >= bound
        const uint32_t mid = (lo + hi) >> 1;
        if (k[mid] < bound) lo = mid + 1; else hi = mid;
    }
    split[t] = lo;
}

template <int LPR>
__global__ void __launch_bounds__(1024)
spmv_ell_windowed_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                         const uint32_t* __restrict__ nnz, const uint32_t* __restrict__ row_order,
                         const uint32_t* __restrict__ split, uint32_t m, uint32_t n, uint32_t win, uint32_t pitch,
                         const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y)
{
    extern __shared__ __align__(16) float xs[];
    const uint32_t lane = threadIdx.x & (LPR - 1);
    const uint32_t groups_per_block = blockDim.x / LPR;
    const uint32_t group = blockIdx.x * groups_per_block + threadIdx.x / LPR;
    const uint32_t stride = gridDim.x * groups_per_block;
    const uint32_t iters = (m + stride - 1) / stride;
    const uint32_t phases = (n + win - 1) / win;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0;      // win is a multiple of 4

    for (uint32_t p = 0; p < phases; ++p) {
        const uint32_t lo = p * win, cnt = min(win, n - lo);
        if (p) __syncthreads();                 // the previous window is no longer read
        const uint32_t n4 = vec_ok ? (cnt >> 2) : 0;
        for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x)
            reinterpret_cast<float4*>(xs)[i] = __ldg(reinterpret_cast<const float4*>(x + lo) + i);
        for (uint32_t i = (n4 << 2) + threadIdx.x; i < cnt; i += blockDim.x) xs[i] = __ldg(x + lo + i);
        __syncthreads();

        // this phase's run [j0, j1) of a row: split table entries p-1 and p (0 and nnz at the ends)
        auto run_of = [&](uint32_t r, uint32_t& b0, uint32_t& b1) {
            b0 = p ? __ldg(split + (size_t)(p - 1) * m + r) : 0u;
            b1 = (p + 1 < phases) ? __ldg(split + (size_t)p * m + r) : __ldg(nnz + r);
        };
        // the next row's run and the id of the row after it are fetched while the current row streams
        uint32_t row = group < m ? __ldg(row_order + group) : 0u;
        uint32_t j0_next = 0, j1_next = 0;
        if (group < m) run_of(row, j0_next, j1_next);
        uint32_t row_next = (uint64_t)group + stride < m ? __ldg(row_order + group + stride) : 0u;
        for (uint32_t it = 0; it < iters; ++it) {
            const uint32_t slot = group + it * stride;
            const bool live = slot < m;
            const uint32_t j0 = j0_next, j1 = j1_next;
            const uint32_t row_after = row_next;
            {
                const uint64_t s1 = (uint64_t)slot + stride, s2 = s1 + stride;
                j0_next = j1_next = 0;
                if (s1 < m) run_of(row_after, j0_next, j1_next);
                row_next = s2 < m ? __ldg(row_order + s2) : 0u;
            }
            const float4* __restrict__ w4 = reinterpret_cast<const float4*>(Wd + (size_t)row * pitch);
            const uint4* __restrict__ k4 = reinterpret_cast<const uint4*>(idx + (size_t)row * pitch);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            constexpr int UNR = 4;
            // vectors from the one holding entry j0; entries outside [j0, j1) belong to other phases
            for (uint32_t j = (j0 & ~3u) + lane * 4; j < j1; j += LPR * 4 * UNR) {
                float4 wv[UNR];
                uint4 kv[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const uint32_t ju = j + u * LPR * 4;
                    if (ju < j1) {
                        wv[u] = __ldcs(w4 + (ju >> 2));
                        kv[u] = __ldcs(k4 + (ju >> 2));
                    } else {
                        wv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        kv[u] = make_uint4(lo, lo, lo, lo);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const uint32_t ju = j + u * LPR * 4;
                    if (ju >= j0 && ju < j1) a0 = fmaf(wv[u].x, xs[kv[u].x - lo], a0);
                    if (ju + 1 >= j0 && ju + 1 < j1) a1 = fmaf(wv[u].y, xs[kv[u].y - lo], a1);
                    if (ju + 2 >= j0 && ju + 2 < j1) a2 = fmaf(wv[u].z, xs[kv[u].z - lo], a2);
                    if (ju + 3 >= j0 && ju + 3 < j1) a3 = fmaf(wv[u].w, xs[kv[u].w - lo], a3);
                }
            }
            float acc = (a0 + a1) + (a2 + a3);
            acc = group_sum<LPR>(acc);
            if (live && lane == 0) {
                if (p == 0) y[row] = (bias ? __ldg(bias + row) : 0.0f) + acc;
                else if (j1 > j0) y[row] += acc;
            }
            row = row_after;
        }
    }
}

// Reference-order variant: reproduces the summation order of the reference's AVX-512 path bit for
// bit (src/ellpack_matvec.cpp:72-99): sixteen partial sums, partial l takes entries j = l, l+16, ...
// with one FMA each starting from 0; then lanes l and l+8, l and l+4, the two horizontal adds, and
// finally bias + sum.  Sixteen lanes per row; slower than spmv_ell_kernel (4-byte loads, chains of
// nnz/16), meant for checking, not for throughput.
__global__ void __launch_bounds__(256)
spmv_reforder_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
                     const uint32_t* __restrict__ nnz, uint32_t m, uint32_t pitch,
                     const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y)
{
    const uint32_t l = threadIdx.x & 15;
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const bool live = row < m;
    const uint32_t nn = live ? __ldg(nnz + row) : 0u;
    const float* __restrict__ w = Wd + (size_t)(live ? row : 0) * pitch;
    const uint32_t* __restrict__ k = idx + (size_t)(live ? row : 0) * pitch;
    float a = 0.0f;
    for (uint32_t j = l; j < nn; j += 16) a = fmaf(__ldg(w + j), __ldg(x + __ldg(k + j)), a);
    a = a + __shfl_xor_sync(0xffffffffu, a, 8);      // l with l+8
    a = a + __shfl_xor_sync(0xffffffffu, a, 4);      // l with l+4
    a = a + __shfl_xor_sync(0xffffffffu, a, 1);      // (0+1), (2+3)
    a = a + __shfl_xor_sync(0xffffffffu, a, 2);      // their sum
    if (live && l == 0) y[row] = (bias ? __ldg(bias + row) : 0.0f) + a;
}

constexpr size_t kSmallX = 32 * 1024;

template <int LPR, bool SMEM>
int launch_one(const spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s,
               int threads, int blocks, size_t smem)
{
    auto kfn = spmv_ell_kernel<LPR, SMEM>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return spx::fail(SPX_ERR_CUDA, "spmv: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    kfn<<<blocks, threads, smem, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->m, e->n, e->pitch, x, bias, y);
    SPX_LAUNCH_CHECK("spmv_ell_kernel");
    return SPX_OK;
}

// Shrinks a persistent grid so that every group runs the same number of row iterations
// (a grid of 9324 groups over 16384 rows would give some groups two rows and others one).
static int balanced_blocks(uint64_t rows, int groups_per_block, int max_blocks)
{
    const uint64_t cap = (uint64_t)max_blocks * groups_per_block;
    const uint64_t iters = (rows + cap - 1) / cap;
    const uint64_t blocks = (rows + iters * groups_per_block - 1) / (iters * groups_per_block);
    return (int)(blocks ? blocks : 1);
}

// Small x (up to 32 KB): the pipelined kernel on a grid with the same number of CTAs on every SM.
template <int LPR>
int launch_small(const spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s)
{
    const int sms = spx::sm_count(e->device);
    const size_t xbytes = (size_t)e->n * sizeof(float);
    const uint64_t groups_needed = e->m;
    // Rows of near-equal length need no schedule: slot == row saves one dependent load per row.
    const uint32_t* order = (e->max_nnz - e->min_nnz) * 8u <= e->max_nnz ? nullptr : e->row_order;
    // Rows per group (iters) as if every SM held 4 CTAs of 512 threads; then the same number of CTAs
    // on every SM -- as few as carry the rows in that many iterations (x is staged once per CTA) --
    // each with equally many groups.  A grid that is not a multiple of the SM count leaves some SMs
    // with one CTA more than others for the whole kernel.
    constexpr int kPerSm = 4, kThreadsFull = 512;
    const uint64_t cap = (uint64_t)sms * kPerSm * (kThreadsFull / LPR);
    const uint64_t iters = (groups_needed + cap - 1) / cap;
    const uint64_t per_iter = (groups_needed + iters - 1) / iters;         // groups that must exist
    int threads = kThreadsFull, blocks = sms * kPerSm;
    for (int k = 1; k <= kPerSm; ++k) {       // (forcing 2 or 4 CTAs per SM measured the same 8.1 us on 4096 x 4096)
        const uint64_t g = (per_iter + (uint64_t)sms * k - 1) / ((uint64_t)sms * k);
        const uint64_t t = (g * LPR + 31) / 32 * 32;
        if (t <= std::min<uint64_t>(1024, 2048 / k)) {
            threads = (int)t;
            blocks = (int)std::min<uint64_t>((uint64_t)sms * k, (per_iter + g - 1) / g);
            break;
        }
    }
    spmv_ell_small_kernel<LPR><<<blocks, threads, xbytes, s>>>(e->Wd, e->idx, e->nnz, order, e->m, e->n, e->pitch, x, bias, y);
    SPX_LAUNCH_CHECK("spmv_ell_small_kernel");
    return SPX_OK;
}

template <int LPR>
int launch_lpr(const spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s)
{
    const int sms = spx::sm_count(e->device);
    const size_t xbytes = (size_t)e->n * sizeof(float);
    // Measured on B200: the pipelined kernel wins for 4096 columns at every sparsity (8.7 -> 8.1 us
    // at 90 %, 12 -> 10.4 us at 80 %); at 16384 columns it is mixed and with x gathered from global
    // memory it is 6 % slower, so larger matrices keep the kernel below.
    if (xbytes <= kSmallX) return launch_small<LPR>(e, x, bias, y, s);
    const size_t kSmemMax = 200 * 1024;      // leaves room for a second small CTA's static needs
    const uint64_t groups_needed = e->m;
    if (xbytes <= kSmemMax) {
        // CTAs per SM limited by the staged copy of x; 2048 threads per SM at most.
        int per_sm = (int)((220 * 1024) / (xbytes + 1024));
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 4) per_sm = 4;
        int threads = 2048 / per_sm;
        if (threads > 1024) threads = 1024;
        threads &= ~31;
        const int blocks = balanced_blocks(groups_needed, threads / LPR, sms * per_sm);
        return launch_one<LPR, true>(e, x, bias, y, s, threads, blocks, xbytes);
    }
    if (e->spmv_split) {
        const int blocks = balanced_blocks(groups_needed, 1024 / LPR, sms);
        const size_t smem = (size_t)e->spmv_win * sizeof(float);
        auto kfn = spmv_ell_windowed_kernel<LPR>;
        cudaError_t err = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return spx::fail(SPX_ERR_CUDA, "spmv: shared memory opt-in failed: %s", cudaGetErrorString(err));
        kfn<<<blocks, 1024, smem, s>>>(e->Wd, e->idx, e->nnz, e->row_order, e->spmv_split, e->m, e->n, e->spmv_win,
                                       e->pitch, x, bias, y);
        SPX_LAUNCH_CHECK("spmv_ell_windowed_kernel");
        return SPX_OK;
    }
    int threads = 512;
    const int blocks = balanced_blocks(groups_needed, threads / LPR, sms * 4);
    return launch_one<LPR, false>(e, x, bias, y, s, threads, blocks, 0);
}

}  // namespace

namespace spx {

int launch_spmv_reforder(const spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s)
{
    if (e->m == 0) return SPX_OK;
    const uint64_t threads = (uint64_t)e->m * 16;
    spmv_reforder_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(e->Wd, e->idx, e->nnz, e->m, e->pitch, x, bias, y);
    SPX_LAUNCH_CHECK("spmv_reforder_kernel");
    return SPX_OK;
}

// x beyond shared memory: up to kMaxWindows equal column windows of at most 200 KB; the per-row
// split table ((windows - 1) * m entries) is built on the first call and cached in the handle.
static int ensure_spmv_windows(spx_ell* e, cudaStream_t s)
{
    constexpr uint32_t kWinMax = 200 * 1024 / sizeof(float), kMaxWindows = 8;
    static const int enabled = [] { const char* v = getenv("SPX_SPMV_WINDOWED"); return v ? atoi(v) : 1; }();
    if (e->spmv_split || e->spmv_win == UINT32_MAX) return SPX_OK;
    e->spmv_win = UINT32_MAX;                                       // decided: stays "no" unless built below
    if (!enabled || !e->cols_ascending || e->n <= kWinMax || e->max_nnz == 0) return SPX_OK;
    const uint32_t windows = (e->n + kWinMax - 1) / kWinMax;
    if (windows > kMaxWindows) return SPX_OK;
    // Measured at 65536 x 65536: 307 vs 321 us at 95 % sparsity and 84 vs 97 us at 99 % (the
    // gathers of x stop crossing L2 -> SM as 32-byte sectors), equal at 90 %, 1117 vs 1086 us at
    // 80 % (long rows stream at 97 % of the copy bandwidth either way and the second pass over the
    // rows only costs): taken when a row's run inside a window is short.  SPX_SPMV_WINDOWED=2 forces it.
    const double run = (double)e->nnz_total / e->m / windows;
    if (enabled != 2 && run > 2500.0) return SPX_OK;
    const uint32_t win = round_up((e->n + windows - 1) / windows, 4u);
    const uint64_t entries = (uint64_t)e->m * (windows - 1);
    if (cudaMalloc(&e->spmv_split, entries * sizeof(uint32_t)) != cudaSuccess) {
        (void)cudaGetLastError();
        e->spmv_split = nullptr;
        return SPX_OK;                                              // no room: gather x from global memory
    }
    spmv_splits_kernel<<<(unsigned)((entries + 255) / 256), 256, 0, s>>>(e->idx, e->nnz, e->m, e->pitch, win, windows - 1,
                                                                       e->spmv_split);
    SPX_LAUNCH_CHECK("spmv_splits_kernel");
    e->spmv_win = win;
    return SPX_OK;
}

int launch_spmv(spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s)
{
    if (e->m == 0) return SPX_OK;
    static const bool exact = [] { const char* v = getenv("SPX_SPMV_REFERENCE_ORDER"); return v && v[0] == '1'; }();
    if (exact) return launch_spmv_reforder(e, x, bias, y, s);
    const int rcw = ensure_spmv_windows(e, s);
    if (rcw != SPX_OK) return rcw;
    // Lanes per row from the mean row length: a lane consumes 4 entries per vector load.
    const double windows = e->spmv_split ? (double)((e->n + e->spmv_win - 1) / e->spmv_win) : 1.0;
    const double mean = e->m ? (double)e->nnz_total / e->m / windows : 0.0;
    if (mean > 192.0) return launch_lpr<32>(e, x, bias, y, s);
    if (mean > 96.0)  return launch_lpr<16>(e, x, bias, y, s);
    if (mean > 40.0)  return launch_lpr<8>(e, x, bias, y, s);
    return launch_lpr<4>(e, x, bias, y, s);
}

}  // namespace spx
