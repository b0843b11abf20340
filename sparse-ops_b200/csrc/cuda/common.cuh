// common.cuh -- shared declarations of the CUDA side of libspx_b200.so (sm_100a only).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "spx_b200.h"

// Device-resident ELLPACK (see include/spx_b200.h).  Row i occupies entries
// [i*pitch, i*pitch + nnz[i]) of Wd / idx; pitch is a multiple of 32 entries so that
// every row starts on a 128-byte boundary and float4 / uint4 loads are aligned.
struct spx_ell {
    int device = 0;
    uint32_t m = 0, n = 0, r = 0;
    uint32_t pitch = 0;          // row pitch in entries (0 when r == 0)
    uint64_t nnz_total = 0;
    uint32_t max_nnz = 0;        // longest row actually stored (<= r)
    uint32_t min_nnz = 0;        // shortest row
    float* Wd = nullptr;         // m * pitch floats
    uint32_t* idx = nullptr;     // m * pitch column ids
    uint32_t* nnz = nullptr;     // m counts
    // Row schedule: row ids sorted by descending nnz (ties by ascending id).  Kernels that give a
    // warp one row take rows in this order, so the warps of a CTA get rows of equal length
    // (no warp idles behind a long row) and the longest rows start first.
    uint32_t* row_order = nullptr;   // m row ids
    uint32_t long_rows = 0;          // rows with at least 512 stored entries (a prefix of row_order)
    // Lazily built, cached conv tap table: idx decoded to packed (cin, kh, kw) for one
    // kernel shape (conv.cu); keyed by (kH, kW).
    uint32_t* taps = nullptr;
    uint32_t taps_kH = 0, taps_kW = 0;
    // True when every row's stored column ids are strictly ascending (always so for handles made
    // from CSR, from a dense matrix or by the encoders; checked at upload for raw arrays).  The
    // tiled convolution kernels rely on it; without it the convolution takes the general kernel.
    bool cols_ascending = true;
    // Lazily built row-block-merged form of the weights for the convolution (conv.cu): per block
    // of 4 rows the ascending union of their column ids; per union column a header
    // (packed tap, 4-bit row mask) and the 4 rows' weights (0.0f where a row has no entry).
    // Block b owns entries [b * rbm_cap, b * rbm_cap + rbm_ncols[b]).
    uint2* rbm_hdr = nullptr;
    float* rbm_w = nullptr;
    uint32_t* rbm_ncols = nullptr;
    uint32_t rbm_cap = 0, rbm_kH = 0, rbm_kW = 0;
    // Raised by a convolution kernel whose bounded wait for a bulk tensor copy ran out: a word in
    // device memory (read by the kernel's later CTAs) and a word in pinned host memory (its device
    // alias is tma_failed_mapped; read by the next convolution call on the handle).
    int* tma_failed_host = nullptr;
    int* tma_failed_mapped = nullptr;
    int* tma_failed_dev = nullptr;
    bool tma_off = false;
    // SpMV with x larger than shared memory (spmv.cu): column window width and the per-row split
    // table, built on the first spx_spmv of such a handle.  spmv_win == UINT32_MAX: not applicable.
    uint32_t* spmv_split = nullptr;
    uint32_t spmv_win = 0;
    // Pinned + device staging for the host-buffer entry points (abi.cu), grown on demand.
    void* stage_dev = nullptr;
    size_t stage_dev_bytes = 0;
    // Scratch of the NCHW convolution path: the input and output in [C,H,W,B] order (conv.cu).
    void* conv_scratch = nullptr;
    size_t conv_scratch_bytes = 0;
    // Scratch of the F-major convolution path: input and output in [C,H,W,B] order (conv.cu).
    void* fm_scratch = nullptr;
    size_t fm_scratch_bytes = 0;
    // Streams of the pipelined host-buffer SpMM (copy in, exchange, multiply, copy out) and the events
    // that chain and time its stages, created on first use and kept.
    cudaStream_t pipe_streams[4] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t pipe_events[64] = {};
    // Row slices for the copy-engine exchange (spx_spmm_exchange, abi.cu): handles over contiguous
    // row ranges of this one that share its Wd / idx / nnz arrays and own only their row schedule
    // (view == true for such a handle).  slice_row0[k] is slice k's first row; the streams carry
    // the peer copies, the events chain them to the multiplications.
    bool view = false;
    uint32_t nslices = 0;
    spx_ell* slices[16] = {};
    uint32_t slice_row0[17] = {};
    cudaStream_t xchg_streams[4] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t xchg_events[24] = {};
};

namespace spx {

int fail(int code, const char* fmt, ...);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int sm_count(int device);

// Rounds up to a multiple of `to`.
template <class T> __host__ __device__ inline T round_up(T v, T to) { return (v + to - 1) / to * to; }

__device__ __forceinline__ float apply_act(float v, int act) {
    // Precise expf / tanhf: the library is built without fast-math so that sigmoid and tanh
    // stay within a few ulp of the C library results of the reference.
    switch (act) {
    case SPX_ACT_RELU:    return v > 0.0f ? v : 0.0f;
    case SPX_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    case SPX_ACT_TANH:    return tanhf(v);
    default:              return v;
    }
}

// (a0, a1) += w * (x0, x1) with ONE instruction: sm_100a's packed fma.rn.f32x2.  Each half is an
// IEEE fused multiply-add rounded to nearest -- exactly fmaf -- so chains stay bit-identical while
// the FMA instruction count halves.  The 64-bit pairs are formed inside the block, which leaves
// the register allocator free to keep the operands in adjacent registers.
__device__ __forceinline__ void fma_pair(float& a0, float& a1, float w, float x0, float x1) {
    asm("{\n\t.reg .b64 pa, px, pw;\n\tmov.b64 pa, {%0, %1};\n\tmov.b64 px, {%3, %4};\n\tmov.b64 pw, {%2, %2};\n\t"
        "fma.rn.f32x2 pa, pw, px, pa;\n\tmov.b64 {%0, %1}, pa;\n\t}"
        : "+f"(a0), "+f"(a1) : "f"(w), "f"(x0), "f"(x1));
}

}  // namespace spx

#define SPX_CUDA(call)                                                                     \
    do {                                                                                   \
        cudaError_t _e = (call);                                                           \
        if (_e != cudaSuccess)                                                             \
            return spx::fail(_e == cudaErrorMemoryAllocation ? SPX_ERR_OOM : SPX_ERR_CUDA, \
                             "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e),       \
                             __FILE__, __LINE__);                                          \
    } while (0)

#define SPX_LAUNCH_CHECK(name)                                                             \
    do {                                                                                   \
        cudaError_t _e = cudaGetLastError();                                               \
        if (_e != cudaSuccess)                                                             \
            return spx::fail(SPX_ERR_CUDA, "launch of %s failed: %s", name,                \
                             cudaGetErrorString(_e));                                      \
        spx::count_launch();                                                               \
    } while (0)

// Kernel launchers implemented in the individual .cu files.
namespace spx {
int launch_spmm(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias,
                int act, float* Y, uint64_t ldy, cudaStream_t s);
int launch_spmm_bcast(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                      float* const* Ys, uint32_t npeers, uint64_t row0, uint64_t ldy, cudaStream_t s, bool mcast = false);
int launch_spmv(spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s);
int launch_spmv_reforder(const spx_ell* e, const float* x, const float* bias, float* y, cudaStream_t s);
int launch_conv2d(spx_ell* e, const spx_conv_geom* g, int layout, const float* in, uint32_t B,
                  const float* bias, int act, float* out, cudaStream_t s);
int launch_eltwise(int op, const float* a, const float* b, float* out, uint64_t count, cudaStream_t s);
int encode_device(const float* dW, uint32_t m, uint32_t n, cudaStream_t s, spx_ell** out);
int decode_device(const spx_ell* e, float* dW, cudaStream_t s);
int csr_to_ell_device(spx_ell* e, const uint64_t* d_rowptr, const uint32_t* d_col, const float* d_val,
                      cudaStream_t s);
int alloc_ell(uint32_t m, uint32_t n, uint32_t r, spx_ell** out, cudaStream_t s);
int check_current_device(const spx_ell* e, const char* what);
// Builds e->row_order from host row counts (counting sort by length) and uploads it.
int set_row_order(spx_ell* e, const uint32_t* host_nnz);
}  // namespace spx
