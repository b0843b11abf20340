// encode.cu -- ELLPACK construction and decoding on the device.
//
// encode_device replaces convert_to_ellpack (src/ellpack_encoder.cpp:6-44) for a dense matrix
// that already lives in device memory: pass 1 counts v != 0.0f per row and finds r = the
// longest row, pass 2 packs values and column ids in ascending column order (a warp walks a
// row 32 columns at a time; ballot + popc give each nonzero its slot, which keeps the order).
// The result is bit-identical to the host encoder: -0.0f is dropped, NaN / inf / denormals are
// kept.  decode_device replaces decode_from_ellpack (:46-60).  csr_to_ell_device fills the
// padded slabs from CSR arrays for matrices that never exist densely.
#include "common.cuh"

#include <vector>

namespace {

constexpr int kWarps = 8;

__global__ void __launch_bounds__(kWarps * 32)
count_kernel(const float* __restrict__ W, uint32_t m, uint32_t n, uint32_t* __restrict__ nnz,
             uint32_t* __restrict__ rmax)
{
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= m) return;
    const float* __restrict__ w = W + (size_t)row * n;
    uint32_t cnt = 0;
    for (uint32_t j = lane; j < n; j += 32) cnt += (w[j] != 0.0f) ? 1u : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) {
        nnz[row] = cnt;
        atomicMax(rmax, cnt);
    }
}

__global__ void __launch_bounds__(kWarps * 32)
pack_kernel(const float* __restrict__ W, uint32_t m, uint32_t n, uint32_t pitch,
            float* __restrict__ Wd, uint32_t* __restrict__ idx)
{
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= m) return;
    const float* __restrict__ w = W + (size_t)row * n;
    float* __restrict__ wd = Wd + (size_t)row * pitch;
    uint32_t* __restrict__ ix = idx + (size_t)row * pitch;
    uint32_t pos = 0;
    for (uint32_t j0 = 0; j0 < n; j0 += 32) {
        const uint32_t j = j0 + lane;
        const float v = j < n ? w[j] : 0.0f;
        const bool nz = v != 0.0f;
        const uint32_t bal = __ballot_sync(0xffffffffu, nz);
        if (nz) {
            const uint32_t slot = pos + __popc(bal & ((1u << lane) - 1u));
            wd[slot] = v;
            ix[slot] = j;
        }
        pos += __popc(bal);
    }
}

__global__ void __launch_bounds__(kWarps * 32)
csr_fill_kernel(const uint64_t* __restrict__ rowptr, const uint32_t* __restrict__ col,
                const float* __restrict__ val, uint32_t m, uint32_t pitch,
                float* __restrict__ Wd, uint32_t* __restrict__ idx, uint32_t* __restrict__ nnz)
{
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= m) return;
    const uint64_t b = rowptr[row], e = rowptr[row + 1];
    const uint32_t cnt = (uint32_t)(e - b);
    for (uint32_t j = lane; j < cnt; j += 32) {
        Wd[(size_t)row * pitch + j] = val[b + j];
        idx[(size_t)row * pitch + j] = col[b + j];
    }
    if (lane == 0) nnz[row] = cnt;
}

__global__ void __launch_bounds__(kWarps * 32)
decode_kernel(const float* __restrict__ Wd, const uint32_t* __restrict__ idx,
              const uint32_t* __restrict__ nnz, uint32_t m, uint32_t n, uint32_t pitch,
              float* __restrict__ W)
{
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= m) return;
    const uint32_t cnt = nnz[row];
    for (uint32_t j = lane; j < cnt; j += 32)
        W[(size_t)row * n + idx[(size_t)row * pitch + j]] = Wd[(size_t)row * pitch + j];
}

}  // namespace

namespace spx {

int encode_device(const float* dW, uint32_t m, uint32_t n, cudaStream_t s, spx_ell** out)
{
    uint32_t* d_nnz = nullptr;
    uint32_t* d_rmax = nullptr;
    uint32_t r = 0;
    if (m) {
        SPX_CUDA(cudaMalloc(&d_nnz, (size_t)m * sizeof(uint32_t)));
        cudaError_t err = cudaMalloc(&d_rmax, sizeof(uint32_t));
        if (err != cudaSuccess) { cudaFree(d_nnz); return fail(SPX_ERR_OOM, "encode: cudaMalloc failed"); }
        cudaMemsetAsync(d_rmax, 0, sizeof(uint32_t), s);
        count_kernel<<<(m + kWarps - 1) / kWarps, kWarps * 32, 0, s>>>(dW, m, n, d_nnz, d_rmax);
        count_launch();
        err = cudaMemcpyAsync(&r, d_rmax, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
        if (err == cudaSuccess) err = cudaStreamSynchronize(s);
        cudaFree(d_rmax);
        if (err != cudaSuccess) { cudaFree(d_nnz); return fail(SPX_ERR_CUDA, "encode: count pass failed: %s", cudaGetErrorString(err)); }
    }
    spx_ell* e = nullptr;
    int rc = alloc_ell(m, n, r, &e, s);      // zero fill on s, ahead of the pack below
    if (rc != SPX_OK) { cudaFree(d_nnz); return rc; }
    if (m) {
        cudaMemcpyAsync(e->nnz, d_nnz, (size_t)m * sizeof(uint32_t), cudaMemcpyDeviceToDevice, s);
        if (r) {
            pack_kernel<<<(m + kWarps - 1) / kWarps, kWarps * 32, 0, s>>>(dW, m, n, e->pitch, e->Wd, e->idx);
            count_launch();
        }
        // totals for the kernel heuristics
        std::vector<uint32_t> h(m);
        cudaError_t err = cudaMemcpyAsync(h.data(), d_nnz, (size_t)m * sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
        if (err == cudaSuccess) err = cudaStreamSynchronize(s);
        cudaFree(d_nnz);
        if (err != cudaSuccess) { spx_ell_destroy(e); return fail(SPX_ERR_CUDA, "encode: pack pass failed: %s", cudaGetErrorString(err)); }
        uint64_t tot = 0;
        for (uint32_t v : h) tot += v;
        e->nnz_total = tot;
        e->max_nnz = r;
        rc = set_row_order(e, h.data());
        if (rc != SPX_OK) { spx_ell_destroy(e); return rc; }
    }
    *out = e;
    return SPX_OK;
}

int decode_device(const spx_ell* e, float* dW, cudaStream_t s)
{
    if (e->m == 0 || e->n == 0) return SPX_OK;
    SPX_CUDA(cudaMemsetAsync(dW, 0, (size_t)e->m * e->n * sizeof(float), s));
    if (e->r == 0) return SPX_OK;
    decode_kernel<<<(e->m + kWarps - 1) / kWarps, kWarps * 32, 0, s>>>(e->Wd, e->idx, e->nnz, e->m, e->n, e->pitch, dW);
    SPX_LAUNCH_CHECK("decode_kernel");
    return SPX_OK;
}

int csr_to_ell_device(spx_ell* e, const uint64_t* d_rowptr, const uint32_t* d_col, const float* d_val,
                      cudaStream_t s)
{
    if (e->m == 0) return SPX_OK;
    csr_fill_kernel<<<(e->m + kWarps - 1) / kWarps, kWarps * 32, 0, s>>>(d_rowptr, d_col, d_val, e->m, e->pitch,
                                                                       e->Wd, e->idx, e->nnz);
    SPX_LAUNCH_CHECK("csr_fill_kernel");
    return SPX_OK;
}

}  // namespace spx
