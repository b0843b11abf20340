// abi.cu -- the extern "C" surface of libspx_b200.so (declared in include/spx_b200.h):
// error reporting, device memory / streams / events / graphs, ELLPACK handle life cycle,
// argument validation in front of every kernel launcher, and the host-buffer entry points
// that copy operands through pinned staging.
#include "common.cuh"

#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

namespace spx {

static thread_local char g_err[512] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count(int device)
{
    static std::mutex mu;
    static int cache[64];
    static bool have[64];
    if (device < 0 || device >= 64) return 148;
    std::lock_guard<std::mutex> lk(mu);
    if (!have[device]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) v = 148;
        cache[device] = v;
        have[device] = true;
    }
    return cache[device];
}

// The zero fill of the slabs is enqueued on `s`, the stream the caller fills them on afterwards:
// a non-blocking stream is not ordered behind work on the default stream.
int alloc_ell(uint32_t m, uint32_t n, uint32_t r, spx_ell** out, cudaStream_t s)
{
    spx_ell* e = new (std::nothrow) spx_ell();
    if (!e) return fail(SPX_ERR_OOM, "out of host memory");
    {
        cudaError_t derr = cudaGetDevice(&e->device);
        if (derr != cudaSuccess) {
            delete e;
            return fail(SPX_ERR_CUDA, "no usable CUDA device: %s", cudaGetErrorString(derr));
        }
    }
    e->m = m; e->n = n; e->r = r;
    e->pitch = r ? round_up<uint32_t>(r, 32u) : 0u;
    const size_t slots = (size_t)m * e->pitch;
    cudaError_t err = cudaSuccess;
    if (slots) {
        err = cudaMalloc(&e->Wd, slots * sizeof(float));
        if (err == cudaSuccess) err = cudaMalloc(&e->idx, slots * sizeof(uint32_t));
        // padding slots hold Wd = 0.0f, idx = 0 like the reference's (src/ellpack_encoder.cpp:25)
        if (err == cudaSuccess) err = cudaMemsetAsync(e->Wd, 0, slots * sizeof(float), s);
        if (err == cudaSuccess) err = cudaMemsetAsync(e->idx, 0, slots * sizeof(uint32_t), s);
    }
    if (err == cudaSuccess && m) err = cudaMalloc(&e->nnz, (size_t)m * sizeof(uint32_t));
    if (err == cudaSuccess && m) err = cudaMemsetAsync(e->nnz, 0, (size_t)m * sizeof(uint32_t), s);
    if (err != cudaSuccess) {
        cudaFree(e->Wd); cudaFree(e->idx); cudaFree(e->nnz);
        delete e;
        return fail(err == cudaErrorMemoryAllocation ? SPX_ERR_OOM : SPX_ERR_CUDA,
                    "ELLPACK device allocation (%zu slots) failed: %s", slots, cudaGetErrorString(err));
    }
    *out = e;
    return SPX_OK;
}

int set_row_order(spx_ell* e, const uint32_t* host_nnz)
{
    if (e->m == 0) return SPX_OK;
    // counting sort by row length, longest first; stable, so ties keep ascending row id
    std::vector<uint64_t> start((size_t)e->r + 2, 0);
    for (uint32_t i = 0; i < e->m; ++i) start[e->r - host_nnz[i] + 1]++;
    for (size_t k = 1; k < start.size(); ++k) start[k] += start[k - 1];
    std::vector<uint32_t> order(e->m);
    for (uint32_t i = 0; i < e->m; ++i) order[start[e->r - host_nnz[i]]++] = i;
    e->long_rows = 0;
    e->min_nnz = host_nnz[0];
    for (uint32_t i = 0; i < e->m; ++i) {
        e->long_rows += host_nnz[i] >= 512 ? 1u : 0u;
        e->min_nnz = std::min(e->min_nnz, host_nnz[i]);
    }
    if (!e->row_order) SPX_CUDA(cudaMalloc(&e->row_order, (size_t)e->m * sizeof(uint32_t)));
    SPX_CUDA(cudaMemcpy(e->row_order, order.data(), (size_t)e->m * sizeof(uint32_t), cudaMemcpyHostToDevice));
    return SPX_OK;
}

// Device scratch owned by a handle for the host-buffer entry points.
static int ensure_stage(spx_ell* e, size_t bytes)
{
    if (e->stage_dev_bytes >= bytes) return SPX_OK;
    if (e->stage_dev) cudaFree(e->stage_dev);
    e->stage_dev = nullptr;
    e->stage_dev_bytes = 0;
    SPX_CUDA(cudaMalloc(&e->stage_dev, bytes));
    e->stage_dev_bytes = bytes;
    return SPX_OK;
}

// Kernel entry points launch on the current device: a handle made on another GPU would hand the
// kernel pointers it cannot reach, so that is refused on the host.
int check_current_device(const spx_ell* e, const char* what)
{
    int cur = -1;
    SPX_CUDA(cudaGetDevice(&cur));
    if (cur != e->device)
        return fail(SPX_ERR_ARG, "%s: the handle lives on device %d but device %d is current", what, e->device, cur);
    return SPX_OK;
}

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
};

}  // namespace spx

using namespace spx;

extern "C" {

const char* spx_last_error(void) { return g_err; }
int spx_version(void) { return 100; }

int spx_device_count(int* count)
{
    if (!count) return fail(SPX_ERR_ARG, "count is null");
    SPX_CUDA(cudaGetDeviceCount(count));
    return SPX_OK;
}
int spx_set_device(int device) { SPX_CUDA(cudaSetDevice(device)); return SPX_OK; }
int spx_get_device(int* device)
{
    if (!device) return fail(SPX_ERR_ARG, "device is null");
    SPX_CUDA(cudaGetDevice(device));
    return SPX_OK;
}
int spx_device_sync(void) { SPX_CUDA(cudaDeviceSynchronize()); return SPX_OK; }
uint64_t spx_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// ---- memory / streams / events -----------------------------------------------------------
int spx_malloc(void** dptr, size_t bytes)
{
    if (!dptr) return fail(SPX_ERR_ARG, "dptr is null");
    *dptr = nullptr;
    if (bytes == 0) return SPX_OK;
    SPX_CUDA(cudaMalloc(dptr, bytes));
    return SPX_OK;
}
int spx_free(void* dptr) { if (dptr) SPX_CUDA(cudaFree(dptr)); return SPX_OK; }
int spx_host_alloc(void** hptr, size_t bytes)
{
    if (!hptr) return fail(SPX_ERR_ARG, "hptr is null");
    *hptr = nullptr;
    if (bytes == 0) return SPX_OK;
    SPX_CUDA(cudaMallocHost(hptr, bytes));
    return SPX_OK;
}
int spx_host_free(void* hptr) { if (hptr) SPX_CUDA(cudaFreeHost(hptr)); return SPX_OK; }
int spx_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream)
{
    if (bytes) SPX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return SPX_OK;
}
int spx_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream)
{
    if (bytes) SPX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return SPX_OK;
}
int spx_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream)
{
    if (bytes) SPX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return SPX_OK;
}
int spx_memset(void* dst, int value, size_t bytes, void* stream)
{
    if (bytes) SPX_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return SPX_OK;
}
int spx_stream_create(void** stream)
{
    if (!stream) return fail(SPX_ERR_ARG, "stream is null");
    cudaStream_t s;
    SPX_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return SPX_OK;
}
int spx_stream_destroy(void* stream) { if (stream) SPX_CUDA(cudaStreamDestroy((cudaStream_t)stream)); return SPX_OK; }
int spx_stream_sync(void* stream) { SPX_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); return SPX_OK; }
int spx_event_create(void** event)
{
    if (!event) return fail(SPX_ERR_ARG, "event is null");
    cudaEvent_t ev;
    SPX_CUDA(cudaEventCreate(&ev));
    *event = ev;
    return SPX_OK;
}
int spx_event_destroy(void* event) { if (event) SPX_CUDA(cudaEventDestroy((cudaEvent_t)event)); return SPX_OK; }
int spx_event_record(void* event, void* stream)
{
    SPX_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return SPX_OK;
}
int spx_event_elapsed_ms(void* start, void* stop, float* ms)
{
    if (!ms) return fail(SPX_ERR_ARG, "ms is null");
    SPX_CUDA(cudaEventSynchronize((cudaEvent_t)stop));
    SPX_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return SPX_OK;
}

// ---- graphs --------------------------------------------------------------------------------
// A captured graph remembers how many of this library's kernels it holds, so that replays keep
// spx_launch_count() truthful.
namespace {
struct GraphExec {
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;
};
thread_local uint64_t t_capture_start = 0;
}  // namespace

int spx_graph_capture_begin(void* stream)
{
    if (!stream) return fail(SPX_ERR_ARG, "graph capture needs a non-default stream");
    SPX_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    t_capture_start = g_launches.load(std::memory_order_relaxed);
    return SPX_OK;
}
int spx_graph_capture_end(void* stream, void** graph_exec)
{
    if (!graph_exec) return fail(SPX_ERR_ARG, "graph_exec is null");
    const uint64_t captured = g_launches.load(std::memory_order_relaxed) - t_capture_start;
    // launches made while capturing were recorded, not run: take them out of the running count
    g_launches.fetch_sub(captured, std::memory_order_relaxed);
    cudaGraph_t g = nullptr;
    SPX_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t ge = nullptr;
    cudaError_t err = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (err != cudaSuccess) return fail(SPX_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(err));
    GraphExec* h = new (std::nothrow) GraphExec();
    if (!h) { cudaGraphExecDestroy(ge); return fail(SPX_ERR_OOM, "out of host memory"); }
    h->exec = ge;
    h->kernels = captured;
    *graph_exec = h;
    return SPX_OK;
}
int spx_graph_launch(void* graph_exec, void* stream)
{
    if (!graph_exec) return fail(SPX_ERR_ARG, "graph_exec is null");
    GraphExec* h = static_cast<GraphExec*>(graph_exec);
    SPX_CUDA(cudaGraphLaunch(h->exec, (cudaStream_t)stream));
    count_launch(h->kernels);
    return SPX_OK;
}
int spx_graph_destroy(void* graph_exec)
{
    if (!graph_exec) return SPX_OK;
    GraphExec* h = static_cast<GraphExec*>(graph_exec);
    cudaError_t err = cudaGraphExecDestroy(h->exec);
    delete h;
    if (err != cudaSuccess) return fail(SPX_ERR_CUDA, "cudaGraphExecDestroy failed: %s", cudaGetErrorString(err));
    return SPX_OK;
}

// ---- ELLPACK handles -------------------------------------------------------------------------
int spx_ell_create(uint32_t m, uint32_t n, uint32_t r, const float* Wd, const uint32_t* idx,
                   const uint32_t* nnz, spx_ell** out)
{
    if (!out) return fail(SPX_ERR_ARG, "out is null");
    *out = nullptr;
    if (m && !nnz) return fail(SPX_ERR_ARG, "nnz is null");
    if ((size_t)m * r && (!Wd || !idx)) return fail(SPX_ERR_ARG, "Wd / idx is null");
    // Host-side validation in place of a device-side sanitizer: every stored column id must
    // be a valid row of X, every count must fit the slab.
    uint64_t total = 0;
    uint32_t longest = 0;
    bool ascending = true;
    for (uint32_t i = 0; i < m; ++i) {
        const uint32_t c = nnz[i];
        if (c > r) return fail(SPX_ERR_ARG, "nnz[%u] = %u exceeds r = %u", i, c, r);
        const uint32_t* row = idx + (size_t)i * r;
        for (uint32_t j = 0; j < c; ++j) {
            if (row[j] >= n) return fail(SPX_ERR_ARG, "idx[%u,%u] = %u is not below n = %u", i, j, row[j], n);
            if (j && row[j] <= row[j - 1]) ascending = false;
        }
        total += c;
        if (c > longest) longest = c;
    }
    spx_ell* e = nullptr;
    int rc = alloc_ell(m, n, r, &e, nullptr);
    if (rc != SPX_OK) return rc;
    e->nnz_total = total;
    e->max_nnz = longest;
    e->cols_ascending = ascending;
    cudaError_t err = cudaSuccess;
    if ((size_t)m * r) {
        err = cudaMemcpy2D(e->Wd, (size_t)e->pitch * 4, Wd, (size_t)r * 4, (size_t)r * 4, m, cudaMemcpyHostToDevice);
        if (err == cudaSuccess)
            err = cudaMemcpy2D(e->idx, (size_t)e->pitch * 4, idx, (size_t)r * 4, (size_t)r * 4, m, cudaMemcpyHostToDevice);
    }
    if (err == cudaSuccess && m) err = cudaMemcpy(e->nnz, nnz, (size_t)m * 4, cudaMemcpyHostToDevice);
    if (err != cudaSuccess) {
        spx_ell_destroy(e);
        return fail(SPX_ERR_CUDA, "ELLPACK upload failed: %s", cudaGetErrorString(err));
    }
    rc = set_row_order(e, nnz);
    if (rc != SPX_OK) { spx_ell_destroy(e); return rc; }
    *out = e;
    return SPX_OK;
}

int spx_ell_create_csr(uint32_t m, uint32_t n, const uint64_t* rowptr, const uint32_t* col,
                       const float* val, spx_ell** out)
{
    if (!out) return fail(SPX_ERR_ARG, "out is null");
    *out = nullptr;
    if (!rowptr) return fail(SPX_ERR_ARG, "rowptr is null");
    if (rowptr[0] != 0) return fail(SPX_ERR_ARG, "rowptr[0] must be 0");
    uint32_t r = 0;
    for (uint32_t i = 0; i < m; ++i) {
        if (rowptr[i + 1] < rowptr[i]) return fail(SPX_ERR_ARG, "rowptr is not non-decreasing at row %u", i);
        const uint64_t c = rowptr[i + 1] - rowptr[i];
        if (c > n) return fail(SPX_ERR_ARG, "row %u has more entries than columns", i);
        if (c > r) r = (uint32_t)c;
    }
    const uint64_t total = rowptr[m];
    if (total && (!col || !val)) return fail(SPX_ERR_ARG, "col / val is null");
    for (uint32_t i = 0; i < m; ++i)
        for (uint64_t j = rowptr[i]; j < rowptr[i + 1]; ++j) {
            if (col[j] >= n) return fail(SPX_ERR_ARG, "col[%llu] = %u is not below n = %u", (unsigned long long)j, col[j], n);
            if (j > rowptr[i] && col[j] <= col[j - 1])
                return fail(SPX_ERR_ARG, "columns of row %u are not strictly ascending", i);
        }
    spx_ell* e = nullptr;
    int rc = alloc_ell(m, n, r, &e, nullptr);
    if (rc != SPX_OK) return rc;
    e->nnz_total = total;
    e->max_nnz = r;
    if (m) {
        uint64_t* d_rowptr = nullptr; uint32_t* d_col = nullptr; float* d_val = nullptr;
        cudaError_t err = cudaMalloc(&d_rowptr, (size_t)(m + 1) * 8);
        if (err == cudaSuccess && total) err = cudaMalloc(&d_col, total * 4);
        if (err == cudaSuccess && total) err = cudaMalloc(&d_val, total * 4);
        if (err == cudaSuccess) err = cudaMemcpy(d_rowptr, rowptr, (size_t)(m + 1) * 8, cudaMemcpyHostToDevice);
        if (err == cudaSuccess && total) err = cudaMemcpy(d_col, col, total * 4, cudaMemcpyHostToDevice);
        if (err == cudaSuccess && total) err = cudaMemcpy(d_val, val, total * 4, cudaMemcpyHostToDevice);
        if (err == cudaSuccess) {
            rc = csr_to_ell_device(e, d_rowptr, d_col, d_val, nullptr);
            if (rc == SPX_OK) err = cudaDeviceSynchronize();
        }
        cudaFree(d_rowptr); cudaFree(d_col); cudaFree(d_val);
        if (err != cudaSuccess || rc != SPX_OK) {
            spx_ell_destroy(e);
            return rc != SPX_OK ? rc : fail(err == cudaErrorMemoryAllocation ? SPX_ERR_OOM : SPX_ERR_CUDA,
                                            "CSR upload failed: %s", cudaGetErrorString(err));
        }
        std::vector<uint32_t> counts(m);
        for (uint32_t i = 0; i < m; ++i) counts[i] = (uint32_t)(rowptr[i + 1] - rowptr[i]);
        rc = set_row_order(e, counts.data());
        if (rc != SPX_OK) { spx_ell_destroy(e); return rc; }
    }
    *out = e;
    return SPX_OK;
}

int spx_ell_encode_device(const float* dW, uint32_t m, uint32_t n, void* stream, spx_ell** out)
{
    if (!out) return fail(SPX_ERR_ARG, "out is null");
    *out = nullptr;
    if ((size_t)m * n && !dW) return fail(SPX_ERR_ARG, "dW is null");
    return encode_device(dW, m, n, (cudaStream_t)stream, out);
}

int spx_ell_destroy(spx_ell* e)
{
    if (!e) return SPX_OK;
    DeviceGuard g(e->device);
    for (uint32_t k = 0; k < e->nslices; ++k) spx_ell_destroy(e->slices[k]);
    e->nslices = 0;
    if (e->view) e->Wd = nullptr, e->idx = nullptr, e->nnz = nullptr;      // the parent's arrays
    for (cudaStream_t st : e->xchg_streams) if (st) cudaStreamDestroy(st);
    for (cudaEvent_t ev : e->xchg_events) if (ev) cudaEventDestroy(ev);
    cudaFree(e->Wd); cudaFree(e->idx); cudaFree(e->nnz); cudaFree(e->row_order); cudaFree(e->taps); cudaFree(e->spmv_split); cudaFree(e->rbm_hdr); cudaFree(e->rbm_w); cudaFree(e->rbm_ncols); cudaFree(e->stage_dev); cudaFree(e->conv_scratch); cudaFree(e->fm_scratch);
    if (e->tma_failed_host) cudaFreeHost(e->tma_failed_host);
    if (e->tma_failed_dev) cudaFree(e->tma_failed_dev);
    for (cudaStream_t st : e->pipe_streams) if (st) cudaStreamDestroy(st);
    for (cudaEvent_t ev : e->pipe_events) if (ev) cudaEventDestroy(ev);
    delete e;
    return SPX_OK;
}

int spx_ell_dims(const spx_ell* e, uint32_t* m, uint32_t* n, uint32_t* r, uint64_t* nnz_total)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (m) *m = e->m;
    if (n) *n = e->n;
    if (r) *r = e->r;
    if (nnz_total) *nnz_total = e->nnz_total;
    return SPX_OK;
}

int spx_ell_download(const spx_ell* e, float* Wd, uint32_t* idx, uint32_t* nnz)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    DeviceGuard g(e->device);
    const size_t rb = (size_t)e->r * 4;
    if ((size_t)e->m * e->r) {
        if (Wd) SPX_CUDA(cudaMemcpy2D(Wd, rb, e->Wd, (size_t)e->pitch * 4, rb, e->m, cudaMemcpyDeviceToHost));
        if (idx) SPX_CUDA(cudaMemcpy2D(idx, rb, e->idx, (size_t)e->pitch * 4, rb, e->m, cudaMemcpyDeviceToHost));
    }
    if (nnz && e->m) SPX_CUDA(cudaMemcpy(nnz, e->nnz, (size_t)e->m * 4, cudaMemcpyDeviceToHost));
    return SPX_OK;
}

int spx_ell_decode_device(const spx_ell* e, float* dW, void* stream)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if ((size_t)e->m * e->n && !dW) return fail(SPX_ERR_ARG, "dW is null");
    return decode_device(e, dW, (cudaStream_t)stream);
}

// ---- kernels ---------------------------------------------------------------------------------
int spx_spmm(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias,
             int act, float* Y, uint64_t ldy, void* stream)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (act < SPX_ACT_NONE || act > SPX_ACT_TANH) return fail(SPX_ERR_ARG, "unknown activation %d", act);
    if (e->m == 0 || C == 0) return SPX_OK;
    if (ldx < C || ldy < C) return fail(SPX_ERR_ARG, "leading dimension smaller than C");
    if (!Y) return fail(SPX_ERR_ARG, "Y is null");
    if (!X && e->nnz_total) return fail(SPX_ERR_ARG, "X is null");
    if (int rc = check_current_device(e, "spmm")) return rc;
    return launch_spmm(e, X, C, ldx, bias, act, Y, ldy, (cudaStream_t)stream);
}

int spx_spmm_bcast(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                   float* const* Ys, uint32_t nbuffers, uint64_t row_offset, uint64_t ldy, void* stream)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (act < SPX_ACT_NONE || act > SPX_ACT_TANH) return fail(SPX_ERR_ARG, "unknown activation %d", act);
    if (!Ys) return fail(SPX_ERR_ARG, "destination list is null");
    if (e->m == 0 || C == 0) return SPX_OK;
    if (ldx < C || ldy < C) return fail(SPX_ERR_ARG, "leading dimension smaller than C");
    if (!X && e->nnz_total) return fail(SPX_ERR_ARG, "X is null");
    if (int rc = check_current_device(e, "spmm_bcast")) return rc;
    return launch_spmm_bcast(e, X, C, ldx, bias, act, Ys, nbuffers, row_offset, ldy, (cudaStream_t)stream);
}

// Cuts the handle's rows into `want` contiguous ranges of near-equal cost (stored entries + 8 per
// row) and makes a view handle with its own row schedule for each.
static int ensure_slices(spx_ell* e, uint32_t want)
{
    if (e->nslices == want) return SPX_OK;
    for (uint32_t k = 0; k < e->nslices; ++k) spx_ell_destroy(e->slices[k]);
    e->nslices = 0;
    std::vector<uint32_t> nnz(e->m);
    SPX_CUDA(cudaMemcpy(nnz.data(), e->nnz, (size_t)e->m * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    uint64_t total = 0;
    for (uint32_t i = 0; i < e->m; ++i) total += nnz[i] + 8u;
    uint32_t r0 = 0;
    uint64_t acc = 0;
    for (uint32_t k = 0; k < want; ++k) {
        const uint64_t target = total * (k + 1) / want;
        uint32_t r1 = r0;
        while (r1 < e->m && (acc < target || k + 1 == want)) acc += nnz[r1++] + 8u;
        spx_ell* v = new spx_ell();
        v->device = e->device;
        v->view = true;
        v->m = r1 - r0; v->n = e->n; v->r = e->r; v->pitch = e->pitch;
        v->Wd = e->Wd + (size_t)r0 * e->pitch;
        v->idx = e->idx + (size_t)r0 * e->pitch;
        v->nnz = e->nnz + r0;
        v->cols_ascending = e->cols_ascending;
        for (uint32_t i = r0; i < r1; ++i) {
            v->nnz_total += nnz[i];
            v->max_nnz = std::max(v->max_nnz, nnz[i]);
        }
        e->slices[k] = v;
        e->slice_row0[k] = r0;
        e->nslices = k + 1;
        if (int rc = set_row_order(v, nnz.data() + r0)) return rc;
        r0 = r1;
    }
    e->slice_row0[want] = e->m;
    return SPX_OK;
}

int spx_spmm_exchange(const spx_ell* ce, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                      float* const* Ys, uint32_t nbuffers, uint32_t self, uint64_t row_offset, uint64_t ldy,
                      uint32_t slices, void* stream)
{
    if (!ce) return fail(SPX_ERR_ARG, "handle is null");
    if (act < SPX_ACT_NONE || act > SPX_ACT_TANH) return fail(SPX_ERR_ARG, "unknown activation %d", act);
    if (!Ys) return fail(SPX_ERR_ARG, "destination list is null");
    if (nbuffers == 0 || nbuffers > 8 || self >= nbuffers) return fail(SPX_ERR_ARG, "spmm_exchange: 1..8 buffers, self among them");
    for (uint32_t g = 0; g < nbuffers; ++g)
        if (!Ys[g]) return fail(SPX_ERR_ARG, "spmm_exchange: destination %u is null", g);
    if (slices == 0) slices = 4;
    if (slices > 16) return fail(SPX_ERR_LIMIT, "spmm_exchange: at most 16 slices");
    if (ce->m == 0 || C == 0) return SPX_OK;
    if (ldx < C || ldy < C) return fail(SPX_ERR_ARG, "leading dimension smaller than C");
    if (!X && ce->nnz_total) return fail(SPX_ERR_ARG, "X is null");
    if (int rc = check_current_device(ce, "spmm_exchange")) return rc;
    spx_ell* e = const_cast<spx_ell*>(ce);
    slices = std::min(slices, e->m);
    if (int rc = ensure_slices(e, slices)) return rc;
    for (cudaStream_t& st : e->xchg_streams)
        if (!st) SPX_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    for (cudaEvent_t& ev : e->xchg_events)
        if (!ev) SPX_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaStream_t s = (cudaStream_t)stream;
    float* own = Ys[self];
    for (uint32_t k = 0; k < slices; ++k) {
        const spx_ell* v = e->slices[k];
        if (v->m == 0) continue;
        const uint32_t r0 = e->slice_row0[k];
        const size_t at = (size_t)(row_offset + r0) * ldy;
        if (int rc = launch_spmm(v, X, C, ldx, bias ? bias + r0 : nullptr, act, own + at, ldy, s)) return rc;
        if (nbuffers == 1) continue;
        // the slice is final: hand it to the copy engines, one stream per peer modulo 4
        SPX_CUDA(cudaEventRecord(e->xchg_events[k], s));
        for (uint32_t g = 0; g < nbuffers; ++g) {
            if (g == self) continue;
            cudaStream_t cs = e->xchg_streams[g % 4];
            SPX_CUDA(cudaStreamWaitEvent(cs, e->xchg_events[k], 0));
            if (ldy == C)
                SPX_CUDA(cudaMemcpyAsync(Ys[g] + at, own + at, (size_t)v->m * C * sizeof(float), cudaMemcpyDeviceToDevice, cs));
            else
                SPX_CUDA(cudaMemcpy2DAsync(Ys[g] + at, ldy * sizeof(float), own + at, ldy * sizeof(float), (size_t)C * sizeof(float),
                                           v->m, cudaMemcpyDeviceToDevice, cs));
        }
    }
    if (nbuffers > 1)
        for (int i = 0; i < 4; ++i) {           // the caller's stream continues when every copy is done
            SPX_CUDA(cudaEventRecord(e->xchg_events[16 + i], e->xchg_streams[i]));
            SPX_CUDA(cudaStreamWaitEvent(s, e->xchg_events[16 + i], 0));
        }
    return SPX_OK;
}

int spx_spmm_mcast(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                   float* Ymc, uint64_t row_offset, uint64_t ldy, void* stream)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (act < SPX_ACT_NONE || act > SPX_ACT_TANH) return fail(SPX_ERR_ARG, "unknown activation %d", act);
    if (!Ymc) return fail(SPX_ERR_ARG, "multicast address is null");
    if (e->m == 0 || C == 0) return SPX_OK;
    if (ldx < C || ldy < C) return fail(SPX_ERR_ARG, "leading dimension smaller than C");
    if (!X && e->nnz_total) return fail(SPX_ERR_ARG, "X is null");
    // multimem.st needs naturally aligned 16-byte vectors: the library's scalar kernels would store
    // single floats, which a multicast mapping also takes, but every shape is kept on one rule
    if (C % 4 || ldx % 4 || ldy % 4 || (reinterpret_cast<uintptr_t>(Ymc) & 15) || (reinterpret_cast<uintptr_t>(X) & 15))
        return fail(SPX_ERR_ARG, "spmm_mcast: C, ldx and ldy must be multiples of 4 and X, Ymc 16-byte aligned");
    if (int rc = check_current_device(e, "spmm_mcast")) return rc;
    float* one[1] = { Ymc };
    return launch_spmm_bcast(e, X, C, ldx, bias, act, one, 1, row_offset, ldy, (cudaStream_t)stream, true);
}

int spx_ipc_export(void* dptr, char handle[SPX_IPC_HANDLE_BYTES])
{
    static_assert(sizeof(cudaIpcMemHandle_t) == SPX_IPC_HANDLE_BYTES, "IPC handle size");
    if (!dptr || !handle) return fail(SPX_ERR_ARG, "null argument");
    cudaIpcMemHandle_t h;
    SPX_CUDA(cudaIpcGetMemHandle(&h, dptr));
    memcpy(handle, &h, sizeof(h));
    return SPX_OK;
}

int spx_ipc_open(const char handle[SPX_IPC_HANDLE_BYTES], void** dptr)
{
    if (!dptr || !handle) return fail(SPX_ERR_ARG, "null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    SPX_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return SPX_OK;
}

int spx_ipc_close(void* dptr)
{
    if (dptr) SPX_CUDA(cudaIpcCloseMemHandle(dptr));
    return SPX_OK;
}

int spx_spmv(const spx_ell* e, const float* x, const float* bias, float* y, void* stream)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (e->m == 0) return SPX_OK;
    if (!y) return fail(SPX_ERR_ARG, "y is null");
    if (!x && e->n) return fail(SPX_ERR_ARG, "x is null");   // the kernels stage all of x before any row
    if (int rc = check_current_device(e, "spmv")) return rc;
    return launch_spmv(const_cast<spx_ell*>(e), x, bias, y, (cudaStream_t)stream);
}

int spx_spmv_reference_order(const spx_ell* e, const float* x, const float* bias, float* y, void* stream)
{
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (e->m == 0) return SPX_OK;
    if (!y) return fail(SPX_ERR_ARG, "y is null");
    if (!x && e->n) return fail(SPX_ERR_ARG, "x is null");
    if (int rc = check_current_device(e, "spmv_reference_order")) return rc;
    return launch_spmv_reforder(e, x, bias, y, (cudaStream_t)stream);
}

int spx_conv2d(const spx_ell* e, const spx_conv_geom* g, int layout, const float* in, uint32_t B,
               const float* bias, int act, float* out, void* stream)
{
    if (!e || !g) return fail(SPX_ERR_ARG, "handle / geometry is null");
    if (layout != SPX_LAYOUT_PF && layout != SPX_LAYOUT_NCHW && layout != SPX_LAYOUT_FMAJOR)
        return fail(SPX_ERR_ARG, "unknown layout %d", layout);
    if (act < SPX_ACT_NONE || act > SPX_ACT_TANH) return fail(SPX_ERR_ARG, "unknown activation %d", act);
    if (g->sH == 0 || g->sW == 0 || g->dH == 0 || g->dW == 0 || g->kH == 0 || g->kW == 0)
        return fail(SPX_ERR_ARG, "stride, dilation and kernel extent must be positive");
    if (e->m != g->Cout) return fail(SPX_ERR_ARG, "ELLPACK rows (%u) != Cout (%u)", e->m, g->Cout);
    if ((uint64_t)g->Cin * g->kH * g->kW != e->n)
        return fail(SPX_ERR_ARG, "ELLPACK columns (%u) != Cin*kH*kW", e->n);
    const uint32_t eh = g->dH * (g->kH - 1) + 1, ew = g->dW * (g->kW - 1) + 1;
    if (g->H + 2 * g->pH < eh || g->W + 2 * g->pW < ew) return fail(SPX_ERR_ARG, "kernel larger than padded input");
    if (g->Ho != (g->H + 2 * g->pH - eh) / g->sH + 1 || g->Wo != (g->W + 2 * g->pW - ew) / g->sW + 1)
        return fail(SPX_ERR_ARG, "Ho / Wo inconsistent with the geometry");
    if (B == 0 || e->m == 0) return SPX_OK;
    if (!in || !out) return fail(SPX_ERR_ARG, "in / out is null");
    if (int rc = check_current_device(e, "conv2d")) return rc;
    return launch_conv2d(const_cast<spx_ell*>(e), g, layout, in, B, bias, act, out, (cudaStream_t)stream);
}

int spx_eltwise(int op, const float* a, const float* b, float* out, uint64_t count, void* stream)
{
    if (op < SPX_OP_RELU || op > SPX_OP_ADD) return fail(SPX_ERR_ARG, "unknown elementwise op %d", op);
    if (count == 0) return SPX_OK;
    if (!a || !out || (op == SPX_OP_ADD && !b)) return fail(SPX_ERR_ARG, "null operand");
    return launch_eltwise(op, a, b, out, count, (cudaStream_t)stream);
}

// Column panels of the pipelined host-buffer SpMM: 256 columns, except that a wide operand starts
// with a panel of 64 (then 192, back on the 256 grid): the first copy out can only begin after
// the first panel has been copied in and multiplied, and that lead time is not overlapped with
// anything, so the first panel is kept small.
static inline uint32_t host_panel_width(uint32_t c0, uint32_t C)
{
    if (C >= 512) {
        if (c0 == 0) return 64;
        if (c0 == 64) return 192;
    }
    return std::min<uint32_t>(256, C - c0);
}

// ---- host-buffer entry points ----------------------------------------------------------------
// Pageable host buffers are copied by the driver through its own pinned bounce buffers; callers
// that pass pinned memory (spx_host_alloc) get direct DMA.  Layout of the staging block:
// [X | bias | Y], each part 256-byte aligned.
int spx_spmm_host(const spx_ell* ce, const float* X, uint32_t C, const float* bias, int act, float* Y)
{
    spx_ell* e = const_cast<spx_ell*>(ce);
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (e->m == 0 || C == 0) return SPX_OK;
    if (!Y || (!X && e->n)) return fail(SPX_ERR_ARG, "X / Y is null");
    DeviceGuard g(e->device);
    const size_t xb = round_up<size_t>((size_t)e->n * C * 4, 256);
    const size_t bb = round_up<size_t>((size_t)e->m * 4, 256);
    const size_t yb = round_up<size_t>((size_t)e->m * C * 4, 256);
    int rc = ensure_stage(e, xb + bb + yb);
    if (rc != SPX_OK) return rc;
    char* base = static_cast<char*>(e->stage_dev);
    float* dX = reinterpret_cast<float*>(base);
    float* dB = reinterpret_cast<float*>(base + xb);
    float* dY = reinterpret_cast<float*>(base + xb + bb);
    // Large, wide operands: the copies dominate (PCIe), so the call is pipelined over 256-column
    // panels on three streams -- panel p+1 is copied in and panel p-1 copied out while panel p is
    // multiplied (strided 2-D copies, 1 KiB per row).  Results are unchanged: a panel is exactly
    // what one pass of the kernel computes anyway.
    if (C >= 512 && C % 4 == 0 && (size_t)e->m * C * 4 >= ((size_t)64 << 20) && e->n) {
        for (cudaStream_t& st : e->pipe_streams)
            if (!st) SPX_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
        cudaStream_t s_in = e->pipe_streams[0], s_mm = e->pipe_streams[2], s_out = e->pipe_streams[3];
        for (int i = 0; i < 2; ++i)
            if (!e->pipe_events[i]) SPX_CUDA(cudaEventCreate(&e->pipe_events[i]));
        cudaEvent_t ev_in = e->pipe_events[0], ev_mm = e->pipe_events[1];
        cudaError_t err = cudaSuccess;
        if (bias) err = cudaMemcpyAsync(dB, bias, (size_t)e->m * 4, cudaMemcpyHostToDevice, s_in);
        for (uint32_t c0 = 0, w = 0; c0 < C && err == cudaSuccess && rc == SPX_OK; c0 += w) {
            w = host_panel_width(c0, C);
            err = cudaMemcpy2DAsync(dX + c0, (size_t)C * 4, X + c0, (size_t)C * 4, (size_t)w * 4, e->n, cudaMemcpyHostToDevice, s_in);
            if (err == cudaSuccess) err = cudaEventRecord(ev_in, s_in);
            if (err == cudaSuccess) err = cudaStreamWaitEvent(s_mm, ev_in, 0);
            if (err != cudaSuccess) break;
            rc = spx_spmm(e, dX + c0, w, C, bias ? dB : nullptr, act, dY + c0, C, s_mm);
            if (rc != SPX_OK) break;
            err = cudaEventRecord(ev_mm, s_mm);
            if (err == cudaSuccess) err = cudaStreamWaitEvent(s_out, ev_mm, 0);
            if (err == cudaSuccess)
                err = cudaMemcpy2DAsync(Y + c0, (size_t)C * 4, dY + c0, (size_t)C * 4, (size_t)w * 4, e->m, cudaMemcpyDeviceToHost, s_out);
        }
        if (err == cudaSuccess) err = cudaStreamSynchronize(s_out);
        // on an error the earlier streams may still be busy: drain them before the staging is reused
        cudaStreamSynchronize(s_in);
        cudaStreamSynchronize(s_mm);
        if (rc != SPX_OK) return rc;
        if (err != cudaSuccess) return fail(SPX_ERR_CUDA, "spmm_host: pipelined copy failed: %s", cudaGetErrorString(err));
        return SPX_OK;
    }
    if (e->n) SPX_CUDA(cudaMemcpyAsync(dX, X, (size_t)e->n * C * 4, cudaMemcpyHostToDevice, nullptr));
    if (bias) SPX_CUDA(cudaMemcpyAsync(dB, bias, (size_t)e->m * 4, cudaMemcpyHostToDevice, nullptr));
    rc = spx_spmm(e, dX, C, C, bias ? dB : nullptr, act, dY, C, nullptr);
    if (rc != SPX_OK) return rc;
    SPX_CUDA(cudaMemcpyAsync(Y, dY, (size_t)e->m * C * 4, cudaMemcpyDeviceToHost, nullptr));
    SPX_CUDA(cudaStreamSynchronize(nullptr));
    return SPX_OK;
}

// Row-sharded SpMM on host buffers, one process per GPU.  Every rank holds the same host X but
// copies only its own block of X's rows over PCIe; the ranks rebuild the replicated X on the
// devices with in-place all-gathers over NVLink, multiply their rows of E and copy their own rows
// of Y back.  The device copy of X is kept panel-major -- panel p is a contiguous
// [rows_per_rank * world x width] matrix -- so that a rank's block of a panel is one contiguous
// slab (what the all-gather wants) and the multiply of panel p can start while panel p+1 is still
// on its way: four streams (copy in, exchange, multiply, copy out) chained by events per panel.
int spx_spmm_host_sharded(spx_comm* comm, const spx_ell* ce, const float* X, uint32_t C, const float* bias, int act,
                          float* Y, float* phase_ms)
{
    spx_ell* e = const_cast<spx_ell*>(ce);
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    int rank = 0, world = 1;
    if (comm) { int rc = spx_comm_info(comm, &rank, &world); if (rc != SPX_OK) return rc; }
    if (phase_ms) phase_ms[0] = phase_ms[1] = phase_ms[2] = phase_ms[3] = 0.0f;
    if (!comm || world == 1) return spx_spmm_host(ce, X, C, bias, act, Y);
    if (C == 0) return SPX_OK;                       // nothing to exchange either: every rank returns here
    if ((!Y && e->m) || (!X && e->n)) return fail(SPX_ERR_ARG, "X / Y is null");
    DeviceGuard g(e->device);
    uint32_t panels = 0;
    for (uint32_t c0 = 0; c0 < C; c0 += host_panel_width(c0, C)) ++panels;
    constexpr uint32_t kMaxPanels = sizeof(e->pipe_events) / sizeof(e->pipe_events[0]) / 8;    // 2 events x 4 stages each
    if (panels > kMaxPanels) return fail(SPX_ERR_LIMIT, "spmm_host_sharded: C beyond %u columns", (kMaxPanels - 1) * 256);
    const uint64_t per = ((uint64_t)e->n + world - 1) / world;       // rows of X per rank (last block may be short)
    const uint64_t lo = std::min<uint64_t>(e->n, per * rank), hi = std::min<uint64_t>(e->n, lo + per);
    const size_t xb = round_up<size_t>((size_t)per * world * C * 4, 256);
    const size_t bb = round_up<size_t>((size_t)e->m * 4 + 4, 256);
    const size_t yb = round_up<size_t>((size_t)e->m * C * 4 + 4, 256);
    int rc = ensure_stage(e, xb + bb + yb);
    if (rc != SPX_OK) return rc;
    char* base = static_cast<char*>(e->stage_dev);
    float* dX = reinterpret_cast<float*>(base);
    float* dB = reinterpret_cast<float*>(base + xb);
    float* dY = reinterpret_cast<float*>(base + xb + bb);
    // The exchange stream gets the highest priority: the all-gather of panel p+1 runs next to the
    // multiply of panel p, and its few CTAs must not queue behind the multiply's thousands.
    int prio_lo = 0, prio_hi = 0;
    SPX_CUDA(cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi));
    for (int i = 0; i < 4; ++i)
        if (!e->pipe_streams[i])
            SPX_CUDA(cudaStreamCreateWithPriority(&e->pipe_streams[i], cudaStreamNonBlocking, i == 1 ? prio_hi : prio_lo));
    for (uint32_t i = 0; i < panels * 8; ++i)
        if (!e->pipe_events[i]) SPX_CUDA(cudaEventCreate(&e->pipe_events[i]));
    cudaStream_t st[4] = {e->pipe_streams[0], e->pipe_streams[1], e->pipe_streams[2], e->pipe_streams[3]};
    auto ev = [&](uint32_t panel, int phase, int end) { return e->pipe_events[(panel * 4 + phase) * 2 + end]; };

    cudaError_t err = cudaSuccess;
    if (bias && e->m) err = cudaMemcpyAsync(dB, bias, (size_t)e->m * 4, cudaMemcpyHostToDevice, st[0]);
    for (uint32_t p = 0, c0 = 0, w = 0; p < panels && err == cudaSuccess && rc == SPX_OK; ++p, c0 += w) {
        w = host_panel_width(c0, C);
        float* dXp = dX + (size_t)per * world * c0;                   // panel p: [per * world x w], contiguous
        // 0: this rank's rows of the panel, host -> device
        err = cudaEventRecord(ev(p, 0, 0), st[0]);
        if (err == cudaSuccess && hi > lo)
            err = cudaMemcpy2DAsync(dXp + lo * w, (size_t)w * 4, X + lo * C + c0, (size_t)C * 4, (size_t)w * 4, hi - lo,
                                    cudaMemcpyHostToDevice, st[0]);
        if (err == cudaSuccess) err = cudaEventRecord(ev(p, 0, 1), st[0]);
        // 1: all ranks' rows of the panel, over NVLink
        if (err == cudaSuccess) err = cudaStreamWaitEvent(st[1], ev(p, 0, 1), 0);
        if (err == cudaSuccess) err = cudaEventRecord(ev(p, 1, 0), st[1]);
        if (err != cudaSuccess) break;
        rc = spx_allgather_rows(comm, dXp, per, w, st[1]);
        if (rc != SPX_OK) break;
        err = cudaEventRecord(ev(p, 1, 1), st[1]);
        // 2: multiply
        if (err == cudaSuccess) err = cudaStreamWaitEvent(st[2], ev(p, 1, 1), 0);
        if (err == cudaSuccess) err = cudaEventRecord(ev(p, 2, 0), st[2]);
        if (err != cudaSuccess) break;
        if (e->m) rc = spx_spmm(e, dXp, w, w, bias ? dB : nullptr, act, dY + c0, C, st[2]);
        if (rc != SPX_OK) break;
        err = cudaEventRecord(ev(p, 2, 1), st[2]);
        // 3: this rank's rows of Y, device -> host
        if (err == cudaSuccess) err = cudaStreamWaitEvent(st[3], ev(p, 2, 1), 0);
        if (err == cudaSuccess) err = cudaEventRecord(ev(p, 3, 0), st[3]);
        if (err == cudaSuccess && e->m)
            err = cudaMemcpy2DAsync(Y + c0, (size_t)C * 4, dY + c0, (size_t)C * 4, (size_t)w * 4, e->m, cudaMemcpyDeviceToHost, st[3]);
        if (err == cudaSuccess) err = cudaEventRecord(ev(p, 3, 1), st[3]);
    }
    // drain every stream (also after an error: the staging is reused by the next call)
    for (int i = 3; i >= 0; --i) {
        cudaError_t e2 = cudaStreamSynchronize(st[i]);
        if (err == cudaSuccess) err = e2;
    }
    if (rc != SPX_OK) return rc;
    if (err != cudaSuccess) return fail(SPX_ERR_CUDA, "spmm_host_sharded: %s", cudaGetErrorString(err));
    if (phase_ms)
        for (uint32_t p = 0; p < panels; ++p)
            for (int ph = 0; ph < 4; ++ph) {
                float ms = 0.0f;
                if (cudaEventElapsedTime(&ms, ev(p, ph, 0), ev(p, ph, 1)) == cudaSuccess) phase_ms[ph] += ms;
            }
    return SPX_OK;
}

int spx_spmv_host(const spx_ell* ce, const float* x, const float* bias, float* y)
{
    spx_ell* e = const_cast<spx_ell*>(ce);
    if (!e) return fail(SPX_ERR_ARG, "handle is null");
    if (e->m == 0) return SPX_OK;
    if (!y || (!x && e->n)) return fail(SPX_ERR_ARG, "x / y is null");
    DeviceGuard g(e->device);
    const size_t xb = round_up<size_t>((size_t)e->n * 4, 256);
    const size_t bb = round_up<size_t>((size_t)e->m * 4, 256);
    int rc = ensure_stage(e, xb + 2 * bb);
    if (rc != SPX_OK) return rc;
    char* base = static_cast<char*>(e->stage_dev);
    float* dx = reinterpret_cast<float*>(base);
    float* dB = reinterpret_cast<float*>(base + xb);
    float* dy = reinterpret_cast<float*>(base + xb + bb);
    if (e->n) SPX_CUDA(cudaMemcpyAsync(dx, x, (size_t)e->n * 4, cudaMemcpyHostToDevice, nullptr));
    if (bias) SPX_CUDA(cudaMemcpyAsync(dB, bias, (size_t)e->m * 4, cudaMemcpyHostToDevice, nullptr));
    rc = spx_spmv(e, dx, bias ? dB : nullptr, dy, nullptr);
    if (rc != SPX_OK) return rc;
    SPX_CUDA(cudaMemcpyAsync(y, dy, (size_t)e->m * 4, cudaMemcpyDeviceToHost, nullptr));
    SPX_CUDA(cudaStreamSynchronize(nullptr));
    return SPX_OK;
}

}  // extern "C"
