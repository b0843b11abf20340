// ellpack.cpp -- see ellpack.hpp.
#include "ellpack.hpp"

#include <algorithm>
#include <cstring>
#include <string>
#include <thread>

namespace spx {

void check(int status, const char* what)
{
    if (status == SPX_OK) return;
    if (status == SPX_ERR_OOM) throw std::bad_alloc();
    throw std::runtime_error(std::string(what) + ": " + spx_last_error());
}

Ellpack::~Ellpack() { spx_ell_destroy(dev); }

Ellpack::Ellpack(Ellpack&& o) noexcept
    : m(o.m), n(o.n), r(o.r), Wd(std::move(o.Wd)), idx(std::move(o.idx)), nnz(std::move(o.nnz)),
      dev(o.dev), last_x(std::move(o.last_x))
{
    o.dev = nullptr;
}

Ellpack& Ellpack::operator=(Ellpack&& o) noexcept
{
    if (this != &o) {
        spx_ell_destroy(dev);
        m = o.m; n = o.n; r = o.r;
        Wd = std::move(o.Wd); idx = std::move(o.idx); nnz = std::move(o.nnz);
        dev = o.dev; o.dev = nullptr;
        last_x = std::move(o.last_x);
    }
    return *this;
}

void Ellpack::upload()
{
    spx_ell_destroy(dev);
    dev = nullptr;
    check(spx_ell_create(m, n, r, Wd.ptr, idx.data(), nnz.data(), &dev), "ELLPACK upload");
}

std::vector<float> Ellpack::gathered_x() const
{
    std::vector<float> xt(size_t(m) * r, 0.0f);
    if (last_x.size() == n)
        for (size_t s = 0; s < xt.size(); ++s) xt[s] = last_x[idx[s]];
    return xt;
}

uint64_t Ellpack::nnz_total() const
{
    uint64_t t = 0;
    for (uint32_t c : nnz) t += c;
    return t;
}

Ellpack Ellpack::shard_range(uint32_t lo, uint32_t hi, bool do_upload) const
{
    if (lo > hi || hi > m) throw std::runtime_error("shard_range: bad row range");
    Ellpack S(hi - lo, n, r);
    if (S.m && r) {
        std::memcpy(S.Wd.ptr, Wd.ptr + size_t(lo) * r, size_t(S.m) * r * sizeof(float));
        std::memcpy(S.idx.data(), idx.data() + size_t(lo) * r, size_t(S.m) * r * sizeof(uint32_t));
    }
    std::copy(nnz.begin() + lo, nnz.begin() + hi, S.nnz.begin());
    if (do_upload) S.upload();
    return S;
}

Ellpack Ellpack::shard_rows(uint32_t g, uint32_t G, bool do_upload) const
{
    if (G == 0 || g >= G) throw std::runtime_error("shard_rows: bad shard index");
    const uint32_t per = (m + G - 1) / G;
    const uint32_t lo = std::min(m, g * per);
    return shard_range(lo, std::min(m, lo + per), do_upload);
}

// Contiguous row ranges of near-equal work: a row costs its stored entries plus `row_cost` (the
// fixed part: its output row and its slot in the schedule), and bound g is placed where the running
// cost is closest to g/G of the total.  Equal row counts are right for iid rows; when the
// long rows cluster (sorted or banded matrices) they leave one rank with most of the nonzeros.
std::vector<uint32_t> Ellpack::balanced_row_split(uint32_t G, uint32_t row_cost) const
{
    if (G == 0) throw std::runtime_error("balanced_row_split: need at least one shard");
    std::vector<uint32_t> bounds(size_t(G) + 1, m);
    bounds[0] = 0;
    uint64_t total = 0;
    for (uint32_t c : nnz) total += uint64_t(c) + row_cost;
    uint64_t run = 0;
    uint32_t g = 1;
    for (uint32_t i = 0; i < m && g < G; ++i) {
        // close shard g-1 in front of row i when that leaves the running cost closer to g/G of the
        // total than taking row i as well would: g*total - G*run <= G*(run + cost_i) - g*total
        const uint64_t cost = uint64_t(nnz[i]) + row_cost;
        while (g < G && 2 * uint64_t(g) * total <= uint64_t(G) * (2 * run + cost)) bounds[g++] = i;
        run += cost;
    }
    return bounds;
}

namespace {

// Runs fn(lo, hi) over [0, m) on a few host threads (rows are independent).
template <class F>
void parallel_rows(uint32_t m, size_t work_per_row, F fn)
{
    unsigned hw = std::thread::hardware_concurrency();
    unsigned nt = hw ? std::min(hw, 16u) : 1u;
    if (size_t(m) * work_per_row < (size_t(1) << 20) || m < nt * 4) nt = 1;
    if (nt <= 1) { fn(0u, m); return; }
    std::vector<std::thread> th;
    const uint32_t per = (m + nt - 1) / nt;
    for (unsigned t = 0; t < nt; ++t) {
        const uint32_t lo = std::min(m, t * per), hi = std::min(m, lo + per);
        if (lo < hi) th.emplace_back(fn, lo, hi);
    }
    for (auto& t : th) t.join();
}

}  // namespace

// Same two passes as the reference encoder (src/ellpack_encoder.cpp:8-41): count entries with
// v != 0.0f per row (drops -0.0f, keeps NaN / inf / denormals), r = the largest count, then pack
// values and column ids in ascending column order; padding slots stay Wd = 0.0f, idx = 0.
Ellpack encode_host(const float* W, uint32_t m, uint32_t n)
{
    std::vector<uint32_t> counts(m);
    parallel_rows(m, n, [&](uint32_t lo, uint32_t hi) {
        for (uint32_t i = lo; i < hi; ++i) {
            const float* row = W + size_t(i) * n;
            uint32_t c = 0;
            for (uint32_t j = 0; j < n; ++j) c += (row[j] != 0.0f) ? 1u : 0u;
            counts[i] = c;
        }
    });
    uint32_t r = 0;
    for (uint32_t c : counts) r = std::max(r, c);
    Ellpack E(m, n, r);
    E.nnz = std::move(counts);
    if (m && r) std::memset(E.Wd.ptr, 0, size_t(m) * r * sizeof(float));
    parallel_rows(m, n, [&](uint32_t lo, uint32_t hi) {
        for (uint32_t i = lo; i < hi; ++i) {
            const float* row = W + size_t(i) * n;
            const size_t base = size_t(i) * r;
            uint32_t pos = 0;
            for (uint32_t j = 0; j < n; ++j) {
                const float v = row[j];
                if (v != 0.0f) {
                    E.Wd.ptr[base + pos] = v;
                    E.idx[base + pos] = j;
                    ++pos;
                }
            }
        }
    });
    return E;
}

Ellpack convert_to_ellpack(const float* W, uint32_t m, uint32_t n)
{
    Ellpack E = encode_host(W, m, n);
    E.upload();
    return E;
}

Ellpack ellpack_from_csr(uint32_t m, uint32_t n, const uint64_t* rowptr, const uint32_t* col, const float* val)
{
    if (!rowptr) throw std::runtime_error("ellpack_from_csr: rowptr is null");
    uint32_t r = 0;
    for (uint32_t i = 0; i < m; ++i) {
        if (rowptr[i + 1] < rowptr[i]) throw std::runtime_error("ellpack_from_csr: rowptr must be non-decreasing");
        r = std::max<uint64_t>(r, rowptr[i + 1] - rowptr[i]);
    }
    Ellpack E(m, n, r);
    if (m && r) std::memset(E.Wd.ptr, 0, size_t(m) * r * sizeof(float));
    for (uint32_t i = 0; i < m; ++i) {
        const uint64_t b = rowptr[i], c = rowptr[i + 1] - b;
        E.nnz[i] = uint32_t(c);
        std::memcpy(E.Wd.ptr + size_t(i) * r, val + b, c * sizeof(float));
        std::memcpy(E.idx.data() + size_t(i) * r, col + b, c * sizeof(uint32_t));
    }
    // The device copy is built from the CSR arrays directly (no padded host traffic).
    check(spx_ell_create_csr(m, n, rowptr, col, val, &E.dev), "ELLPACK upload (CSR)");
    return E;
}

// Reference: src/ellpack_encoder.cpp:46-60.
void decode_from_ellpack(const Ellpack& E, float* W_out)
{
    std::fill(W_out, W_out + size_t(E.m) * E.n, 0.0f);
    for (uint32_t i = 0; i < E.m; ++i)
        for (uint32_t j = 0; j < E.nnz[i]; ++j)
            W_out[size_t(i) * E.n + E.idx[size_t(i) * E.r + j]] = E.Wd.ptr[size_t(i) * E.r + j];
}

static void need_device(const Ellpack& E)
{
    if (!E.dev) throw std::runtime_error("Ellpack has no device copy (call upload() first)");
}

void ellpack_matvec(const Ellpack& E, const float* x, const float* bias, float* y)
{
    need_device(E);
    E.last_x.assign(x, x + E.n);
    check(spx_spmv_host(E.dev, x, bias, y), "ellpack_matvec");
}

void ellpack_matmul(const Ellpack& E, const float* X, uint32_t C, const float* bias, float* Y)
{
    need_device(E);
    check(spx_spmm_host(E.dev, X, C, bias, SPX_ACT_NONE, Y), "ellpack_matmul");
}

template <bool USE_MASK, bool FUSE_RELU>
void ellpack_matmul_fused(const Ellpack& E, const float* X, uint32_t C, const float* bias, float* Y)
{
    need_device(E);
    check(spx_spmm_host(E.dev, X, C, bias, FUSE_RELU ? SPX_ACT_RELU : SPX_ACT_NONE, Y), "ellpack_matmul_fused");
}
template void ellpack_matmul_fused<false, false>(const Ellpack&, const float*, uint32_t, const float*, float*);
template void ellpack_matmul_fused<false, true>(const Ellpack&, const float*, uint32_t, const float*, float*);
template void ellpack_matmul_fused<true, false>(const Ellpack&, const float*, uint32_t, const float*, float*);
template void ellpack_matmul_fused<true, true>(const Ellpack&, const float*, uint32_t, const float*, float*);

void ellpack_matmul_device(const Ellpack& E, const float* dX, uint32_t C, uint64_t ldx, const float* dbias,
                           int act, float* dY, uint64_t ldy, void* stream)
{
    need_device(E);
    check(spx_spmm(E.dev, dX, C, ldx, dbias, act, dY, ldy, stream), "ellpack_matmul_device");
}

void ellpack_matvec_device(const Ellpack& E, const float* dx, const float* dbias, float* dy, void* stream)
{
    need_device(E);
    check(spx_spmv(E.dev, dx, dbias, dy, stream), "ellpack_matvec_device");
}

}  // namespace spx
