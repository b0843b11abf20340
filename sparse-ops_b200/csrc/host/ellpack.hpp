// ellpack.hpp -- host-side C++ interface of the ELLPACK hot path, source-compatible with the
// reference's headers: struct Ellpack (include/ellpack_encoder.hpp:6-23), AlignedBuffer
// (include/aligned_buffer.hpp:8-30), convert_to_ellpack / decode_from_ellpack
// (include/ellpack_encoder.hpp:28-32), ellpack_matvec (include/ellpack_matvec.hpp),
// ellpack_matmul and ellpack_matmul_fused<USE_MASK,FUSE_RELU> (include/ellpack_matmul.hpp:13-43).
//
// Differences a caller can observe: the encoded matrix is also resident on the CUDA device that
// is current when it is created (handle `dev`), and every multiply runs there through the C ABI
// of libspx_b200.so -- there is no CPU compute path; a missing GPU raises std::runtime_error.
// Xt (the reference's gather scratch) is not stored; Ellpack::gathered_x() rebuilds it on demand.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <new>
#include <stdexcept>
#include <utility>
#include <vector>

#include "spx_b200.h"

namespace spx {

// 64-byte aligned, move-only float buffer (reference: include/aligned_buffer.hpp:8-30).
struct AlignedBuffer {
    float* ptr{nullptr};
    size_t size{0};
    AlignedBuffer() = default;
    explicit AlignedBuffer(size_t n) : size(n) {
        size_t bytes = (n * sizeof(float) + 63) / 64 * 64;
        if (bytes == 0) bytes = 64;
        void* p = nullptr;
        if (posix_memalign(&p, 64, bytes) != 0 || !p) throw std::bad_alloc();
        ptr = static_cast<float*>(p);
    }
    ~AlignedBuffer() { std::free(ptr); }
    AlignedBuffer(const AlignedBuffer&) = delete;
    AlignedBuffer& operator=(const AlignedBuffer&) = delete;
    AlignedBuffer(AlignedBuffer&& o) noexcept : ptr(o.ptr), size(o.size) { o.ptr = nullptr; o.size = 0; }
    AlignedBuffer& operator=(AlignedBuffer&& o) noexcept { std::swap(ptr, o.ptr); std::swap(size, o.size); return *this; }
};

// Throws std::runtime_error (std::bad_alloc for SPX_ERR_OOM) carrying spx_last_error().
void check(int status, const char* what);

struct Ellpack {
    uint32_t m;   ///< rows
    uint32_t n;   ///< original columns
    uint32_t r;   ///< max nonzeros per row

    AlignedBuffer Wd;             ///< m*r floats, host copy in the reference layout
    std::vector<uint32_t> idx;    ///< m*r column ids
    std::vector<uint32_t> nnz;    ///< m counts
    spx_ell* dev{nullptr};        ///< device-resident copy (created by upload())
    mutable std::vector<float> last_x;   ///< operand of the latest ellpack_matvec (for gathered_x)

    Ellpack(uint32_t m_, uint32_t n_, uint32_t r_)
        : m(m_), n(n_), r(r_), Wd(size_t(m_) * r_), idx(size_t(m_) * r_), nnz(m_) {}
    ~Ellpack();
    Ellpack(const Ellpack&) = delete;
    Ellpack& operator=(const Ellpack&) = delete;
    Ellpack(Ellpack&& o) noexcept;
    Ellpack& operator=(Ellpack&& o) noexcept;

    /// (Re)creates the device copy from the host arrays on the current device.
    void upload();
    /// x[idx] for all m*r slots: what the reference leaves in Xt after a matvec
    /// (src/ellpack_matvec.cpp:48-52); zeros before the first matvec.
    std::vector<float> gathered_x() const;
    /// Rows [g*ceil(m/G), (g+1)*ceil(m/G)) clipped to m, as an independent matrix, for row-sharded
    /// runs (uploaded unless upload == false).  Every shard keeps the parent's r.
    Ellpack shard_rows(uint32_t g, uint32_t G, bool upload = true) const;
    /// Rows [lo, hi) as an independent matrix (keeps the parent's r).
    Ellpack shard_range(uint32_t lo, uint32_t hi, bool upload = true) const;
    /// G + 1 ascending row bounds (first 0, last m) cutting the rows into G contiguous ranges of
    /// near-equal work, a row counting as nnz[i] + row_cost: the split to use instead of equal row
    /// counts when the long rows cluster.  The reference's row loop (src/ellpack_matmul.cpp:26-30)
    /// leaves that balance to OpenMP's static schedule.
    std::vector<uint32_t> balanced_row_split(uint32_t G, uint32_t row_cost = 8) const;
    uint64_t nnz_total() const;
};

/// Encode a dense row-major m x n matrix (host memory) and upload it.
Ellpack convert_to_ellpack(const float* W, uint32_t m, uint32_t n);
/// Host-only encoding (no device copy); used by the planner before sharding decisions.
Ellpack encode_host(const float* W, uint32_t m, uint32_t n);
/// Build directly from CSR (columns strictly ascending per row) and upload.
Ellpack ellpack_from_csr(uint32_t m, uint32_t n, const uint64_t* rowptr, const uint32_t* col, const float* val);
/// W_out must hold m*n floats.
void decode_from_ellpack(const Ellpack& E, float* W_out);

/// y = E x + bias on host buffers (bias may be nullptr).
void ellpack_matvec(const Ellpack& E, const float* x, const float* bias, float* y);
/// Y = E X + bias on host buffers: X is n x C, Y is m x C, row-major (bias may be nullptr).
void ellpack_matmul(const Ellpack& E, const float* X, uint32_t C, const float* bias, float* Y);
/// Same with the reference's template switches; USE_MASK has no meaning on the GPU.
template <bool USE_MASK, bool FUSE_RELU>
void ellpack_matmul_fused(const Ellpack& E, const float* X, uint32_t C, const float* bias, float* Y);

/// Device-resident operands (pointers into the handle's device), asynchronous on `stream`.
void ellpack_matmul_device(const Ellpack& E, const float* dX, uint32_t C, uint64_t ldx, const float* dbias,
                           int act, float* dY, uint64_t ldy, void* stream);
void ellpack_matvec_device(const Ellpack& E, const float* dx, const float* dbias, float* dy, void* stream);

}  // namespace spx

#ifndef SPX_NO_GLOBAL_NAMES
using spx::AlignedBuffer;
using spx::Ellpack;
using spx::convert_to_ellpack;
using spx::decode_from_ellpack;
using spx::ellpack_matmul;
using spx::ellpack_matmul_fused;
using spx::ellpack_matvec;
#endif
