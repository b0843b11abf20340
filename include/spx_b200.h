/*
 * spx_b200.h -- C ABI of libspx_b200.so: the CUDA (sm_100a) implementation of the
 * sparse-ops ELLPACK hot path.  Plain pointers and sizes only; no C++ or torch types.
 *
 * Conventions
 *   - Every function returns an int status (SPX_OK == 0).  On failure a thread-local
 *     message is available from spx_last_error().  No exception crosses this boundary.
 *   - "device pointer" arguments must point into the memory of the CUDA device that was
 *     current (spx_set_device) when the spx_ell handle was created.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream).  Kernel
 *     entry points only enqueue work; they do not synchronise.
 *   - A handle may be used from several host threads for kernel launches, but entry points
 *     that grow per-handle scratch (spx_conv2d's first call per kernel shape, its NCHW and
 *     F-major layouts and batch sizes that are not a multiple of 4,
 *     the first spx_spmv of a handle with n > 51200, the *_host calls) must not run concurrently
 *     on the same handle.
 *   - There is no CPU fallback: without a usable CUDA device every compute entry point
 *     fails with SPX_ERR_CUDA.
 *
 * Each declaration cites the reference interface it replaces (paths inside the
 * sparse-ops project).
 */
#ifndef SPX_B200_H
#define SPX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPX_OK            0
#define SPX_ERR_ARG       1   /* bad argument (null pointer, shape mismatch, misuse) */
#define SPX_ERR_CUDA      2   /* a CUDA runtime call failed */
#define SPX_ERR_OOM       3   /* device or pinned-host allocation failed */
#define SPX_ERR_LIMIT     4   /* size beyond what an entry point supports */
#define SPX_ERR_COMM      5   /* NCCL / communicator failure */

/* Activation fused into a kernel epilogue.  RELU replaces the FUSE_RELU template flag of
 * ellpack_matmul_fused (src/ellpack_matmul.cpp:11,68-70); SIGMOID / TANH replace the
 * separate applySigmoid / applyTanh passes (src/layers/activation.cpp:24-61). */
#define SPX_ACT_NONE      0
#define SPX_ACT_RELU      1
#define SPX_ACT_SIGMOID   2
#define SPX_ACT_TANH      3

/* Activation tensor layouts of the convolution. */
#define SPX_LAYOUT_PF     0   /* [C,H,W,B], batch fastest: conv2d_patchmajor_tiled, src/layers/conv_kernels.cpp:342 */
#define SPX_LAYOUT_NCHW   1   /* [B,C,H,W]: conv2d_tiled_im2col_cmajor, src/layers/conv_kernels.cpp:233 */
#define SPX_LAYOUT_FMAJOR 2   /* b + B*(c + C*(h + H*w)), i.e. [W,H,C,B]: the output of conv2d_tiled_im2col_fmajor
                               * (src/layers/conv_kernels.cpp:150-230), input and output of conv2d_rbm_fmajor_implicit
                               * (:66-147); same indexing as src/layers/pool.cpp:17-21 */

/* Elementwise operators of spx_eltwise. */
#define SPX_OP_RELU       1
#define SPX_OP_SIGMOID    2
#define SPX_OP_TANH       3
#define SPX_OP_ADD        4

/* Device-resident ELLPACK matrix: replaces struct Ellpack (include/ellpack_encoder.hpp:6-23).
 * Wd / idx live in device memory as row-major slabs whose row pitch is r rounded up to 32
 * entries (128-byte aligned rows); nnz[m] drives every kernel, padding is never multiplied.
 * The reference's Xt gather scratch has no device counterpart. */
typedef struct spx_ell spx_ell;

/* Geometry of one convolution: the numeric fields of ConvAttr (include/sparse_onnx.hpp:64-92).
 * Begin pads only, as the loader reads them (src/sparse_onnx.cpp:411).
 * Ho = (H + 2*pH - (dH*(kH-1)+1))/sH + 1, likewise Wo (src/sparse_onnx.cpp:428-429). */
typedef struct spx_conv_geom {
    uint32_t Cin, Cout, kH, kW;
    uint32_t sH, sW, pH, pW, dH, dW;
    uint32_t H, W, Ho, Wo;
} spx_conv_geom;

/* ---- library / device ----------------------------------------------------------------- */
const char* spx_last_error(void);
int spx_version(void);
int spx_device_count(int* count);
int spx_set_device(int device);
int spx_get_device(int* device);
int spx_device_sync(void);
/* Number of kernels this library has launched in this process (all entry points). */
uint64_t spx_launch_count(void);

/* ---- memory, streams, events (so that host code above this ABI needs no CUDA headers) -- */
int spx_malloc(void** dptr, size_t bytes);            /* 256-byte aligned device memory */
int spx_free(void* dptr);
int spx_host_alloc(void** hptr, size_t bytes);        /* pinned host memory */
int spx_host_free(void* hptr);
int spx_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
int spx_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
int spx_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int spx_memset(void* dst, int value, size_t bytes, void* stream);
int spx_stream_create(void** stream);
int spx_stream_destroy(void* stream);
int spx_stream_sync(void* stream);
int spx_event_create(void** event);
int spx_event_destroy(void* event);
int spx_event_record(void* event, void* stream);
int spx_event_elapsed_ms(void* start, void* stop, float* ms);   /* synchronises on stop */

/* ---- CUDA graphs (the captured layer loop of SparseOnnxModel::run) ---------------------- */
int spx_graph_capture_begin(void* stream);
int spx_graph_capture_end(void* stream, void** graph_exec);
int spx_graph_launch(void* graph_exec, void* stream);
int spx_graph_destroy(void* graph_exec);

/* ---- ELLPACK handles ------------------------------------------------------------------- */
/* Upload host arrays in the reference layout (Wd, idx: m*r row-major; nnz: m).
 * Replaces the Ellpack constructor + convert_to_ellpack's output (src/ellpack_encoder.cpp:20-41).
 * Every idx < n and nnz[i] <= r is checked on the host before the upload. */
int spx_ell_create(uint32_t m, uint32_t n, uint32_t r, const float* Wd, const uint32_t* idx,
                   const uint32_t* nnz, spx_ell** out);
/* Build the device ELLPACK from host CSR (rowptr: m+1 entries; columns ascending per row).
 * For matrices whose dense form cannot exist; r = the longest row.  The reference only has
 * the dense route (src/ellpack_encoder.cpp:6). */
int spx_ell_create_csr(uint32_t m, uint32_t n, const uint64_t* rowptr, const uint32_t* col,
                       const float* val, spx_ell** out);
/* Encode a dense row-major m*n device matrix on the device: same result as
 * convert_to_ellpack (src/ellpack_encoder.cpp:6-44): entries with v != 0.0f, ascending columns. */
int spx_ell_encode_device(const float* dW, uint32_t m, uint32_t n, void* stream, spx_ell** out);
int spx_ell_destroy(spx_ell* e);
int spx_ell_dims(const spx_ell* e, uint32_t* m, uint32_t* n, uint32_t* r, uint64_t* nnz_total);
/* Copy back in the reference layout (any pointer may be NULL). */
int spx_ell_download(const spx_ell* e, float* Wd, uint32_t* idx, uint32_t* nnz);
/* Dense m*n row-major device output: decode_from_ellpack (src/ellpack_encoder.cpp:46-60). */
int spx_ell_decode_device(const spx_ell* e, float* dW, void* stream);

/* ---- kernels on device-resident operands ------------------------------------------------ */
/* Y[i,c] = act(bias[i] + sum_j Wd[i,j] * X[idx[i,j], c]), j in storage order, one FMA each.
 * Replaces ellpack_matmul (include/ellpack_matmul.hpp:23-43) and
 * ellpack_matmul_fused<USE_MASK,FUSE_RELU> (src/ellpack_matmul.cpp:11-92).
 * X: n rows of ldx floats (C used), Y: m rows of ldy floats.  bias may be NULL (= 0). */
int spx_spmm(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias,
             int act, float* Y, uint64_t ldy, void* stream);
/* y[i] = bias[i] + sum_j Wd[i,j] * x[idx[i,j]].  Replaces ellpack_matvec
 * (src/ellpack_matvec.cpp:20-147).  bias may be NULL.  For n above 51200 (x larger than shared
 * memory) the first call builds and caches a per-row table of column-window boundaries in the
 * handle (a device allocation of up to 28 bytes per row; make that call outside a stream capture). */
int spx_spmv(const spx_ell* e, const float* x, const float* bias, float* y, void* stream);
/* spx_spmv in the reference's own summation order (sixteen partial sums by j mod 16, then the
 * pairwise tree of src/ellpack_matvec.cpp:88-96): bit-identical to the reference's AVX-512 path,
 * slower than spx_spmv.  For checking.  Setting SPX_SPMV_REFERENCE_ORDER=1 in the environment
 * routes spx_spmv here as well. */
int spx_spmv_reference_order(const spx_ell* e, const float* x, const float* bias, float* y, void* stream);
/* Sparse convolution by implicit im2col; e is the ELLPACK of the weight flattened to
 * [Cout x Cin*kH*kW].  Replaces conv2d_patchmajor_tiled / conv2d_tiled_im2col_cmajor /
 * conv2d_tiled_im2col_fmajor / conv2d_rbm_fmajor_implicit (src/layers/conv_kernels.cpp:66-470)
 * and, on the device, build_rbm_from_ellpack (src/layers/rbm_conv.cpp:7-73): the first call per
 * handle and kernel shape builds and caches a tap table and, where the batch size and weight
 * density favour it, the row-block-merged form of the weights (device allocations; make that
 * call outside a stream capture).  Results do not depend on which kernel is chosen.  The
 * row-block-merged kernel fetches its input with bulk tensor copies and bounded waits; should a
 * wait ever run out, the next spx_conv2d on the handle returns SPX_ERR_CUDA once (the output of
 * the call that was in flight is invalid) and the handle falls back to per-thread copies. */
int spx_conv2d(const spx_ell* e, const spx_conv_geom* g, int layout, const float* in, uint32_t B,
               const float* bias, int act, float* out, void* stream);
/* spx_conv2d for callers that must not allocate device memory (no counterpart in the
 * reference, which runs on the CPU).  Some hosts hand all device memory to their own pool at
 * start-up, so a later cudaMalloc has nothing to take, and a latency-bound serving loop cannot
 * accept the device-wide synchronisation an allocation may imply.  spx_conv2d allocates its
 * per-handle tables on first use; this variant keeps the one table it needs in a fixed 4 MiB
 * array inside the library image instead (held by every GPU that loads the library until the process exits) and
 * calls no cudaMalloc / cudaFree or allocating routine.  Limits and rules: Cout * (r rounded up
 * to 32) must not exceed 1 048 576 slots, else SPX_ERR_LIMIT; the handle's device must be
 * current; all calls share the one array, so calls that overlap on the GPU race -- serialise
 * them; the first call on a device looks up the array's address and should come before any
 * stream capture.  The CUDA runtime places the library's device code, and with it the 4 MiB
 * array, on a GPU when the library is first used there: make one warm-up call per device (or any
 * other call into this library) at start-up, before the host's own pool claims the remaining
 * memory.  Same arguments and results as spx_conv2d, for the layouts SPX_LAYOUT_PF and
 * SPX_LAYOUT_NCHW (the F-major layout needs scratch tensors and is refused with SPX_ERR_ARG). */
int spx_conv2d_static(const spx_ell* e, const spx_conv_geom* g, int layout, const float* in, uint32_t B,
                      const float* bias, int act, float* out, void* stream);
/* out = op(a[, b]) elementwise; replaces applyRelu/Sigmoid/Tanh (src/layers/activation.cpp:3-62),
 * relu/sigmoid/tanh_inplace (src/activations.cpp:20-68) and applyAdd (src/layers/add.cpp:9-76).
 * out may alias a. */
int spx_eltwise(int op, const float* a, const float* b, float* out, uint64_t count, void* stream);

/* MaxPool on a [C,H,W,B] tensor: max over the in-image taps of each window, -inf when a window
 * lies entirely in the padding.  Ho = (H + pH0 + pH1 - kH)/sH + 1 (likewise Wo); out is
 * [C,Ho,Wo,B].  Replaces applyMaxPool (src/layers/pool.cpp:28-104). */
int spx_maxpool2d(const float* in, uint32_t C, uint32_t H, uint32_t W, uint32_t B, uint32_t kH, uint32_t kW,
                  uint32_t sH, uint32_t sW, uint32_t pH0, uint32_t pW0, uint32_t pH1, uint32_t pW1, float* out,
                  void* stream);
/* Mean over H*W of a [C,H,W,B] tensor into [C,B]: sequential sum in storage order times
 * 1.0f/(H*W).  Replaces applyGlobalAveragePool (src/layers/pool.cpp:106-154). */
int spx_global_avgpool(const float* in, uint32_t C, uint32_t H, uint32_t W, uint32_t B, float* out, void* stream);

/* ---- the same calls on HOST buffers (what the reference's Python binding does) ---------- */
/* X, bias, Y are host arrays; copies in and out go through pinned staging owned by the
 * handle's device context.  Replaces the ellpack_matmul / ellpack_matvec lambdas of
 * src/bindings.cpp:91-139.  Synchronous. */
int spx_spmm_host(const spx_ell* e, const float* X, uint32_t C, const float* bias, int act, float* Y);
int spx_spmv_host(const spx_ell* e, const float* x, const float* bias, float* y);

/* ---- communicator for the row-sharded paths (one process per GPU, NCCL) ------------------ */
typedef struct spx_comm spx_comm;
#define SPX_UNIQUE_ID_BYTES 128
int spx_comm_unique_id(char id[SPX_UNIQUE_ID_BYTES]);
int spx_comm_create(int rank, int world, const char id[SPX_UNIQUE_ID_BYTES], spx_comm** out);
int spx_comm_destroy(spx_comm* c);
/* In-place all-gather of row slabs: rank g's rows_per_rank*ld floats already sit at
 * Y + g*rows_per_rank*ld of the full buffer.  (The reference has no multi-device path; this is
 * the exchange step of row-sharded SpMM, src/ellpack_matmul.cpp:26 being the row loop it splits.) */
int spx_allgather_rows(spx_comm* c, float* Y, uint64_t rows_per_rank, uint64_t ld, void* stream);

int spx_comm_info(const spx_comm* c, int* rank, int* world);      /* either pointer may be NULL */

/* Row-sharded spx_spmm_host, one process per GPU: e holds this rank's rows of E (the split is the
 * row loop of src/ellpack_matmul.cpp:26; the host-buffer call it replaces is the ellpack_matmul
 * lambda of src/bindings.cpp:110-139).  X is the whole host operand (n x C, the same on every
 * rank); each rank copies only rows [rank*ceil(n/world), ...) of it over PCIe, the ranks rebuild the
 * replicated X on their devices with in-place all-gathers over NVLink, multiply, and copy their own
 * rows of Y (m x C, m = this rank's rows) back to the host -- 256-column panels pipelined over four
 * streams.  Collective: every rank of the communicator must make the call with the same n and C.
 * phase_ms (may be NULL): four floats, the device time this rank spent in the copy in, the
 * exchange, the multiply and the copy out, summed over the panels (the stages overlap, so their
 * sum exceeds the call's duration).  comm == NULL or a world of 1: same as spx_spmm_host.
 * Synchronous.  Up to 1792 columns. */
int spx_spmm_host_sharded(spx_comm* comm, const spx_ell* e, const float* X, uint32_t C, const float* bias,
                          int act, float* Y, float* phase_ms);

/* Stream-ordered barrier over the communicator (a one-float all-reduce): when it completes on this
 * rank's stream, every rank has finished the work it enqueued before its own call. */
int spx_comm_barrier(spx_comm* c, void* stream);

/* ---- peer buffers and the fused SpMM + all-gather ----------------------------------------- */
/* Share a device allocation made with spx_malloc with the other ranks of this node (one process
 * per GPU): export an opaque handle, send it to the peers by any host channel, open it there.
 * The opened pointer addresses the exporter's memory over NVLink. */
#define SPX_IPC_HANDLE_BYTES 64
int spx_ipc_export(void* dptr, char handle[SPX_IPC_HANDLE_BYTES]);
int spx_ipc_open(const char handle[SPX_IPC_HANDLE_BYTES], void** dptr);
int spx_ipc_close(void* dptr);
/* Row-sharded SpMM whose epilogue IS the all-gather: e holds this rank's rows, which occupy rows
 * [row_offset, row_offset + m) of the full Y; every finished output vector is stored into each of
 * the nbuffers (<= 8) full-size buffers Ys[g] (this rank's own buffer and its peers' buffers
 * opened with spx_ipc_open), leading dimension ldy, with ordinary stores over NVLink, so the
 * exchange overlaps the multiply.  Follow it with spx_comm_barrier before any rank reads Y.
 * Same arithmetic as spx_spmm (the split is the row loop of src/ellpack_matmul.cpp:26). */
int spx_spmm_bcast(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                   float* const* Ys, uint32_t nbuffers, uint64_t row_offset, uint64_t ldy, void* stream);
/* The same exchange through the copy engines: the rank's rows are multiplied in `slices` (0 = 4,
 * at most 16) contiguous slices of near-equal work on `stream`, each written into Ys[self]; as
 * soon as a slice is final it is copied into every other buffer Ys[g] with asynchronous
 * device-to-device copies on internal streams, so the NVLink transfer of slice k overlaps the
 * multiplication of slices k+1.. and takes no load/store slots from the SMs.  `stream` continues
 * once all copies are done (fork / join by events; works under stream capture after a first,
 * uncaptured call has built the slices).  Follow it with spx_comm_barrier before any rank reads Y.
 * Same arithmetic as spx_spmm. */
int spx_spmm_exchange(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                      float* const* Ys, uint32_t nbuffers, uint32_t self, uint64_t row_offset, uint64_t ldy,
                      uint32_t slices, void* stream);
/* The same with one destination: Ymc is an NVLink multicast address under which every rank's full
 * Y buffer is bound (an NVLS multicast object; e.g. the multicast_ptr of a torch symmetric-memory
 * rendezvous over those buffers).  Each finished vector leaves this GPU once (multimem.st) and the
 * NVSwitch replicates it into all bound buffers, this rank's included: (G-1)x less traffic out of
 * every GPU than spx_spmm_bcast.  C, ldx, ldy multiples of 4; X and Ymc 16-byte aligned.  Follow
 * it with spx_comm_barrier before any rank reads Y. */
int spx_spmm_mcast(const spx_ell* e, const float* X, uint32_t C, uint64_t ldx, const float* bias, int act,
                   float* Ymc, uint64_t row_offset, uint64_t ldy, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPX_B200_H */
