/*
 * ellpack_oracle.c -- CPU restatement of the sparse-ops ELLPACK hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the
 * smoke test and the CPU-baseline leg of the benchmark compare the CUDA path
 * against.  Nothing in the product library links, loads or calls it.
 *
 * Every function restates, in plain scalar C, the arithmetic of one function
 * of the reference project (citations are paths inside that project).  The
 * order of floating-point operations follows the reference's AVX-512 code
 * path, so results are bit-identical to the reference binary on an AVX-512
 * host; the parity pin is tests/golden/ (outputs of the reference binary).
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -mfma -fopenmp).
 * -ffp-contract=off matters: every fused multiply-add below is an explicit
 * fmaf(), every other operation must stay unfused.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ------------------------------------------------------------------------
 * Encoder.  Reference: src/ellpack_encoder.cpp:6-44 (convert_to_ellpack).
 * Pass 1 counts entries with v != 0.0f per row (so -0.0f is dropped, NaN,
 * infinities and denormals are kept) and returns r = the largest count.
 * ---------------------------------------------------------------------- */
uint32_t orc_ell_count(const float* W, uint32_t m, uint32_t n, uint32_t* nnz)
{
    uint32_t r = 0;
    for (uint32_t i = 0; i < m; ++i) {
        const float* row = W + (size_t)i * n;
        uint32_t cnt = 0;
        for (uint32_t j = 0; j < n; ++j)
            if (row[j] != 0.0f) ++cnt;
        nnz[i] = cnt;
        if (cnt > r) r = cnt;
    }
    return r;
}

/* Pass 2: values and column ids in ascending column order, padding slots
 * hold Wd = 0.0f and idx = 0.  Reference: src/ellpack_encoder.cpp:25-41. */
void orc_ell_pack(const float* W, uint32_t m, uint32_t n, uint32_t r,
                  float* Wd, uint32_t* idx)
{
    memset(Wd, 0, (size_t)m * r * sizeof(float));
    memset(idx, 0, (size_t)m * r * sizeof(uint32_t));
    for (uint32_t i = 0; i < m; ++i) {
        const float* row = W + (size_t)i * n;
        size_t base = (size_t)i * r;
        uint32_t pos = 0;
        for (uint32_t j = 0; j < n; ++j) {
            float v = row[j];
            if (v != 0.0f) {
                Wd[base + pos] = v;
                idx[base + pos] = j;
                ++pos;
            }
        }
    }
}

/* Decoder.  Reference: src/ellpack_encoder.cpp:46-60 (decode_from_ellpack). */
void orc_ell_decode(uint32_t m, uint32_t n, uint32_t r, const float* Wd,
                    const uint32_t* idx, const uint32_t* nnz, float* W)
{
    memset(W, 0, (size_t)m * n * sizeof(float));
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < nnz[i]; ++j)
            W[(size_t)i * n + idx[(size_t)i * r + j]] = Wd[(size_t)i * r + j];
}

/* ------------------------------------------------------------------------
 * Activations.  Reference: src/layers/activation.cpp:3-62 and
 * src/activations.cpp:20-68.  act: 0 none, 1 relu, 2 sigmoid, 3 tanh.
 * ---------------------------------------------------------------------- */
static inline float orc_act(float v, int act)
{
    switch (act) {
    case 1: return v > 0.0f ? v : 0.0f;
    case 2: return 1.0f / (1.0f + expf(-v));
    case 3: return tanhf(v);
    default: return v;
    }
}

void orc_activation(const float* src, float* dst, size_t count, int act)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; ++i) dst[i] = orc_act(src[i], act);
}

/* Same-shape elementwise add.  Reference: src/layers/add.cpp:9-76. */
void orc_add(const float* a, const float* b, float* dst, size_t count)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; ++i) dst[i] = a[i] + b[i];
}

/* ------------------------------------------------------------------------
 * SpMM.  Reference: src/ellpack_matmul.cpp:11-92 (ellpack_matmul_fused).
 * Per output element: start from bias[i] (or 0), then one fused multiply-add
 * per stored nonzero of the row in storage order (:56-66), then the optional
 * activation (:68-70 has ReLU only; sigmoid/tanh are the model's separate
 * activation layers applied to the stored value).  X is [n x C] with leading
 * dimension ldx, Y is [m x C] with leading dimension ldy.
 * ---------------------------------------------------------------------- */
void orc_spmm(uint32_t m, uint32_t r, const float* Wd, const uint32_t* idx,
              const uint32_t* nnz, const float* X, uint32_t C, size_t ldx,
              const float* bias, int act, float* Y, size_t ldy)
{
#pragma omp parallel for schedule(dynamic, 16)
    for (uint32_t i = 0; i < m; ++i) {
        const float* w = Wd + (size_t)i * r;
        const uint32_t* ci = idx + (size_t)i * r;
        const uint32_t cnt = nnz[i];
        float* y = Y + (size_t)i * ldy;
        const float b = bias ? bias[i] : 0.0f;
        for (uint32_t c = 0; c < C; ++c) y[c] = b;
        for (uint32_t j = 0; j < cnt; ++j) {
            const float wj = w[j];
            const float* x = X + (size_t)ci[j] * ldx;
            for (uint32_t c = 0; c < C; ++c) y[c] = fmaf(wj, x[c], y[c]);
        }
        if (act)
            for (uint32_t c = 0; c < C; ++c) y[c] = orc_act(y[c], act);
    }
}

/* ------------------------------------------------------------------------
 * SpMV.  Reference: src/ellpack_matvec.cpp:20-100 (AVX-512 branch).
 * Sixteen partial sums: lane l accumulates entries j = l, l+16, ... with one
 * fused multiply-add each (:72-85, the masked tail leaves other lanes as
 * they are: fma(0,0,acc) == acc).  Reduction (:88-96): lanes l and l+8,
 * then l and l+4, then the two horizontal adds (0+1, 2+3, then their sum).
 * Finally y[i] = bias[i] + acc (:30-34, :99).
 * ---------------------------------------------------------------------- */
void orc_spmv(uint32_t m, uint32_t r, const float* Wd, const uint32_t* idx,
              const uint32_t* nnz, const float* x, const float* bias, float* y)
{
#pragma omp parallel for schedule(static)
    for (uint32_t i = 0; i < m; ++i) {
        const float* w = Wd + (size_t)i * r;
        const uint32_t* ci = idx + (size_t)i * r;
        const uint32_t cnt = nnz[i];
        float a[16];
        for (int l = 0; l < 16; ++l) a[l] = 0.0f;
        for (uint32_t j = 0; j < cnt; ++j)
            a[j & 15] = fmaf(w[j], x[ci[j]], a[j & 15]);
        float s8[8], s4[4];
        for (int l = 0; l < 8; ++l) s8[l] = a[l] + a[l + 8];
        for (int l = 0; l < 4; ++l) s4[l] = s8[l] + s8[l + 4];
        const float h0 = s4[0] + s4[1];
        const float h1 = s4[2] + s4[3];
        const float acc = h0 + h1;
        const float b = bias ? bias[i] : 0.0f;
        y[i] = b + acc;
    }
}

/* Per-element magnitude bound sum_j |w_ij| |x_idx| (+ |bias_i|) that the
 * floating-point tolerance 1e-5 * bound is stated against. */
void orc_spmv_absbound(uint32_t m, uint32_t r, const float* Wd, const uint32_t* idx,
                       const uint32_t* nnz, const float* x, const float* bias,
                       double* bound)
{
#pragma omp parallel for schedule(static)
    for (uint32_t i = 0; i < m; ++i) {
        double s = bias ? fabs((double)bias[i]) : 0.0;
        for (uint32_t j = 0; j < nnz[i]; ++j)
            s += fabs((double)Wd[(size_t)i * r + j]) * fabs((double)x[idx[(size_t)i * r + j]]);
        bound[i] = s;
    }
}

/* ------------------------------------------------------------------------
 * Sparse convolution.  Reference: src/layers/conv_kernels.cpp:342-470
 * (conv2d_patchmajor_tiled, layout 0 = patch-major [C,H,W,B], batch fastest)
 * and :233-339 (conv2d_tiled_im2col_cmajor, layout 1 = NCHW).  Both pack an
 * explicit im2col tile with zeros outside the image and hand it to
 * ellpack_matmul_fused, so per output element the arithmetic is the SpMM
 * chain over the row's nonzeros k = (cin, kh, kw) in storage order, with the
 * operand 0.0f for taps outside the image.  Layout 2 = F-major,
 * b + B*(c + C*(h + H*w)) for input and output: the indexing of
 * conv2d_rbm_fmajor_implicit (:66-147, off4_BCHW :8-11; it gathers on the fly,
 * skips taps outside the image and walks each row's entries in ascending k,
 * i.e. the same chain) and of the output of conv2d_tiled_im2col_fmajor
 * (:150-230, whose input is read in the [C,H,W,B] order of patch_indices).  Geometry as in
 * src/sparse_onnx.cpp:411-451: begin pads only, ih = oh*stride + kh*dil - pad.
 * The reference's two tiled kernels mis-index stride_w > 1 (they advance the
 * input column by 1 per output column, :305-306 and :438-439); this
 * restatement uses the mathematically correct stride, so parity with the
 * reference binary is defined for stride_w == 1 only.
 * ---------------------------------------------------------------------- */
void orc_conv2d(uint32_t Cout, uint32_t r, const float* Wd, const uint32_t* idx,
                const uint32_t* nnz, uint32_t Cin, uint32_t kH, uint32_t kW,
                uint32_t sH, uint32_t sW, uint32_t pH, uint32_t pW, uint32_t dH,
                uint32_t dW, uint32_t H, uint32_t W, uint32_t Ho, uint32_t Wo,
                int layout, const float* src, uint32_t B, const float* bias,
                int act, float* dst)
{
    (void)Cin;
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t mo = 0; mo < Cout; ++mo) {
        for (uint32_t oh = 0; oh < Ho; ++oh) {
            const float* w = Wd + (size_t)mo * r;
            const uint32_t* ci = idx + (size_t)mo * r;
            const uint32_t cnt = nnz[mo];
            const float bi = bias ? bias[mo] : 0.0f;
            for (uint32_t ow = 0; ow < Wo; ++ow) {
                for (uint32_t b = 0; b < B; ++b) {
                    float y = bi;
                    for (uint32_t j = 0; j < cnt; ++j) {
                        const uint32_t k = ci[j];
                        const uint32_t cin = k / (kH * kW);
                        const uint32_t kh = (k / kW) % kH;
                        const uint32_t kw = k % kW;
                        const int ih = (int)(oh * sH) + (int)(kh * dH) - (int)pH;
                        const int iw = (int)(ow * sW) + (int)(kw * dW) - (int)pW;
                        float xv = 0.0f;
                        if ((unsigned)ih < H && (unsigned)iw < W) {
                            size_t off = layout == 0
                                ? (((size_t)cin * H + ih) * W + iw) * B + b
                                : layout == 2
                                ? (((size_t)iw * H + ih) * Cin + cin) * B + b
                                : (((size_t)b * Cin + cin) * H + ih) * W + iw;
                            xv = src[off];
                        }
                        y = fmaf(w[j], xv, y);
                    }
                    y = orc_act(y, act);
                    size_t o = layout == 0
                        ? (((size_t)mo * Ho + oh) * Wo + ow) * B + b
                        : layout == 2
                        ? (((size_t)ow * Ho + oh) * Cout + mo) * B + b
                        : (((size_t)b * Cout + mo) * Ho + oh) * Wo + ow;
                    dst[o] = y;
                }
            }
        }
    }
}

/* ------------------------------------------------------------------------
 * Pools on [C,H,W,B] tensors.  Arithmetic of the reference's applyMaxPool
 * (src/layers/pool.cpp:28-104: max over in-image taps from -inf) and
 * applyGlobalAveragePool (:106-154: sum over h then w from 0, times
 * 1.0f/(H*W)).  The reference indexes them as b + B*(c + C*(h + H*w)); the
 * per-(c,b) order of operations is the same, so on the same logical tensor
 * the results are bit-identical.
 * ---------------------------------------------------------------------- */
void orc_maxpool_pf(const float* in, uint32_t C, uint32_t H, uint32_t W, uint32_t B,
                    uint32_t kH, uint32_t kW, uint32_t sH, uint32_t sW,
                    uint32_t pH0, uint32_t pW0, uint32_t pH1, uint32_t pW1, float* out)
{
    const uint32_t Ho = (H + pH0 + pH1 - kH) / sH + 1, Wo = (W + pW0 + pW1 - kW) / sW + 1;
    for (uint32_t c = 0; c < C; ++c)
        for (uint32_t oh = 0; oh < Ho; ++oh)
            for (uint32_t ow = 0; ow < Wo; ++ow)
                for (uint32_t b = 0; b < B; ++b) {
                    float v = -INFINITY;
                    for (uint32_t kh = 0; kh < kH; ++kh) {
                        const int ih = (int)(oh * sH) - (int)pH0 + (int)kh;
                        if ((unsigned)ih >= H) continue;
                        for (uint32_t kw = 0; kw < kW; ++kw) {
                            const int iw = (int)(ow * sW) - (int)pW0 + (int)kw;
                            if ((unsigned)iw >= W) continue;
                            const float x = in[(((size_t)c * H + ih) * W + iw) * B + b];
                            v = x > v ? x : v;
                        }
                    }
                    out[(((size_t)c * Ho + oh) * Wo + ow) * B + b] = v;
                }
}

void orc_gap_pf(const float* in, uint32_t C, uint32_t H, uint32_t W, uint32_t B, float* out)
{
    const float scale = 1.0f / (float)(H * W);
    for (uint32_t c = 0; c < C; ++c)
        for (uint32_t b = 0; b < B; ++b) {
            float s = 0.0f;
            for (uint32_t i = 0; i < H * W; ++i) s += in[((size_t)c * H * W + i) * B + b];
            out[(size_t)c * B + b] = s * scale;
        }
}
