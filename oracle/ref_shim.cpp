// ref_shim.cpp -- extern "C" handles onto the UNMODIFIED reference implementation.
//
// TEST INFRASTRUCTURE ONLY.  oracle/Makefile compiles the reference project's own
// src/*.cpp and src/layers/*.cpp where they lie (nothing is copied) together with this
// file into oracle/_ref/libsparseops_ref.so.  The wrappers let Python (ctypes) drive the
// reference's C++ functions: they add no arithmetic of their own.  Used to (1) validate
// oracle/ellpack_oracle.c, (2) generate tests/golden/, (3) time the reference's CPU path
// as the benchmark's reference arm.  The product library never loads it.
#include <cstdint>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "conv_kernels.hpp"
#include "ellpack_encoder.hpp"
#include "ellpack_matmul.hpp"
#include "ellpack_matvec.hpp"
#include "rbm_conv.hpp"
#include "sparse_onnx.hpp"

extern "C" {

// ---- Ellpack (include/ellpack_encoder.hpp:6-23) -------------------------------------
void* ref_ell_encode(const float* W, uint32_t m, uint32_t n) {
    return new Ellpack(convert_to_ellpack(W, m, n));
}
// Fill the public fields directly (used for matrices too large to exist densely).
void* ref_ell_from_arrays(uint32_t m, uint32_t n, uint32_t r, const float* Wd,
                          const uint32_t* idx, const uint32_t* nnz) {
    Ellpack* E = new Ellpack(m, n, r);
    std::memcpy(E->Wd.ptr, Wd, size_t(m) * r * sizeof(float));
    std::memcpy(E->idx.data(), idx, size_t(m) * r * sizeof(uint32_t));
    std::memcpy(E->nnz.data(), nnz, size_t(m) * sizeof(uint32_t));
    return E;
}
void ref_ell_free(void* e) { delete static_cast<Ellpack*>(e); }
void ref_ell_dims(void* e, uint32_t* m, uint32_t* n, uint32_t* r) {
    auto* E = static_cast<Ellpack*>(e);
    *m = E->m; *n = E->n; *r = E->r;
}
void ref_ell_copy(void* e, float* Wd, uint32_t* idx, uint32_t* nnz) {
    auto* E = static_cast<Ellpack*>(e);
    size_t tot = size_t(E->m) * E->r;
    if (Wd) std::memcpy(Wd, E->Wd.ptr, tot * sizeof(float));
    if (idx) std::memcpy(idx, E->idx.data(), tot * sizeof(uint32_t));
    if (nnz) std::memcpy(nnz, E->nnz.data(), size_t(E->m) * sizeof(uint32_t));
}
void ref_ell_decode(void* e, float* W) { decode_from_ellpack(*static_cast<Ellpack*>(e), W); }

// ---- SpMM / SpMV --------------------------------------------------------------------
// include/ellpack_matmul.hpp:23-43 (the dispatcher the Python binding calls).
void ref_matmul(void* e, const float* X, uint32_t C, const float* bias, float* Y) {
    ellpack_matmul(*static_cast<Ellpack*>(e), X, C, bias, Y);
}
// src/ellpack_matmul.cpp:11-92 with the masked variant, optional fused ReLU (what the
// model's applyMatMul and the conv kernels call).
void ref_matmul_fused(void* e, const float* X, uint32_t C, const float* bias, float* Y, int relu) {
    if (relu) ellpack_matmul_fused<true, true>(*static_cast<Ellpack*>(e), X, C, bias, Y);
    else      ellpack_matmul_fused<true, false>(*static_cast<Ellpack*>(e), X, C, bias, Y);
}
// src/ellpack_matvec.cpp:20-147.
void ref_matvec(void* e, const float* x, const float* bias, float* y) {
    ellpack_matvec(*static_cast<Ellpack*>(e), x, bias, y);
}

// ---- Conv (include/sparse_onnx.hpp:64-92 ConvAttr; src/sparse_onnx.cpp:380-520) -----
// Builds a ConvAttr from a dense [Cout][Cin][kH][kW] weight the way the loader does:
// encode the flattened weight, begin-pads only, kmap in (cin,kh,kw) order.  The bias
// array is copied and owned by the returned object.
struct RefConv { ConvAttr attr; std::vector<float> bias; };

void* ref_conv_create(const float* weight, uint32_t Cout, uint32_t Cin, uint32_t kH, uint32_t kW,
                      uint32_t sH, uint32_t sW, uint32_t pH, uint32_t pW, uint32_t dH, uint32_t dW,
                      uint32_t H, uint32_t W, const float* bias, int relu) {
    const uint32_t K = Cin * kH * kW;
    auto* rc = new RefConv{ ConvAttr{ convert_to_ellpack(weight, Cout, K) }, {} };
    ConvAttr& c = rc->attr;
    c.Cin = Cin; c.Cout = Cout; c.kH = kH; c.kW = kW;
    c.stride_h = sH; c.stride_w = sW; c.pad_h = pH; c.pad_w = pW; c.dil_h = dH; c.dil_w = dW;
    c.group = 1; c.H_in = H; c.W_in = W;
    c.H_out = (H + 2 * pH - (dH * (kH - 1) + 1)) / sH + 1;
    c.W_out = (W + 2 * pW - (dW * (kW - 1) + 1)) / sW + 1;
    c.kmap.reserve(K);
    for (uint32_t ci = 0; ci < Cin; ++ci)
        for (uint32_t kh = 0; kh < kH; ++kh)
            for (uint32_t kw = 0; kw < kW; ++kw)
                c.kmap.push_back(KMap{ ci, int32_t(kh * dH) - int32_t(pH), int32_t(kw * dW) - int32_t(pW) });
    if (bias) { rc->bias.assign(bias, bias + Cout); c.bias_ptr = rc->bias.data(); }
    c.fuse_relu = relu != 0;
    // the tables the F-major kernels read, filled as the loader fills them
    // (src/sparse_onnx.cpp:476-502): offsets of every (patch, k) in [C,H,W] order, one past the
    // end for taps outside the image, and the row-block-merged plan
    c.sentinel_off = size_t(Cin) * H * W;
    c.patch_indices.resize(size_t(K) * c.H_out * c.W_out);
    for (uint32_t ph = 0; ph < c.H_out; ++ph)
        for (uint32_t pw = 0; pw < c.W_out; ++pw)
            for (uint32_t k = 0; k < K; ++k) {
                const int ih = int(ph) * int(sH) + c.kmap[k].dh, iw = int(pw) * int(sW) + c.kmap[k].dw;
                const bool in = (unsigned)ih < H && (unsigned)iw < W;
                c.patch_indices[(size_t(ph) * c.W_out + pw) * K + k] =
                    in ? (size_t(c.kmap[k].cin) * H + size_t(ih)) * W + size_t(iw) : c.sentinel_off;
            }
    c.rbm = build_rbm_from_ellpack(c.E, c.bias_ptr, 8);
    c.use_rbm = true;
    return rc;
}
void ref_conv_free(void* h) { delete static_cast<RefConv*>(h); }
void ref_conv_out_dims(void* h, uint32_t* Ho, uint32_t* Wo) {
    auto* rc = static_cast<RefConv*>(h);
    *Ho = rc->attr.H_out; *Wo = rc->attr.W_out;
}
void* ref_conv_ell(void* h) { return &static_cast<RefConv*>(h)->attr.E; }
// layout 0: conv2d_patchmajor_tiled (src/layers/conv_kernels.cpp:342-470, [C,H,W,B]);
// layout 1: conv2d_tiled_im2col_cmajor (:233-339, NCHW);
// layout 2: conv2d_tiled_im2col_fmajor (:150-230, reads [C,H,W,B], writes F-major [W,H,C,B]);
// layout 3: conv2d_rbm_fmajor_implicit (:66-147, F-major in and out).
void ref_conv_run(void* h, int layout, const float* src, uint32_t B, float* dst) {
    auto* rc = static_cast<RefConv*>(h);
    if (layout == 0)      conv2d_patchmajor_tiled(rc->attr, src, B, dst);
    else if (layout == 2) conv2d_tiled_im2col_fmajor(rc->attr, src, B, dst);
    else if (layout == 3) conv2d_rbm_fmajor_implicit(rc->attr, src, B, dst);
    else                  conv2d_tiled_im2col_cmajor(rc->attr, src, B, dst);
}

// ---- RBM plan (src/layers/rbm_conv.cpp:7-73) ----------------------------------------
void* ref_rbm_build(void* e, const float* bias, uint32_t ct_max) {
    return new RBMPlan(build_rbm_from_ellpack(*static_cast<Ellpack*>(e), bias, ct_max));
}
void ref_rbm_free(void* p) { delete static_cast<RBMPlan*>(p); }
uint32_t ref_rbm_num_blocks(void* p) { return (uint32_t)static_cast<RBMPlan*>(p)->blocks.size(); }
void ref_rbm_block_sizes(void* p, uint32_t b, uint32_t* M0, uint32_t* Ct, uint32_t* U, uint32_t* npairs, uint32_t* nbias) {
    const RBMBlock& B = static_cast<RBMPlan*>(p)->blocks[b];
    *M0 = B.M0; *Ct = B.Ct; *U = (uint32_t)B.krel.size(); *npairs = (uint32_t)B.pairs.size(); *nbias = (uint32_t)B.bias.size();
}
void ref_rbm_block_copy(void* p, uint32_t b, uint32_t* krel, uint32_t* colptr, uint16_t* rows, float* w, float* bias) {
    const RBMBlock& B = static_cast<RBMPlan*>(p)->blocks[b];
    std::memcpy(krel, B.krel.data(), B.krel.size() * sizeof(uint32_t));
    std::memcpy(colptr, B.colptr.data(), B.colptr.size() * sizeof(uint32_t));
    for (size_t t = 0; t < B.pairs.size(); ++t) { rows[t] = B.pairs[t].row; w[t] = B.pairs[t].w; }
    if (!B.bias.empty()) std::memcpy(bias, B.bias.data(), B.bias.size() * sizeof(float));
}

// ---- Model (include/sparse_onnx.hpp:139-163; src/model_run.cpp:3-140) ---------------
// Returns nullptr and fills err (if given) when the constructor throws.
void* ref_model_load(const char* path, char* err, size_t errlen) {
    try {
        return new SparseOnnxModel(std::string(path));
    } catch (const std::exception& ex) {
        if (err && errlen) { std::strncpy(err, ex.what(), errlen - 1); err[errlen - 1] = 0; }
        return nullptr;
    }
}
void ref_model_free(void* m) { delete static_cast<SparseOnnxModel*>(m); }
int ref_model_output_shape(void* m, uint64_t* dims, int maxdims) {
    auto s = static_cast<SparseOnnxModel*>(m)->output_shape();
    for (int i = 0; i < (int)s.size() && i < maxdims; ++i) dims[i] = s[i];
    return (int)s.size();
}
int ref_model_run(void* m, const float* in, uint32_t B, float* out, char* err, size_t errlen) {
    try {
        static_cast<SparseOnnxModel*>(m)->run(in, B, out);
        return 0;
    } catch (const std::exception& ex) {
        if (err && errlen) { std::strncpy(err, ex.what(), errlen - 1); err[errlen - 1] = 0; }
        return 1;
    }
}

}  // extern "C"
