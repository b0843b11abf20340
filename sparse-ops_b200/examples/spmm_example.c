/*
 * spmm_example.c -- the C ABI of libspx_b200.so used from plain C, the way a binding in another
 * host language would: encode a small matrix on the host, upload it once, multiply with host
 * buffers (spx_spmm_host) and with device buffers (spx_spmm), compare with a scalar loop.
 *
 *   gcc -std=c11 -I../../include spmm_example.c -L.. -lspx_b200 -Wl,-rpath,'$ORIGIN/..' -lm -o spmm_example
 *
 * Exit code 0 and "ok" on success; any status other than SPX_OK is printed with spx_last_error().
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "spx_b200.h"

#define CHECK(call)                                                                  \
    do {                                                                             \
        int st_ = (call);                                                            \
        if (st_ != SPX_OK) {                                                         \
            fprintf(stderr, "%s -> status %d: %s\n", #call, st_, spx_last_error()); \
            return 1;                                                                \
        }                                                                            \
    } while (0)

int main(void)
{
    enum { M = 37, N = 53, C = 20 };
    static float W[M][N], X[N][C], bias[M], Y[M][C], Y2[M][C], want[M][C];
    unsigned seed = 12345u;
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            seed = seed * 1664525u + 1013904223u;
            W[i][j] = (seed >> 28) == 0 ? (float)((int)(seed >> 8 & 0xff) - 128) / 64.0f : 0.0f;   /* ~6 % dense */
        }
    for (int j = 0; j < N; ++j)
        for (int c = 0; c < C; ++c) X[j][c] = (float)((j * 7 + c * 3) % 11) / 11.0f - 0.5f;
    for (int i = 0; i < M; ++i) bias[i] = 0.25f * (float)(i % 5);

    /* ELLPACK encoding on the host: count, then pack in ascending column order */
    unsigned nnz[M], r = 0;
    for (int i = 0; i < M; ++i) {
        nnz[i] = 0;
        for (int j = 0; j < N; ++j) nnz[i] += W[i][j] != 0.0f;
        if (nnz[i] > r) r = nnz[i];
    }
    float* Wd = calloc((size_t)M * (r ? r : 1), sizeof(float));
    unsigned* idx = calloc((size_t)M * (r ? r : 1), sizeof(unsigned));
    for (int i = 0; i < M; ++i) {
        unsigned pos = 0;
        for (int j = 0; j < N; ++j)
            if (W[i][j] != 0.0f) { Wd[i * r + pos] = W[i][j]; idx[i * r + pos] = (unsigned)j; ++pos; }
    }
    /* the reference result: bias first, then one fused multiply-add per stored entry, ReLU */
    for (int i = 0; i < M; ++i)
        for (int c = 0; c < C; ++c) {
            float y = bias[i];
            for (unsigned t = 0; t < nnz[i]; ++t) y = fmaf(Wd[i * r + t], X[idx[i * r + t]][c], y);
            want[i][c] = y > 0.0f ? y : 0.0f;
        }

    spx_ell* e = NULL;
    CHECK(spx_set_device(0));
    CHECK(spx_ell_create(M, N, r, Wd, idx, nnz, &e));
    CHECK(spx_spmm_host(e, &X[0][0], C, bias, SPX_ACT_RELU, &Y[0][0]));

    float *dX = NULL, *dB = NULL, *dY = NULL;
    void* stream = NULL;
    CHECK(spx_stream_create(&stream));
    CHECK(spx_malloc((void**)&dX, sizeof(X)));
    CHECK(spx_malloc((void**)&dB, sizeof(bias)));
    CHECK(spx_malloc((void**)&dY, sizeof(Y2)));
    CHECK(spx_memcpy_h2d(dX, X, sizeof(X), stream));
    CHECK(spx_memcpy_h2d(dB, bias, sizeof(bias), stream));
    CHECK(spx_spmm(e, dX, C, C, dB, SPX_ACT_RELU, dY, C, stream));
    CHECK(spx_memcpy_d2h(Y2, dY, sizeof(Y2), stream));
    CHECK(spx_stream_sync(stream));

    if (memcmp(Y, want, sizeof(Y)) != 0 || memcmp(Y2, want, sizeof(Y2)) != 0) {
        fprintf(stderr, "result differs from the scalar loop\n");
        return 2;
    }
    CHECK(spx_free(dX));
    CHECK(spx_free(dB));
    CHECK(spx_free(dY));
    CHECK(spx_stream_destroy(stream));
    CHECK(spx_ell_destroy(e));
    free(Wd);
    free(idx);
    printf("ok: %llu kernels launched\n", (unsigned long long)spx_launch_count());
    return 0;
}
