/*
 * Harness around the reference's own, unmodified CPU forward.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is compiled together with the reference's
 * src/ortho.c (taken from the reference tree where it lies, never copied) into
 * oracle/_ref/libortho_ref*.so by the Makefile in this directory.  It is used to pin the
 * restatement in ortho_oracle.c, to generate the committed golden vectors, and as the timed
 * CPU baseline of the benchmark.  The shipped library never loads it.
 *
 * What it works around: orth_layer_forward (src/ortho.c:327-402) only reads the legacy
 * coordinate list, whose flat index row*K+col is a uint16 (include/ortho.h:49,
 * src/ortho.c:386-392).  A layer with N*K > 65536 therefore cannot be expressed in one call.
 * Output rows are independent in that function (src/ortho.c:354-366, 389-396), so the
 * harness calls it on chunks of R = floor(65536 / K) consecutive rows, each chunk with its
 * own layer view {q_weight + r0*K/2, q_scales + r0, in=K, out=rows}, chunk-local uint16
 * indices, format 0, and scatters the chunk's [M, rows] output into [M, N].  Chunking changes
 * no arithmetic of any output element.
 */

#define _POSIX_C_SOURCE 200809L
#include "ortho.h"
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* direct call for the reference's own known-answer layout (16-bit coordinate list) */
int ref_forward_coo16(const uint8_t *packed, const float *scales,
                      const uint16_t *flat_idx, const float *vals, int count,
                      const float *x, float *y, size_t M, size_t K, size_t N, float alpha)
{
    orth_layer_t layer;
    memset(&layer, 0, sizeof(layer));
    layer.base.q_weight = (void *)packed;
    layer.base.q_scales = (void *)scales;
    layer.base.q_bits = 4;
    layer.base.in_features = K;
    layer.base.out_features = N;
    layer.ortho.indices = (uint16_t *)flat_idx;
    layer.ortho.values = (float *)vals;
    layer.ortho.count = count;
    layer.ortho.format = 0;
    layer.alpha = alpha;
    return orth_layer_forward(&layer, x, y, M);
}

typedef struct {
    const uint8_t *packed; const float *scales;
    const int32_t *row_ptr; const int32_t *col; const float *vals;
    const float *x; float *y; size_t M, K, N; float alpha;
    size_t rows_per_chunk, chunk0, chunk1;
    int status;
} ref_job;

static void *ref_worker(void *p)
{
    ref_job *j = (ref_job *)p;
    size_t R = j->rows_per_chunk;
    float *ytmp = (float *)malloc(sizeof(float) * j->M * R);
    uint16_t *idx = (uint16_t *)malloc(sizeof(uint16_t) * (R * j->K + 1));
    float *val = (float *)malloc(sizeof(float) * (R * j->K + 1));
    if (!ytmp || !idx || !val) { j->status = -1; free(ytmp); free(idx); free(val); return NULL; }
    for (size_t c = j->chunk0; c < j->chunk1; c++) {
        size_t r0 = c * R, r1 = r0 + R;
        if (r1 > j->N) r1 = j->N;
        size_t rows = r1 - r0;
        int count = 0;
        if (j->row_ptr && j->col && j->vals) {
            for (size_t r = r0; r < r1; r++)
                for (int32_t i = j->row_ptr[r]; i < j->row_ptr[r + 1]; i++) {
                    idx[count] = (uint16_t)((r - r0) * j->K + (size_t)j->col[i]);
                    val[count] = j->vals[i];
                    count++;
                }
        }
        orth_layer_t layer;
        memset(&layer, 0, sizeof(layer));
        layer.base.q_weight = (void *)(j->packed + r0 * j->K / 2);
        layer.base.q_scales = (void *)(j->scales + r0);
        layer.base.q_bits = 4;
        layer.base.in_features = j->K;
        layer.base.out_features = rows;
        layer.ortho.indices = idx;
        layer.ortho.values = val;
        layer.ortho.count = count;
        layer.ortho.format = 0;
        layer.alpha = j->alpha;
        if (orth_layer_forward(&layer, j->x, ytmp, j->M) != 0) { j->status = -1; break; }
        for (size_t m = 0; m < j->M; m++)
            memcpy(j->y + m * j->N + r0, ytmp + m * rows, sizeof(float) * rows);
    }
    free(ytmp); free(idx); free(val);
    return NULL;
}

/* CSR in, row-chunked calls of the unmodified reference forward, chunks spread over threads */
int ref_forward_csr(const uint8_t *packed, const float *scales,
                    const int32_t *row_ptr, const int32_t *col, const float *vals, int64_t nnz,
                    const float *x, float *y, size_t M, size_t K, size_t N, float alpha,
                    int nthreads)
{
    (void)nnz;
    if (!packed || !scales || !x || !y || K == 0 || K > 65536 || (K & 1)) return -1;
    size_t R = 65536 / K;
    if (R * K > 65536 || R == 0) return -1;
    /* the last flat index of a chunk, R*K-1, must fit a uint16 */
    size_t nchunks = (N + R - 1) / R;
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 256) nthreads = 256;
    if ((size_t)nthreads > nchunks) nthreads = (int)nchunks;
    ref_job jobs[256]; pthread_t th[256];
    for (int t = 0; t < nthreads; t++) {
        ref_job j = { packed, scales, row_ptr, col, vals, x, y, M, K, N, alpha, R,
                      nchunks * (size_t)t / (size_t)nthreads,
                      nchunks * (size_t)(t + 1) / (size_t)nthreads, 0 };
        jobs[t] = j;
    }
    for (int t = 1; t < nthreads; t++) pthread_create(&th[t], NULL, ref_worker, &jobs[t]);
    ref_worker(&jobs[0]);
    int status = jobs[0].status;
    for (int t = 1; t < nthreads; t++) { pthread_join(th[t], NULL); if (jobs[t].status) status = -1; }
    return status;
}

/* lifecycle smoke: init / alloc / set_alpha / free of the reference, returns 0 when the
 * buffers come back 128-byte aligned as include/ortho.h:19-21 promises */
int ref_lifecycle_check(size_t K, size_t N, size_t nnz)
{
    orth_layer_t layer;
    if (orth_layer_init(&layer, K, N, 4) != 0) return -1;
    int ok = (((uintptr_t)layer.base.q_weight & 127u) == 0) && (((uintptr_t)layer.base.q_scales & 127u) == 0);
    if (nnz && orth_layer_alloc_ortho_csr(&layer, nnz, N) != 0) ok = 0;
    if (nnz && layer.ortho.format != 1) ok = 0;
    orth_layer_set_alpha(&layer, 0.25f);
    if (layer.alpha != 0.25f) ok = 0;
    orth_layer_free(&layer);
    return ok ? 0 : -2;
}
