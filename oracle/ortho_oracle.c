/*
 * CPU oracle for the OrthoLinear forward
 *
 *     Y[M,N] = X[M,K] . dequant(W_base_int4[N,K])^T  +  alpha . X[M,K] . W_ortho[N,K]^T
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference's CPU
 * algorithm and exists to check the CUDA kernels and to time a CPU baseline.  Nothing in
 * the shipped library links, loads or calls it; only the test-suite, the smoke entry and
 * the benchmark's cpu_baseline / reference legs do.
 *
 * Parity status: PINNED.  The restatement is compared bit-for-bit with the reference's own
 * compiled src/ortho.c (see ref_harness.c in this directory) on the reference's three
 * known-answer cases (tests/test_cpu_forward.c:147-334) and on seeded cases of the benchmark
 * shapes; the resulting vectors are committed under tests/golden/.
 *
 * Each function cites the reference lines it follows (paths relative to the reference tree).
 */

#define _POSIX_C_SOURCE 200809L
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------
 * INT4 unpack.  Follows src/ortho.c:315-325 (same rule in src/dual_gemm.cu:30-40 and
 * tests/test_cpu_forward.c:21-28): element idx lives in byte idx/2, low nibble when idx is
 * even, high nibble when odd; the nibble is a 4-bit two's-complement integer in [-8, 7].
 * ------------------------------------------------------------------------------------------ */
static inline int oracle_nibble(const uint8_t *packed, size_t idx)
{
    unsigned b = packed[idx >> 1];
    unsigned nib = (idx & 1u) ? (b >> 4) : (b & 0x0Fu);
    return (int)nib - (int)((nib & 0x8u) << 1);
}

int8_t oracle_unpack_int4(const uint8_t *packed, size_t idx)
{
    return (int8_t)oracle_nibble(packed, idx);
}

/* Raw integers and the FP32 dequantised weight (float)w_int * scale[row] for every element.
 * The product follows src/ortho.c:363 exactly (int -> float, then one FP32 multiply). */
int oracle_dequant(const uint8_t *packed, const float *scales, size_t N, size_t K,
                   int8_t *w_int_out, float *w_deq_out)
{
    if (!packed || !scales) return -1;
    for (size_t n = 0; n < N; n++) {
        float s = scales[n];
        for (size_t k = 0; k < K; k++) {
            int w = oracle_nibble(packed, n * K + k);
            if (w_int_out) w_int_out[n * K + k] = (int8_t)w;
            if (w_deq_out) w_deq_out[n * K + k] = (float)w * s;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Base term for a range of output rows of one token.  Follows src/ortho.c:354-366:
 *     acc = 0;  for k in 0..K-1:  acc += x[k] * ((float)w_int * scale);   y[n] = acc
 * The sum is strictly left to right in FP32 (build without -ffast-math).  Four rows are
 * walked side by side only to give the CPU independent add chains; every row keeps its own
 * accumulator and its own k order, so the result per element is the reference's.
 * ------------------------------------------------------------------------------------------ */
static void base_rows(const uint8_t *packed, const float *scales, const float *x, float *y,
                      size_t K, size_t n0, size_t n1)
{
    size_t n = n0;
    for (; n + 4 <= n1; n += 4) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        float s0 = scales[n], s1 = scales[n + 1], s2 = scales[n + 2], s3 = scales[n + 3];
        size_t b0 = n * K, b1 = b0 + K, b2 = b1 + K, b3 = b2 + K;
        for (size_t k = 0; k < K; k++) {
            float xv = x[k];
            a0 += xv * ((float)oracle_nibble(packed, b0 + k) * s0);
            a1 += xv * ((float)oracle_nibble(packed, b1 + k) * s1);
            a2 += xv * ((float)oracle_nibble(packed, b2 + k) * s2);
            a3 += xv * ((float)oracle_nibble(packed, b3 + k) * s3);
        }
        y[n] = a0; y[n + 1] = a1; y[n + 2] = a2; y[n + 3] = a3;
    }
    for (; n < n1; n++) {
        float acc = 0.f, s = scales[n];
        size_t b = n * K;
        for (size_t k = 0; k < K; k++)
            acc += x[k] * ((float)oracle_nibble(packed, b + k) * s);
        y[n] = acc;
    }
}

/* ------------------------------------------------------------------------------------------
 * Forward with the ortho term given as CSR (the layout the operator API passes,
 * torch_bind/ortho_linear.py:142-151).  The reference CPU forward walks a row-major sorted
 * coordinate list and adds one entry at a time after the base sum (src/ortho.c:384-398):
 *     if (alpha > 0 && count > 0)  for each entry:  y[row] += alpha * value * x[col]
 * A CSR produced by tools/sieve.py:119-152 lists exactly that order, so walking the rows in
 * order and each row's entries in order reproduces the same sequence of FP32 additions.
 * Entries whose column is outside [0,K) are skipped like the range check at src/ortho.c:394.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    const uint8_t *packed; const float *scales;
    const int32_t *row_ptr; const int32_t *col; const float *vals; int64_t nnz;
    const float *x; float *y; size_t M, K, N; float alpha;
    size_t m0, m1, n0, n1;
} oracle_job;

static void run_job(const oracle_job *j)
{
    int has_ortho = (j->alpha > 0.0f && j->nnz > 0 && j->row_ptr && j->col && j->vals);
    for (size_t m = j->m0; m < j->m1; m++) {
        const float *x = j->x + m * j->K;
        float *y = j->y + m * j->N;
        base_rows(j->packed, j->scales, x, y, j->K, j->n0, j->n1);
        if (has_ortho) {
            for (size_t n = j->n0; n < j->n1; n++) {
                for (int32_t i = j->row_ptr[n]; i < j->row_ptr[n + 1]; i++) {
                    int32_t c = j->col[i];
                    if (c >= 0 && (size_t)c < j->K)
                        y[n] += j->alpha * j->vals[i] * x[c];
                }
            }
        }
    }
}

static void *job_thread(void *p) { run_job((const oracle_job *)p); return NULL; }

/* nthreads <= 1 runs inline.  Work is split over tokens when M >= nthreads, otherwise over
 * row ranges; either split leaves every output element's arithmetic untouched because
 * tokens and rows are independent in the reference (src/ortho.c:346-349, 354-366, 389-396). */
int oracle_forward_csr(const uint8_t *packed, const float *scales,
                       const int32_t *row_ptr, const int32_t *col, const float *vals, int64_t nnz,
                       const float *x, float *y, size_t M, size_t K, size_t N, float alpha,
                       int nthreads)
{
    if (!packed || !scales || !x || !y) return -1;          /* src/ortho.c:331-333 */
    oracle_job base = { packed, scales, row_ptr, col, vals, nnz, x, y, M, K, N, alpha, 0, M, 0, N };
    if (nthreads <= 1 || (M <= 1 && N < 8)) { run_job(&base); return 0; }
    if (nthreads > 256) nthreads = 256;
    oracle_job jobs[256]; pthread_t th[256];
    int nj = 0;
    if (M >= (size_t)nthreads) {
        for (int t = 0; t < nthreads; t++) {
            jobs[nj] = base;
            jobs[nj].m0 = M * (size_t)t / (size_t)nthreads;
            jobs[nj].m1 = M * (size_t)(t + 1) / (size_t)nthreads;
            if (jobs[nj].m1 > jobs[nj].m0) nj++;
        }
    } else {
        for (int t = 0; t < nthreads; t++) {
            jobs[nj] = base;
            jobs[nj].n0 = N * (size_t)t / (size_t)nthreads;
            jobs[nj].n1 = N * (size_t)(t + 1) / (size_t)nthreads;
            if (jobs[nj].n1 > jobs[nj].n0) nj++;
        }
    }
    for (int t = 1; t < nj; t++) pthread_create(&th[t], NULL, job_thread, &jobs[t]);
    run_job(&jobs[0]);
    for (int t = 1; t < nj; t++) pthread_join(th[t], NULL);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Forward with the ortho term as the legacy 16-bit coordinate list, exactly as the reference
 * CPU forward consumes it (src/ortho.c:384-398): flat = row*K + col in a uint16, entries
 * applied in list order, duplicates allowed, out-of-range entries skipped.  Used to replay
 * the reference's own known-answer cases (tests/test_cpu_forward.c:132-141).
 * ------------------------------------------------------------------------------------------ */
int oracle_forward_coo16(const uint8_t *packed, const float *scales,
                         const uint16_t *flat_idx, const float *vals, int count,
                         const float *x, float *y, size_t M, size_t K, size_t N, float alpha)
{
    if (!packed || !scales || !x || !y) return -1;
    int has_ortho = (alpha > 0.0f && count > 0);
    for (size_t m = 0; m < M; m++) {
        const float *xr = x + m * K;
        float *yr = y + m * N;
        base_rows(packed, scales, xr, yr, K, 0, N);
        if (has_ortho) {
            for (int i = 0; i < count; i++) {
                size_t f = flat_idx[i];
                size_t row = f / K, c = f % K;
                if (row < N && c < K)
                    yr[row] += alpha * vals[i] * xr[c];
            }
        }
    }
    return 0;
}
