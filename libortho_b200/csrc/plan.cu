// Plan: one-time GPU-side re-layout of a layer's sparse ortho component, and the two probe
// kernels that let a test prove the integer/index handling bit-exact.
//
// The reference kernels read CSR as three separate streams per row (row_ptr, then col_indices
// and float values; src/dual_gemm.cu:106-130).  The re-layout keeps the CSR row-major order
// (tools/sieve.py:131-136) but fuses column and value into one 32-bit word per entry
// ({f16 value bits | 16-bit column}; an entry outside [0, K) becomes an explicit zero) and keeps its own
// copy of the row pointers, so that every kernel reads one word per entry instead of two.
#include <new>
#include <vector>

#include "common.cuh"

namespace ob {

// one warp per output row: pack the row's entries, track the longest row, the largest magnitude of every row
// (NaN counts as infinite) and whether every row lists its columns in strictly ascending order inside [0, K)
// (info[0] = longest row, info[1] != 0: some row does not)
__global__ void relayout_rows_kernel(const int32_t *__restrict__ row_ptr, const int32_t *__restrict__ col,
                                     const __half *__restrict__ val, int N, int K,
                                     uint32_t *__restrict__ entries, int32_t *__restrict__ row_ptr_copy,
                                     float *__restrict__ row_max, int *__restrict__ info)
{
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    for (int n = blockIdx.x * warps_per_block + (threadIdx.x >> 5); n <= N; n += gridDim.x * warps_per_block) {
        const int e0 = row_ptr[n];
        if (lane == 0) row_ptr_copy[n] = e0;
        if (n == N) continue;
        const int e1 = row_ptr[n + 1];
        float vmax = 0.f;
        bool unordered = false;
        for (int e = e0 + lane; e < e1; e += 32) {
            int c = col[e];
            unsigned short vb = __half_as_ushort(val[e]);
            if (e > e0 && col[e - 1] >= c) unordered = true;
            // an entry outside [0,K) is skipped by the reference (src/ortho.c:394); store it as an
            // explicit zero so that it contributes nothing
            if ((unsigned)c >= (unsigned)K) { c = 0; vb = 0; unordered = true; }
            const float av = fabsf(__half2float(__ushort_as_half(vb)));
            vmax = (av != av) ? __int_as_float(0x7f800000) : fmaxf(vmax, av);
            entries[e] = ((uint32_t)vb << 16) | (uint32_t)c;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        unordered = __any_sync(0xffffffffu, unordered);
        if (lane == 0) {
            row_max[n] = vmax;
            atomicMax(&info[0], e1 - e0);
            if (unordered) atomicExch(&info[1], 1);
        }
    }
}

// one warp per output row: the row of an entry is recovered from the plan's own row pointers
__global__ void plan_decode_dump_kernel(const uint32_t *__restrict__ entries, const int32_t *__restrict__ row_ptr,
                                        int N, int32_t *__restrict__ rows, int32_t *__restrict__ cols,
                                        __half *__restrict__ vals)
{
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    for (int n = blockIdx.x * warps_per_block + (threadIdx.x >> 5); n < N; n += gridDim.x * warps_per_block) {
        const int e0 = row_ptr[n], e1 = row_ptr[n + 1];
        for (int e = e0 + lane; e < e1; e += 32) {
            const uint32_t pk = entries[e];
            rows[e] = n;
            cols[e] = (int32_t)(pk & 0xFFFFu);
            vals[e] = __ushort_as_half((unsigned short)(pk >> 16));
        }
    }
}

// every thread unpacks one 32-bit word (8 elements) with the forward kernels' own converters:
// elements 0..7 come back from the pair-order converter, and the natural-order converter of the tensor-core
// kernels must agree with it, otherwise a poison value is written.
__global__ void dequant_dump_kernel(const uint32_t *__restrict__ w32, const __half *__restrict__ scales,
                                    int64_t N, int64_t K, int8_t *__restrict__ w_int, float *__restrict__ w_deq)
{
    const int64_t words_per_row = K >> 3;
    const int64_t total = N * words_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / words_per_row;
        const uint32_t w = w32[i];
        uint32_t hp[4], hn[4];
        int4x8_to_half2x4(w, hp);
        int4x8_to_half2x4_natural(w, hn);
        float e[8];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const __half2 pr = *reinterpret_cast<const __half2 *>(&hp[q]);
            e[q] = __low2float(pr);        // pair q = (e_q, e_{q+4})
            e[q + 4] = __high2float(pr);
        }
        bool agree = true;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const __half2 pr = *reinterpret_cast<const __half2 *>(&hn[q]);
            agree = agree && (__low2float(pr) == e[2 * q]) && (__high2float(pr) == e[2 * q + 1]);
        }
        const float s = __half2float(scales[n]);
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const float v = agree ? e[q] : 127.f;
            if (w_int) w_int[i * 8 + q] = (int8_t)v;
            if (w_deq) w_deq[i * 8 + q] = __fmul_rn(v, s);
        }
    }
}

}  // namespace ob

using namespace ob;

extern "C" int ortho_b200_plan_create(ortho_b200_plan **plan_out, const int32_t *row_ptr,
                                      const int32_t *col_indices, const void *values_f16, int64_t nnz,
                                      int64_t in_features, int64_t out_features, void *stream)
{
    if (!plan_out) return ORTHO_B200_ERR_NULL;
    *plan_out = nullptr;
    const int64_t K = in_features, N = out_features;
    if (K <= 0 || N <= 0 || nnz < 0 || K > 65536 || (K % 32) != 0 || nnz > 0x7fffffffLL || N > 0x7fffff00LL)
        return ORTHO_B200_ERR_SHAPE;
    if (nnz > 0 && (!row_ptr || !col_indices || !values_f16)) return ORTHO_B200_ERR_NULL;
    Plan *pl = new (std::nothrow) Plan();
    if (!pl) return ORTHO_B200_ERR_ALLOC;
    pl->magic = kPlanMagic; pl->K = K; pl->N = N; pl->nnz = nnz; pl->max_row_nnz = 0;
    pl->row_ptr = nullptr; pl->entries = nullptr; pl->row_max = nullptr; pl->ordered = false;
    pl->heavy = kLongRowMin; pl->n_long = 0; pl->n_pad = 0;
    pl->hrow = nullptr; pl->hdense = nullptr;
    cudaError_t e = cudaGetDevice(&pl->device);
    if (e != cudaSuccess) { note_cuda_error(e); delete pl; return ORTHO_B200_ERR_CUDA; }
    if (nnz > 0) {
        cudaStream_t st = (cudaStream_t)stream;
        int *d_max = nullptr;
        e = cudaMalloc(&pl->row_ptr, sizeof(int32_t) * (N + 1));
        if (e == cudaSuccess) e = cudaMalloc(&pl->entries, sizeof(uint32_t) * nnz);
        if (e == cudaSuccess) e = cudaMalloc(&pl->row_max, sizeof(float) * N);
        if (e == cudaSuccess) e = cudaMalloc(&d_max, 2 * sizeof(int));
        if (e == cudaSuccess) e = cudaMemsetAsync(d_max, 0, 2 * sizeof(int), st);
        if (e == cudaSuccess) {
            const int threads = 256, wpb = threads / 32;
            int64_t blocks = ceil_div(N + 1, wpb);
            if (blocks > 148 * 16) blocks = 148 * 16;
            relayout_rows_kernel<<<(unsigned)blocks, threads, 0, st>>>(
                row_ptr, col_indices, (const __half *)values_f16, (int)N, (int)K, pl->entries, pl->row_ptr, pl->row_max, d_max);
            count_launch();
            e = cudaGetLastError();
        }
        int h_info[2] = {0, 0};
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_info, d_max, 2 * sizeof(int), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (d_max) cudaFree(d_max);
        if (e != cudaSuccess) {
            note_cuda_error(e);
            ortho_b200_plan_destroy(reinterpret_cast<ortho_b200_plan *>(pl));
            return ORTHO_B200_ERR_CUDA;
        }
        const int h_max = h_info[0];
        pl->max_row_nnz = h_max;
        pl->ordered = h_info[1] == 0;
        const int64_t mean = (nnz + N - 1) / N;
        const int lmin = tuning_snapshot().long_row_min;
        pl->heavy = (int)(4 * mean > lmin ? (4 * mean > 65536 ? 65536 : 4 * mean) : lmin);
        if (h_max > pl->heavy) {
            // list the long rows on the host (one pass over the row pointers); the threshold doubles until their
            // dense copy fits its budget
            std::vector<int32_t> rp((size_t)N + 1), hr;
            e = cudaMemcpy(rp.data(), row_ptr, sizeof(int32_t) * (N + 1), cudaMemcpyDeviceToHost);
            if (e == cudaSuccess) {
                for (;;) {
                    hr.clear();
                    for (int64_t n = 0; n < N; n++)
                        if (rp[n + 1] - rp[n] > pl->heavy) hr.push_back((int32_t)n);
                    const int64_t n_pad = ((int64_t)hr.size() + 127) / 128 * 128;
                    if (n_pad * K * 2 <= kLongDenseMaxBytes || pl->heavy >= 65536) break;
                    pl->heavy *= 2;
                }
                const size_t nl = hr.size();
                if (nl > 0 && (int64_t)((nl + 127) / 128 * 128) * K * 2 <= kLongDenseMaxBytes) {
                    e = cudaMalloc(&pl->hrow, sizeof(int32_t) * nl);
                    if (e == cudaSuccess) e = cudaMemcpy(pl->hrow, hr.data(), sizeof(int32_t) * nl, cudaMemcpyHostToDevice);
                    if (e == cudaSuccess) {
                        pl->n_long = (int64_t)nl;
                        bool dup = false;
                        e = (cudaError_t)plan_build_long_rows(pl, st, &dup);
                        if (e == cudaSuccess && dup) {         // a repeated column: every row stays with the in-kernel pass
                            cudaFree(pl->hdense); pl->hdense = nullptr;
                            cudaFree(pl->hrow); pl->hrow = nullptr;
                            pl->n_long = 0; pl->n_pad = 0;
                        }
                    }
                }
            }
            if (e != cudaSuccess) {
                note_cuda_error(e);
                ortho_b200_plan_destroy(reinterpret_cast<ortho_b200_plan *>(pl));
                return ORTHO_B200_ERR_CUDA;
            }
        }
    }
    *plan_out = reinterpret_cast<ortho_b200_plan *>(pl);
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_plan_destroy(ortho_b200_plan *plan)
{
    Plan *pl = reinterpret_cast<Plan *>(plan);
    if (!pl) return ORTHO_B200_OK;
    if (pl->magic != kPlanMagic) return ORTHO_B200_ERR_PLAN;
    if (pl->row_ptr) cudaFree(pl->row_ptr);
    if (pl->entries) cudaFree(pl->entries);
    if (pl->row_max) cudaFree(pl->row_max);
    if (pl->hrow) cudaFree(pl->hrow);
    if (pl->hdense) cudaFree(pl->hdense);
    pl->magic = 0;
    delete pl;
    return ORTHO_B200_OK;
}

extern "C" int64_t ortho_b200_plan_nnz(const ortho_b200_plan *plan)
{
    const Plan *pl = reinterpret_cast<const Plan *>(plan);
    return (pl && pl->magic == kPlanMagic) ? pl->nnz : -1;
}

extern "C" int64_t ortho_b200_plan_max_row_nnz(const ortho_b200_plan *plan)
{
    const Plan *pl = reinterpret_cast<const Plan *>(plan);
    return (pl && pl->magic == kPlanMagic) ? pl->max_row_nnz : -1;
}

extern "C" int ortho_b200_plan_rows_ordered(const ortho_b200_plan *plan)
{
    const Plan *pl = reinterpret_cast<const Plan *>(plan);
    if (!pl || pl->magic != kPlanMagic) return -1;
    return (pl->nnz == 0 || pl->ordered) ? 1 : 0;
}

extern "C" int64_t ortho_b200_plan_workspace_bytes(const ortho_b200_plan *plan, int64_t M)
{
    const Plan *pl = reinterpret_cast<const Plan *>(plan);
    if (!pl || pl->magic != kPlanMagic) return -1;
    if (pl->nnz == 0) return 0;
    const int64_t plain = ortho_b200_workspace_bytes(M, pl->K, pl->N);
    // the tensor-core prefill kernel takes the sums of the plan's long rows from a pre-pass
    return plain + (decode_regime(M, pl->N, pl->K) ? 0 : long_rows_workspace_bytes(pl, M));
}

extern "C" int ortho_b200_plan_decode_dump(const ortho_b200_plan *plan, int32_t *rows_out, int32_t *cols_out,
                                           void *values_f16_out, void *stream)
{
    const Plan *pl = reinterpret_cast<const Plan *>(plan);
    if (!pl || pl->magic != kPlanMagic) return ORTHO_B200_ERR_PLAN;
    if (pl->nnz == 0) return ORTHO_B200_OK;
    if (!rows_out || !cols_out || !values_f16_out) return ORTHO_B200_ERR_NULL;
    int64_t blocks = ceil_div(pl->N, 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    plan_decode_dump_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        pl->entries, pl->row_ptr, (int)pl->N, rows_out, cols_out, (__half *)values_f16_out);
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_dequant_dump(const void *q_weight, const void *q_scales_f16, int64_t out_features,
                                       int64_t in_features, int8_t *w_int_out, float *w_deq_out, void *stream)
{
    if (!q_weight || !q_scales_f16) return ORTHO_B200_ERR_NULL;
    if (out_features <= 0 || in_features <= 0 || (in_features % 8) != 0) return ORTHO_B200_ERR_SHAPE;
    if (((uintptr_t)q_weight & 3u) != 0) return ORTHO_B200_ERR_ALIGN;
    if (!w_int_out && !w_deq_out) return ORTHO_B200_OK;
    const int64_t total = out_features * (in_features / 8);
    int64_t blocks = ceil_div(total, 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    dequant_dump_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint32_t *)q_weight, (const __half *)q_scales_f16, out_features, in_features, w_int_out, w_deq_out);
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}
