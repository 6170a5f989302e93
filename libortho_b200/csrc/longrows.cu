// Sparse sums of the plan's long rows for the prefill regime, computed ahead of the tensor-core kernel:
//
//     OL[h][m] = sum over the entries i of long row hrow[h] of v_i * x[m, c_i]            (FP32)
//
// A layer whose entries pile up in a few rows (power-law row loads) has rows with thousands of entries; inside
// the tensor-core kernel one warp walks a row, so such a row would hold up its whole tile.  Here every segment
// of at most kLongSeg entries gets a CTA per block of 256 tokens: its eight warps take the segment's 32-entry
// batches in turn (eight 16-byte gathers in flight per lane from the transposed activations), their partial sums
// meet in shared memory in warp order, and a second kernel adds a row's segments in segment order.  No atomics:
// the result does not depend on scheduling.  The reference walks every coordinate serially per token
// (src/ortho.c:384-398).
#include "common.cuh"

namespace ob {

constexpr int kLrTok = 256;

__global__ void __launch_bounds__(256)
long_segments_kernel(const OrthoView ov, const int32_t *__restrict__ vbeg, const int32_t *__restrict__ vend,
                     const __half *__restrict__ xt, float *__restrict__ part_out, int K, int Mp)
{
    __shared__ float part[8][kLrTok];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int v = blockIdx.x;
    const int tok0 = blockIdx.y * kLrTok;
    const int e0 = vbeg[v], e1 = vend[v];
    const __half *xbase = xt + tok0 + lane * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int eb = e0 + warp * 32; eb < e1; eb += 8 * 32) {
        int cl = 0; float vl = 0.f;
        if (eb + lane < e1) ortho_entry(ov, eb + lane, K, cl, vl);
        const int nb = min(32, e1 - eb);
        for (int j0 = 0; j0 < nb; j0 += 8) {
            uint4 xv[8]; float vv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c = __shfl_sync(0xffffffffu, cl, (j0 + j) & 31);
                vv[j] = __shfl_sync(0xffffffffu, vl, (j0 + j) & 31);      // slots past the batch hold v = 0, c = 0
                xv[j] = *reinterpret_cast<const uint4 *>(xbase + (size_t)c * Mp);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const __half2 *h = reinterpret_cast<const __half2 *>(&xv[j]);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 f = __half22float2(h[q]);
                    acc[2 * q] = fmaf(vv[j], f.x, acc[2 * q]);
                    acc[2 * q + 1] = fmaf(vv[j], f.y, acc[2 * q + 1]);
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < 8; q++) part[warp][lane * 8 + q] = acc[q];
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) s += part[w][threadIdx.x];
    part_out[(size_t)v * Mp + tok0 + threadIdx.x] = s;
}

__global__ void __launch_bounds__(256)
long_combine_kernel(const int32_t *__restrict__ hptr, const float *__restrict__ part, float *__restrict__ ol, int Mp)
{
    const int h = blockIdx.x;
    const int m = blockIdx.y * 256 + threadIdx.x;
    const int v0 = hptr[h], v1 = hptr[h + 1];
    const float *src = part + m;
    float s = 0.f;
    int v = v0;
    for (; v + 4 <= v1; v += 4) {          // four loads in flight, added in segment order
        float t[4];
#pragma unroll
        for (int i = 0; i < 4; i++) t[i] = src[(size_t)(v + i) * Mp];
#pragma unroll
        for (int i = 0; i < 4; i++) s += t[i];
    }
    for (; v < v1; v++) s += src[(size_t)v * Mp];
    ol[(size_t)h * Mp + m] = s;
}

static int64_t lr_mp(int64_t M) { return ceil_div(M, kLrTok) * kLrTok; }

// [ OL : n_long * Mp floats ][ per-segment partial sums : n_seg * Mp floats ]
int64_t long_rows_workspace_bytes(const Plan *pl, int64_t M)
{
    if (!pl || pl->n_long == 0) return 0;
    return (((pl->n_long + pl->n_seg) * lr_mp(M) * 4 + 255) / 256) * 256;
}

// xt: transposed activations [K][Mp]; ws: long_rows_workspace_bytes() bytes, 256-byte aligned.  *ol_out = OL.
int launch_long_rows(const FwdArgs &a, const __half *xt, int Mp, void *ws, const float **ol_out)
{
    const Plan *pl = a.plan;
    float *ol = reinterpret_cast<float *>(ws);
    float *part = ol + (size_t)pl->n_long * Mp;
    dim3 g1((unsigned)pl->n_seg, (unsigned)(Mp / kLrTok));
    long_segments_kernel<<<g1, 256, 0, a.stream>>>(a.ortho, pl->vbeg, pl->vend, xt, part, (int)a.K, Mp);
    count_launch();
    OB_CUDA(cudaGetLastError());
    dim3 g2((unsigned)pl->n_long, (unsigned)(Mp / 256));
    long_combine_kernel<<<g2, 256, 0, a.stream>>>(pl->hptr, part, ol, Mp);
    count_launch();
    OB_CUDA(cudaGetLastError());
    *ol_out = ol;
    return ORTHO_B200_OK;
}

}  // namespace ob
