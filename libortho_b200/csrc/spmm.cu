// Sparse ortho term for the prefill regime, computed ahead of the tensor-core kernel:
//
//     O[n, m] = sum_{i in row n} v_i * x[m, c_i]            (FP32, alpha is applied in the epilogue)
//
// The reference adds this term one coordinate at a time per token (src/ortho.c:384-398) or, on the
// GPU, scans the coordinate list per output element (src/dual_gemm_tensor_core.cu:180-207).  Here
// the activations are first transposed once per forward (Xt[k][m]) so that one sparse entry touches
// a contiguous run of tokens; a warp then walks one output row's entries and keeps 8 tokens per
// lane in FP32 registers, so every entry costs one 16-byte load and 8 FMAs per lane.  Rows longer
// than SpmmParams::heavy entries are split over the 8 warps of the CTA and their partial sums are combined in
// shared memory in a fixed order, so the result does not depend on scheduling.  The tensor-core
// kernel's epilogue adds alpha * O to scale * D before the single FP16 rounding.
#include "common.cuh"

namespace ob {

constexpr int kSpTok = 256;       // tokens per CTA (8 per lane)
constexpr int kSpRows = 8;        // warps per CTA; each warp owns 8 consecutive rows

// X[M][K] (FP16) -> Xt[K][Mp] (FP16), zero padded for m >= M.  64 x 64 tiles; 16-byte global loads
// along k, 16-byte global stores along m, transposition through a padded shared tile.
__global__ void __launch_bounds__(256)
transpose_x_kernel(const __half *__restrict__ x, __half *__restrict__ xt, int M, int K, int Mp)
{
    __shared__ __half tile[64][72];                 // [k][m], row pitch 144 B keeps 16-byte alignment
    const int k0 = blockIdx.x * 64, m0 = blockIdx.y * 64;
    const int t = threadIdx.x;
    for (int i = t; i < 64 * 8; i += 256) {         // 64 token rows x 8 chunks of 8 k
        const int r = i >> 3, ch = i & 7;
        const int m = m0 + r, k = k0 + ch * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < M && k < K) v = *reinterpret_cast<const uint4 *>(x + (size_t)m * K + k);   // K % 8 == 0
        const __half *h = reinterpret_cast<const __half *>(&v);
#pragma unroll
        for (int j = 0; j < 8; j++) tile[ch * 8 + j][r] = h[j];
    }
    __syncthreads();
    for (int i = t; i < 64 * 8; i += 256) {         // 64 k rows x 8 chunks of 8 tokens
        const int r = i >> 3, ch = i & 7;
        const int k = k0 + r, m = m0 + ch * 8;
        if (k < K && m < Mp) *reinterpret_cast<uint4 *>(xt + (size_t)k * Mp + m) = *reinterpret_cast<const uint4 *>(&tile[r][ch * 8]);
    }
}

int launch_transpose_x(const __half *x, __half *xt, int M, int K, int Mp, cudaStream_t stream)
{
    dim3 tg((unsigned)ceil_div(K, 64), (unsigned)ceil_div(Mp, 64));
    transpose_x_kernel<<<tg, 256, 0, stream>>>(x, xt, M, K, Mp);
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}

struct SpmmParams {
    OrthoView ov;
    const int32_t *rbeg, *rend;    // entry range of work row r: [rbeg[r], rend[r]) (row_ptr / row_ptr + 1, or segments)
    const __half *xt; float *o;    // o already points at the first output slot of this launch
    int nrows, K, Mp;
    int heavy;                     // rows with more entries are processed by the whole CTA, or ...
    int skip_long;                 // ... skipped here because the plan carries them as segments
};

__device__ __forceinline__ void spmm_entry(const SpmmParams &p, int e, int &c, float &v)
{
    if (p.ov.entries) {
        const uint32_t pk = p.ov.entries[e];
        c = (int)(pk & 0xFFFFu);
        v = __half2float(__ushort_as_half((unsigned short)(pk >> 16)));
    } else {
        c = p.ov.col[e];
        v = __half2float(p.ov.val[e]);
        if ((unsigned)c >= (unsigned)p.K) { c = 0; v = 0.f; }     // out-of-range entries are skipped
    }
}

// Entries e_begin, e_begin + e_step, ... < e_end of one row.  A batch of 32 entries is fetched with
// one coalesced load (lane l takes the l-th entry of the batch) and broadcast by shuffles; the 16-byte
// activation loads of 8 consecutive entries are independent, so 8 of them are in flight per lane.
__device__ __forceinline__ void spmm_accumulate(const SpmmParams &p, int e_begin, int e_end, int e_step, int tok0, int lane, float (&acc)[8])
{
    const __half *xbase = p.xt + tok0;
    for (int eb = e_begin; eb < e_end; eb += 32 * e_step) {
        int cl = 0; float vl = 0.f;
        const int e_mine = eb + lane * e_step;
        if (e_mine < e_end) spmm_entry(p, e_mine, cl, vl);
        const int nb = min(32, (e_end - eb + e_step - 1) / e_step);
        for (int j0 = 0; j0 < nb; j0 += 8) {
            uint4 xv[8]; float vv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c = __shfl_sync(0xffffffffu, cl, (j0 + j) & 31);
                vv[j] = __shfl_sync(0xffffffffu, vl, (j0 + j) & 31);      // lanes past the batch hold v = 0, c = 0
                xv[j] = *reinterpret_cast<const uint4 *>(xbase + (size_t)c * p.Mp);
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
}

// CTA = 8 warps x 8 rows each = 64 consecutive output rows, one block of 256 tokens.  A warp first
// fetches the 9 row pointers of its rows with one load, then the first 32 entries of all 8 rows
// (independent loads), and only then walks the rows: per row the dependent chain is a single round
// of activation loads.
template <int RPW>     // rows per warp: 8 for ordinary rows, 1 for the (long) segments
__global__ void __launch_bounds__(kSpRows * 32, 4)
spmm_ortho_kernel(const SpmmParams p)
{
    __shared__ float part[kSpRows][kSpTok];
    __shared__ int heavy_rows[kSpRows * RPW];
    __shared__ int n_heavy;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * (kSpRows * RPW) + warp * RPW;
    const int tok0 = blockIdx.y * kSpTok + lane * 8;
    if (threadIdx.x == 0) n_heavy = 0;
    __syncthreads();
    int rb = 0, re = 0;
    if (lane < RPW && row0 + lane < p.nrows) { rb = p.rbeg[row0 + lane]; re = p.rend[row0 + lane]; }
    int cl[RPW]; float vl[RPW];
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        const int e0 = __shfl_sync(0xffffffffu, rb, r), e1 = __shfl_sync(0xffffffffu, re, r);
        cl[r] = 0; vl[r] = 0.f;
        if (e0 + lane < e1) spmm_entry(p, e0 + lane, cl[r], vl[r]);
    }
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        const int e0 = __shfl_sync(0xffffffffu, rb, r), e1 = __shfl_sync(0xffffffffu, re, r);
        const int cnt = e1 - e0;
        if (cnt > p.heavy) {
            if (!p.skip_long && lane == 0) heavy_rows[atomicAdd(&n_heavy, 1)] = warp * RPW + r;
        } else if (cnt > 0) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const __half *xbase = p.xt + tok0;
            const int nb = min(32, cnt);
            for (int j0 = 0; j0 < nb; j0 += 4) {
                uint4 xv[4]; float vv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int c = __shfl_sync(0xffffffffu, cl[r], (j0 + j) & 31);
                    vv[j] = __shfl_sync(0xffffffffu, vl[r], (j0 + j) & 31);   // slots past the row hold v = 0, c = 0
                    xv[j] = *reinterpret_cast<const uint4 *>(xbase + (size_t)c * p.Mp);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const __half2 *h = reinterpret_cast<const __half2 *>(&xv[j]);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float2 f = __half22float2(h[q]);
                        acc[2 * q] = fmaf(vv[j], f.x, acc[2 * q]);
                        acc[2 * q + 1] = fmaf(vv[j], f.y, acc[2 * q + 1]);
                    }
                }
            }
            if (cnt > 32) spmm_accumulate(p, e0 + 32, e1, 1, tok0, lane, acc);
            float4 *dst = reinterpret_cast<float4 *>(p.o + (size_t)(row0 + r) * p.Mp + tok0);
            dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
    }
    __syncthreads();
    const int nh = n_heavy;
    if (nh == 0) return;
    // long rows: every warp takes every 8th entry of the row, partials meet in shared memory and are
    // added in warp order 0..7 (fixed); rows are visited in index order, not in registration order
    for (int w = 0; w < kSpRows * RPW; w++) {
        bool is_heavy = false;
        for (int i = 0; i < nh; i++) is_heavy |= (heavy_rows[i] == w);
        if (!is_heavy) continue;
        const int hn = blockIdx.x * (kSpRows * RPW) + w;
        const int h0 = p.rbeg[hn], h1 = p.rend[hn];
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        spmm_accumulate(p, h0 + warp, h1, kSpRows, tok0, lane, acc);
#pragma unroll
        for (int q = 0; q < 8; q++) part[warp][lane * 8 + q] = acc[q];
        __syncthreads();
        {
            const int t = threadIdx.x;     // 256 threads <-> 256 tokens
            float s = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < kSpRows; w2++) s += part[w2][t];
            p.o[(size_t)hn * p.Mp + blockIdx.y * kSpTok + t] = s;
        }
        __syncthreads();
    }
}

// O[hrow[h]][m] = sum of the row's segments (output slots nrows_real + v), in segment order
__global__ void combine_segments_kernel(const int32_t *__restrict__ hrow, const int32_t *__restrict__ hptr,
                                        float *__restrict__ o, int nrows_real, int Mp)
{
    const int h = blockIdx.x;
    const int m = blockIdx.y * 256 + threadIdx.x;
    if (m >= Mp) return;
    float s = 0.f;
    const int v0 = hptr[h], v1 = hptr[h + 1];
    const float *src = o + (size_t)nrows_real * Mp + m;
    int v = v0;
    for (; v + 8 <= v1; v += 8) {          // eight loads in flight, added in segment order
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = src[(size_t)(v + i) * Mp];
#pragma unroll
        for (int i = 0; i < 8; i++) s += t[i];
    }
    for (; v < v1; v++) s += src[(size_t)v * Mp];
    o[(size_t)hrow[h] * Mp + m] = s;
}

// workspace layout: [ Xt : K * Mp halves ][ O : N * Mp floats ], Mp = M rounded up to 256; with a plan
// that carries segments of long rows, N counts those extra output slots too
int64_t spmm_workspace_bytes(int64_t M, int64_t K, int64_t N)
{
    const int64_t Mp = ceil_div(M, kSpTok) * kSpTok;
    return ((K * Mp * 2 + 255) / 256) * 256 + N * Mp * 4;
}

int launch_spmm(const FwdArgs &a, const float **o_out, int *mp_out)
{
    const int64_t Mp = ceil_div(a.M, kSpTok) * kSpTok;
    const int64_t nv = (a.plan && a.ortho.entries) ? a.plan->n_virtual : 0;
    if (!a.workspace || a.workspace_bytes < spmm_workspace_bytes(a.M, a.K, a.N + nv)) return ORTHO_B200_ERR_WORKSPACE;
    if (((uintptr_t)a.workspace & 255u) != 0) return ORTHO_B200_ERR_ALIGN;
    __half *xt = reinterpret_cast<__half *>(a.workspace);
    float *o = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(a.workspace) + ((a.K * Mp * 2 + 255) / 256) * 256);
    dim3 tg((unsigned)ceil_div(a.K, 64), (unsigned)(Mp / 64));
    transpose_x_kernel<<<tg, 256, 0, a.stream>>>(a.x, xt, (int)a.M, (int)a.K, (int)Mp);
    count_launch();
    OB_CUDA(cudaGetLastError());
    SpmmParams p;
    p.ov = a.ortho; p.xt = xt; p.K = (int)a.K; p.Mp = (int)Mp;
    p.heavy = (a.plan && a.ortho.entries) ? a.plan->heavy : kNoPlanHeavy;
    // real rows (long ones are skipped when the plan provides their segments)
    p.rbeg = a.ortho.row_ptr; p.rend = a.ortho.row_ptr + 1; p.nrows = (int)a.N; p.o = o; p.skip_long = nv > 0 ? 1 : 0;
    dim3 sg((unsigned)ceil_div(a.N, kSpRows * 8), (unsigned)(Mp / kSpTok));
    spmm_ortho_kernel<8><<<sg, kSpRows * 32, 0, a.stream>>>(p);
    count_launch();
    OB_CUDA(cudaGetLastError());
    if (nv > 0) {
        // segments of the long rows go to output slots N + v, then are summed into the row's own slot
        p.rbeg = a.plan->vbeg; p.rend = a.plan->vend; p.nrows = (int)nv; p.o = o + (size_t)a.N * Mp; p.skip_long = 0;
        dim3 vg((unsigned)ceil_div(nv, kSpRows), (unsigned)(Mp / kSpTok));
        spmm_ortho_kernel<1><<<vg, kSpRows * 32, 0, a.stream>>>(p);
        count_launch();
        OB_CUDA(cudaGetLastError());
        dim3 cg((unsigned)a.plan->n_long, (unsigned)(Mp / 256));
        combine_segments_kernel<<<cg, 256, 0, a.stream>>>(a.plan->hrow, a.plan->hptr, o, (int)a.N, (int)Mp);
        count_launch();
        OB_CUDA(cudaGetLastError());
    }
    *o_out = o;
    *mp_out = (int)Mp;
    return ORTHO_B200_OK;
}

}  // namespace ob
