// Device-side Hessian sieve: the split of a full-precision weight matrix into the INT4-representable base
// and the sparse residual that the packer (pack.cu) then turns into the operator's buffers.
//
// Follows hessian_sieve / quantize_int4 of the reference (tools/sieve.py:13-23, 25-76) operation by
// operation in IEEE FP32, so that the two outputs are bit-identical to that torch chain:
//   scale[n]  = max(rowmax|W|, 1e-8) / 7
//   base      = clamp(round_half_even(W / scale), -8, 7) * scale        (non-finite -> 0)
//   residual  = W - base
//   score     = residual^2 / (diag(H_inv) + 1e-6)
//   ortho     = residual * (score > threshold)
// The threshold is a given constant (curvature threshold) or the k-th largest score ("keep the top
// fraction", tools/sieve.py:61-66); the k-th largest is found with a four-pass byte-wise radix select over
// the scores' bit patterns, recomputing the scores from W in every pass instead of storing them.
// Everything is element-wise, HBM-bound work: W is read once per pass with 16-byte loads.
#include "common.cuh"

namespace ob {

__device__ __forceinline__ float sv_div(float a, float b) { float r; asm("div.rn.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ float sv_rint(float a) { float r; asm("cvt.rni.f32.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }
__device__ __forceinline__ bool sv_finite(float v) { return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u; }

// base value and residual of one weight; returns the score
__device__ __forceinline__ float sieve_one(float w, float scale, float hs, float &base, float &res)
{
    float q = sv_rint(sv_div(w, scale));
    const bool q_nan = (q != q);
    q = fminf(fmaxf(q, -8.f), 7.f);
    base = __fmul_rn(q, scale);
    if (q_nan || !sv_finite(base)) base = 0.f;
    res = __fsub_rn(w, base);
    return sv_div(__fmul_rn(res, res), hs);
}
// order-preserving map of a float to an unsigned key (larger float <-> larger key)
__device__ __forceinline__ uint32_t score_key(float s)
{
    const uint32_t b = __float_as_uint(s);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_score(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// one CTA per row: scale[n] = max(rowmax|W|, 1e-8) / 7
__global__ void __launch_bounds__(256)
sieve_row_scale_kernel(const float *__restrict__ w, int64_t N, int K, float *__restrict__ scales)
{
    __shared__ float wmax[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int64_t n = blockIdx.x; n < N; n += gridDim.x) {
        const float4 *row = reinterpret_cast<const float4 *>(w + (size_t)n * K);
        float m = 0.f;
        for (int i = tid; i < K / 4; i += 256) {
            const float4 v = row[i];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) wmax[warp] = m;
        __syncthreads();
        if (tid == 0) {
            float mm = wmax[0];
            for (int i = 1; i < 8; i++) mm = fmaxf(mm, wmax[i]);
            scales[n] = sv_div(fmaxf(mm, 1e-8f), 7.0f);
        }
        __syncthreads();
    }
}

// radix-select state in device memory: hist[256], prefix, remaining rank, result
struct SelectState { unsigned int hist[256]; unsigned int prefix; unsigned long long krem; float threshold; };

// pass p (0 = most significant byte): histogram of byte p of the keys whose higher bytes equal the prefix
__global__ void __launch_bounds__(256)
sieve_hist_kernel(const float *__restrict__ w, const float *__restrict__ hinv, const float *__restrict__ scales,
                  int64_t N, int K, int pass, SelectState *__restrict__ st)
{
    __shared__ unsigned int h[256];
    h[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t prefix = st->prefix;
    const int shift = 24 - 8 * pass;
    const int64_t quads = N * (int64_t)(K / 4);
    const int kq = K / 4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < quads; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / kq;
        const int c = (int)(i - n * kq) * 4;
        const float4 v = reinterpret_cast<const float4 *>(w)[i];
        const float4 hv = *reinterpret_cast<const float4 *>(hinv + c);
        const float sc = scales[n];
        const float ww[4] = {v.x, v.y, v.z, v.w}, hh[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float b, r;
            const uint32_t key = score_key(sieve_one(ww[e], sc, __fadd_rn(hh[e], 1e-6f), b, r));
            if (pass == 0 || (key >> (shift + 8)) == prefix) atomicAdd(&h[(key >> shift) & 255u], 1u);
        }
    }
    __syncthreads();
    if (h[threadIdx.x]) atomicAdd(&st->hist[threadIdx.x], h[threadIdx.x]);
}

// one CTA: the bin that holds the krem-th largest key of this pass; clears the histogram for the next pass
__global__ void __launch_bounds__(256)
sieve_select_kernel(SelectState *__restrict__ st, int pass)
{
    __shared__ unsigned long long above[257];
    const int t = threadIdx.x;
    if (t == 0) {
        unsigned long long run = 0;
        above[256] = 0;
        for (int b = 255; b >= 0; b--) { above[b] = run; run += st->hist[b]; }     // keys in bins > b
    }
    __syncthreads();
    const unsigned long long k = st->krem;
    const unsigned long long cnt = st->hist[t];
    const bool mine = above[t] < k && k <= above[t] + cnt;
    __syncthreads();
    st->hist[t] = 0;
    if (mine) {
        st->prefix = (st->prefix << 8) | (unsigned)t;
        st->krem = k - above[t];
        if (pass == 3) st->threshold = key_score((st->prefix));
    }
}

__global__ void __launch_bounds__(256)
sieve_split_kernel(const float *__restrict__ w, const float *__restrict__ hinv, const float *__restrict__ scales,
                   int64_t N, int K, const float *__restrict__ thr_dev, float thr_host,
                   float *__restrict__ w_base, float *__restrict__ w_ortho)
{
    const float thr = thr_dev ? *thr_dev : thr_host;
    const int64_t quads = N * (int64_t)(K / 4);
    const int kq = K / 4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < quads; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / kq;
        const int c = (int)(i - n * kq) * 4;
        const float4 v = reinterpret_cast<const float4 *>(w)[i];
        const float4 hv = *reinterpret_cast<const float4 *>(hinv + c);
        const float sc = scales[n];
        const float ww[4] = {v.x, v.y, v.z, v.w}, hh[4] = {hv.x, hv.y, hv.z, hv.w};
        float bo[4], oo[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float r;
            const float s = sieve_one(ww[e], sc, __fadd_rn(hh[e], 1e-6f), bo[e], r);
            oo[e] = __fmul_rn(r, (s > thr) ? 1.f : 0.f);        // residual * mask, signed zeros as torch produces them
        }
        reinterpret_cast<float4 *>(w_base)[i] = make_float4(bo[0], bo[1], bo[2], bo[3]);
        reinterpret_cast<float4 *>(w_ortho)[i] = make_float4(oo[0], oo[1], oo[2], oo[3]);
    }
}

static unsigned sieve_grid(int64_t quads)
{
    int64_t blocks = ceil_div(quads, 256 * 4);
    const int64_t cap = (int64_t)device_sm_count(current_device_index()) * 8;
    return (unsigned)(blocks < 1 ? 1 : blocks > cap ? cap : blocks);
}

}  // namespace ob

using namespace ob;

extern "C" int64_t ortho_b200_sieve_scratch_bytes(int64_t N) { return N > 0 ? ((N * 4 + 255) / 256) * 256 + (int64_t)sizeof(SelectState) + 256 : -1; }

extern "C" int ortho_b200_sieve(const float *w, const float *h_inv_diag, int64_t N, int64_t K,
                                float curvature_thresh, int64_t keep_top_k,
                                float *w_base_out, float *w_ortho_out,
                                void *scratch, int64_t scratch_bytes, void *stream)
{
    if (!w || !h_inv_diag || !w_base_out || !w_ortho_out || !scratch) return ORTHO_B200_ERR_NULL;
    if (N <= 0 || K <= 0 || (K % 4) != 0 || keep_top_k < -1 || keep_top_k > N * K) return ORTHO_B200_ERR_SHAPE;
    if ((((uintptr_t)w | (uintptr_t)h_inv_diag | (uintptr_t)w_base_out | (uintptr_t)w_ortho_out) & 15u) != 0 ||
        ((uintptr_t)scratch & 255u) != 0)
        return ORTHO_B200_ERR_ALIGN;
    if (scratch_bytes < ortho_b200_sieve_scratch_bytes(N)) return ORTHO_B200_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    float *scales = reinterpret_cast<float *>(scratch);
    SelectState *sel = reinterpret_cast<SelectState *>(reinterpret_cast<unsigned char *>(scratch) + ((N * 4 + 255) / 256) * 256);
    const int64_t quads = N * (K / 4);
    sieve_row_scale_kernel<<<(unsigned)(N < 148 * 8 ? N : 148 * 8), 256, 0, st>>>(w, N, (int)K, scales);
    count_launch();
    OB_CUDA(cudaGetLastError());
    const float *thr_dev = nullptr;
    float thr_host = curvature_thresh;
    if (keep_top_k > 0) {
        // threshold = k-th largest score: four histogram passes over the key bytes
        SelectState init;
        memset(&init, 0, sizeof(init));
        init.krem = (unsigned long long)keep_top_k;
        OB_CUDA(cudaMemcpyAsync(sel, &init, sizeof(init), cudaMemcpyHostToDevice, st));
        for (int pass = 0; pass < 4; pass++) {
            sieve_hist_kernel<<<sieve_grid(quads), 256, 0, st>>>(w, h_inv_diag, scales, N, (int)K, pass, sel);
            sieve_select_kernel<<<1, 256, 0, st>>>(sel, pass);
            count_launch(2);
            OB_CUDA(cudaGetLastError());
        }
        thr_dev = &sel->threshold;
    } else if (keep_top_k == 0) {
        thr_host = __builtin_inff();          // "keep nothing" (tools/sieve.py:65-66)
    }
    sieve_split_kernel<<<sieve_grid(quads), 256, 0, st>>>(w, h_inv_diag, scales, N, (int)K, thr_dev, thr_host, w_base_out, w_ortho_out);
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}
