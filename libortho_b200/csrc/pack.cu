// Device-side producer of the layout the forward consumes: INT4 quantise + nibble-pack of the base and
// CSR build of the ortho residual.  Follows OrthoLinear.load_from_weights
// (torch_bind/ortho_linear.py:79-128) and pack_ortho_sparse(..., "csr") (tools/sieve.py:119-152) of the
// reference operation by operation, so the results are bit-identical to that torch chain:
//   scale   = max(rowmax|W| / 7, 1e-6)                 (IEEE FP32 division; stored as FP16, round to nearest)
//   w_int   = clamp(round_half_even(W / scale_fp32), -8, 7)
//   byte    = (w_int[2i] & 15) | (w_int[2i+1] & 15) << 4       (even flat index in the low nibble)
//   CSR     = positions with W_ortho != 0 in row-major order, int32 indices, values rounded to FP16
// All of it is HBM-bound element-wise work: one pass over W (the second read of a row hits L2).
#include "common.cuh"

namespace ob {

// the library is built with fast-math; the packer needs the IEEE operations spelled out
__device__ __forceinline__ float div_rn_ieee(float a, float b) {
    float r;
    asm("div.rn.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
// W != 0 exactly as IEEE compares it (no flush of subnormals; NaN counts as non-zero)
__device__ __forceinline__ bool is_nonzero(float v) { return (__float_as_uint(v) << 1) != 0u; }
__device__ __forceinline__ int quantise_one(float w, float scale) {
    float q;
    asm("cvt.rni.f32.f32 %0, %1;" : "=f"(q) : "f"(div_rn_ieee(w, scale)));   // round half to even
    q = fminf(fmaxf(q, -8.f), 7.f);             // NaN -> -8 here; torch leaves NaN undefined after the int8 cast
    return (int)q;
}

// one CTA per output row
__global__ void __launch_bounds__(256)
pack_base_kernel(const float *__restrict__ w, const float *__restrict__ scales_in, int64_t N, int K,
                 uint32_t *__restrict__ packed, __half *__restrict__ scales_out)
{
    __shared__ float wmax[8];
    __shared__ float s_scale;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int64_t n = blockIdx.x; n < N; n += gridDim.x) {
        const float4 *row = reinterpret_cast<const float4 *>(w + (size_t)n * K);
        float scale;
        if (scales_in) {
            scale = scales_in[n];
        } else {
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
                s_scale = fmaxf(div_rn_ieee(mm, 7.0f), 1e-6f);
            }
            __syncthreads();
            scale = s_scale;
        }
        if (tid == 0) scales_out[n] = __float2half_rn(scale);
        uint32_t *out = packed + (size_t)n * (K / 8);
        for (int i = tid; i < K / 8; i += 256) {          // 8 weights -> one 32-bit word
            const float4 a = row[2 * i], b = row[2 * i + 1];
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            uint32_t word = 0;
#pragma unroll
            for (int e = 0; e < 8; e++) word |= ((uint32_t)quantise_one(v[e], scale) & 0xFu) << (4 * e);
            out[i] = word;
        }
        __syncthreads();      // wmax / s_scale are reused by the next row
    }
}

// nnz per row (one warp per row), then an exclusive scan by one CTA
__global__ void __launch_bounds__(256)
csr_count_kernel(const float *__restrict__ w, int64_t N, int K, int32_t *__restrict__ row_ptr)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t n = (int64_t)blockIdx.x * 8 + warp; n < N; n += (int64_t)gridDim.x * 8) {
        const float *row = w + (size_t)n * K;
        int c = 0;
        for (int k = lane; k < K; k += 32) c += is_nonzero(row[k]) ? 1 : 0;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) row_ptr[n + 1] = c;
    }
}

__global__ void __launch_bounds__(1024)
csr_scan_kernel(int64_t N, int32_t *__restrict__ row_ptr, int *__restrict__ overflow)
{
    __shared__ int warp_sum[32];
    __shared__ long long carry;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { carry = 0; row_ptr[0] = 0; }
    __syncthreads();
    for (int64_t base = 0; base < N; base += 1024) {
        const int64_t i = base + tid;
        int v = (i < N) ? row_ptr[i + 1] : 0, s = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, s, o); if (lane >= o) s += t; }
        if (lane == 31) warp_sum[warp] = s;
        __syncthreads();
        if (warp == 0) {
            int ws = warp_sum[lane], t2 = ws;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, t2, o); if (lane >= o) t2 += t; }
            warp_sum[lane] = t2 - ws;              // exclusive prefix of the warp totals
        }
        __syncthreads();
        const long long incl = carry + warp_sum[warp] + s;
        if (i < N) {
            if (incl > 0x7fffffffLL) atomicExch(overflow, 1);
            row_ptr[i + 1] = (int32_t)incl;
        }
        __syncthreads();
        if (tid == 1023) carry = incl;
        __syncthreads();
    }
}

// one warp per row: ballot compaction keeps the column order
__global__ void __launch_bounds__(256)
csr_fill_kernel(const float *__restrict__ w, int64_t N, int K, const int32_t *__restrict__ row_ptr,
                int32_t *__restrict__ col, __half *__restrict__ val)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t n = (int64_t)blockIdx.x * 8 + warp; n < N; n += (int64_t)gridDim.x * 8) {
        const float *row = w + (size_t)n * K;
        int at = row_ptr[n];
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int k = k0 + lane;
            const float v = (k < K) ? row[k] : 0.0f;
            const unsigned m = __ballot_sync(0xffffffffu, is_nonzero(v));
            if (is_nonzero(v)) {
                const int pos = at + __popc(m & ((1u << lane) - 1u));
                col[pos] = k;
                val[pos] = __float2half_rn(v);
            }
            at += __popc(m);
        }
    }
}

int *kernel_status_word();   // api.cu

}  // namespace ob

using namespace ob;

static int check_pack_args(const void *w, int64_t N, int64_t K)
{
    if (!w) return ORTHO_B200_ERR_NULL;
    if (N <= 0 || K <= 0 || (K % 8) != 0 || K > 0x7fffffffLL || N > 0x7fffff00LL) return ORTHO_B200_ERR_SHAPE;
    if (((uintptr_t)w & 15u) != 0) return ORTHO_B200_ERR_ALIGN;
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_pack_base(const float *w, int64_t N, int64_t K, const float *scales_in,
                                    void *q_weight_out, void *q_scales_f16_out, void *stream)
{
    int st = check_pack_args(w, N, K);
    if (st != ORTHO_B200_OK) return st;
    if (!q_weight_out || !q_scales_f16_out) return ORTHO_B200_ERR_NULL;
    if (((uintptr_t)q_weight_out & 3u) != 0 || ((uintptr_t)q_scales_f16_out & 1u) != 0) return ORTHO_B200_ERR_ALIGN;
    const unsigned grid = (unsigned)(N < 148 * 8 ? N : 148 * 8);
    pack_base_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w, scales_in, N, (int)K, (uint32_t *)q_weight_out,
                                                             (__half *)q_scales_f16_out);
    OB_CUDA(cudaGetLastError());
    count_launch();
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_csr_count(const float *w_ortho, int64_t N, int64_t K, int32_t *row_ptr_out, void *stream)
{
    int st = check_pack_args(w_ortho, N, K);
    if (st != ORTHO_B200_OK) return st;
    if (!row_ptr_out) return ORTHO_B200_ERR_NULL;
    int *status = ob::kernel_status_word();
    if (!status) return ORTHO_B200_ERR_CUDA;
    const int64_t blocks = ceil_div(N, 8);
    csr_count_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(w_ortho, N, (int)K, row_ptr_out);
    OB_CUDA(cudaGetLastError());
    csr_scan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(N, row_ptr_out, status);
    OB_CUDA(cudaGetLastError());
    count_launch(2);
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_csr_fill(const float *w_ortho, int64_t N, int64_t K, const int32_t *row_ptr,
                                   int32_t *col_out, void *val_f16_out, void *stream)
{
    int st = check_pack_args(w_ortho, N, K);
    if (st != ORTHO_B200_OK) return st;
    if (!row_ptr) return ORTHO_B200_ERR_NULL;
    const int64_t blocks = ceil_div(N, 8);
    csr_fill_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, (cudaStream_t)stream>>>(
        w_ortho, N, (int)K, row_ptr, col_out, (__half *)val_f16_out);
    OB_CUDA(cudaGetLastError());
    count_launch();
    return ORTHO_B200_OK;
}
