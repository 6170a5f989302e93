// Activations transposed once per forward for the sparse term of the tensor-core regimes:
//
//     Xt[k][m] = X[m][k]        (FP16, row pitch Mp >= M, zero for m >= M)
//
// so that one sparse entry (a column k) touches a contiguous run of tokens.  The reference adds the sparse term
// one coordinate at a time per token (src/ortho.c:384-398) or, on the GPU, scans the coordinate list per output
// element (src/dual_gemm_tensor_core.cu:180-207); here the gather along tokens is one or a few 16-byte loads
// per entry (prefill.cu, mid.cu).
#include "common.cuh"

namespace ob {

// X[M][K] (FP16) -> Xt[K][Mp] (FP16), zero padded for m >= M.  64 x 64 tiles; 16-byte global loads
// along k, 16-byte global stores along m, transposition through a shared tile whose row pitch of 33 words keeps
// both the scattered 2-byte writes (8 different k per quarter-warp) and the row reads free of bank conflicts.
__global__ void __launch_bounds__(256)
transpose_x_kernel(const __half *__restrict__ x, __half *__restrict__ xt, int M, int K, int Mp)
{
    __shared__ __half tile[64][66];                 // [k][m]
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
        if (k < K && m < Mp) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(&tile[r][ch * 8]);
            *reinterpret_cast<uint4 *>(xt + (size_t)k * Mp + m) = make_uint4(src[0], src[1], src[2], src[3]);
        }
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

}  // namespace ob
