// Standalone microbenchmark (not linked into the library): cycles per tcgen05.mma.cta_group::1.kind::f16 (K = 16)
// as a function of M (128 / 64) and N (16 .. 256), with the A operand in tensor memory (.ts) or in shared memory
// (.ss), on one CTA and on one CTA per SM.  One thread issues 4096 MMAs back to back on constant operands
// (FP16 ones), commits to an mbarrier and waits (bounded); clock64() brackets issue + completion.  The tile
// shapes of mid.cu and prefill.cu were chosen from its output.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue_probe mma_issue_probe.cu && ./mma_issue_probe
#include <cstdio>
#include <cuda_runtime.h>
#include "umma.cuh"
using namespace ob;

struct Res { long long cyc; int ok; };

__global__ void __launch_bounds__(128, 1) probe(int Mrows, int N, int ss, int nmma, int nacc, Res *out)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t bar;
    __shared__ uint32_t tbase;
    // fill 48 KB of smem with 1.0 halves
    for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(base)[i] = 0x3C003C00u;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
    if (threadIdx.x < 32) { tmem_alloc(&tbase, 512); tmem_relinquish(); }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tbase;
    // A region in TMEM: columns [384, 512): 1.0 halves
    {
        uint32_t r[32];
        for (int i = 0; i < 32; i++) r[i] = 0x3C003C00u;
        const int q = threadIdx.x >> 5;
        for (int c = 384; c < 512; c += 32) tmem_st_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + c, r);
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    long long t0 = 0, t1 = 0;
    int ok = 1;
    if (threadIdx.x == 0) {
        const uint32_t idesc = umma_idesc_f16(Mrows, N);
        const uint64_t adesc = umma_desc_sw128(smem_u32(base));              // 16 KB A tile
        const uint64_t bdesc = umma_desc_sw128(smem_u32(base + 16 * 1024));  // up to 32 KB B tile
        t0 = clock64();
        for (int i = 0; i < nmma; i++) {
            const uint32_t d = tmem + (uint32_t)((i % nacc) * N);
            const int kk = i & 3;
            if (ss) umma_f16_ss(d, adesc + (uint64_t)(2 * kk), bdesc + (uint64_t)(2 * kk), idesc, i >= nacc);
            else umma_f16_ts(d, tmem + 384 + kk * 8, bdesc + (uint64_t)(2 * kk), idesc, i >= nacc);
        }
        umma_commit(&bar);
        ok = mbar_wait(&bar, 0, 1u << 22) ? 1 : 0;
        t1 = clock64();
        out[blockIdx.x].cyc = t1 - t0;
        out[blockIdx.x].ok = ok;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

int main()
{
    Res *d; cudaMalloc(&d, sizeof(Res) * 148);
    cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    const int nmma = 4096;
    for (int grid : {1, 148})
        for (int Mrows : {128, 64})
            for (int ss : {0, 1})
                for (int N : {16, 32, 64, 128, 256}) {
                    for (int nacc : {1, 2}) {
                        if (nacc * N > 384) continue;
                        probe<<<grid, 128, 64 * 1024>>>(Mrows, N, ss, nmma, nacc, d);
                        cudaError_t e = cudaDeviceSynchronize();
                        Res h[148];
                        cudaMemcpy(h, d, sizeof(Res) * grid, cudaMemcpyDeviceToHost);
                        long long mx = 0; int ok = 1;
                        for (int i = 0; i < grid; i++) { if (h[i].cyc > mx) mx = h[i].cyc; ok &= h[i].ok; }
                        printf("grid=%3d M=%3d N=%3d %s nacc=%d : %.1f cycles/MMA  (ok=%d err=%d)\n", grid, Mrows, N, ss ? "ss" : "ts", nacc,
                               (double)mx / nmma, ok, (int)e);
                        if (e != cudaSuccess) return 1;
                    }
                }
    return 0;
}
