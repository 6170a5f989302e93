// Prefill-regime (large M) OrthoLinear forward for sm_100a on the 5th-generation tensor cores.
//
// Replaces the reference's WMMA kernels (src/dual_gemm_tensor_core.cu:70-174, 215-337), which
// quantise activations to int8 and scan the whole coordinate list per output element.  Here the
// base term is a real FP16 contraction with FP32 accumulation in tensor memory:
//
//     D[n, m] = sum_k  w_int[n, k] * x[m, k]          (tcgen05.mma, kind::f16)
//     y[m, n] = scale[n] * D[n, m]  (+ alpha * ortho[m, n])
//
// The weight tile is the M operand of the MMA and lives in TENSOR MEMORY: TMA brings the packed
// INT4 bytes of 128 output rows x 64 k into shared memory, four converter warps (one thread per
// output row) unpack them in registers to exact small-integer halves and write them with
// tcgen05.st, so the converted weights never touch shared memory.  The token tile (128 tokens x
// 64 k, FP16, 128-byte swizzle) is the N operand and goes from global to shared memory by TMA and
// from there straight into the MMA.  One elected thread issues the MMAs; accumulators are double
// buffered in TMEM (2 x 128 columns) so that the epilogue of a tile runs while the next tile is
// being accumulated.  The per-row scale is applied in the FP32 epilogue (it factors out of the K
// sum, src/ortho.c:356,363), outputs are transposed through shared memory and stored coalesced.
//
// Warp roles (CTA = 1 SM, persistent over tiles):
//   warp 0      TMA producer          warp 1      MMA issuer, TMEM allocator
//   warps 2-5   INT4 -> FP16 -> TMEM  warps 6-9   epilogue (TMEM -> scale -> FP16 -> global)
#include "common.cuh"
#include "umma.cuh"

namespace ob {

int launch_decode(const FwdArgs &a);
int *kernel_status_word();

namespace pf {
constexpr int TN = 128;            // output rows per tile   (MMA M)
constexpr int TM = 128;            // tokens per tile        (MMA N)
constexpr int KB = 64;             // k per pipeline stage
constexpr int STAGES = 6;
constexpr int ASTAGES = 4;
constexpr int X_BYTES = TM * KB * 2;     // 16 KB
constexpr int W_BYTES = TN * KB / 2;     // 4 KB
constexpr int YS_PITCH = TN + 8;         // halves per staged token row (pad against bank conflicts)
constexpr int NWARPS = 10;
constexpr int TMEM_COLS = 512;
constexpr int A_COL0 = 2 * TM;           // accumulators occupy [0, 2*TM), converted weights follow

struct Params {
    const __half *scales; __half *y;
    int M, K, N;
    int tiles_n, tiles_m, kblocks;
    int *status;
};

struct Smem {
    uint64_t x_full[STAGES], x_empty[STAGES];
    uint64_t a_full[ASTAGES], a_empty[ASTAGES];
    uint64_t d_full[2], d_empty[2];
    uint32_t tmem_base;
};

constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * (X_BYTES + W_BYTES) + 32 * YS_PITCH * 2 + sizeof(Smem) + 256;
}  // namespace pf

__global__ void __launch_bounds__(pf::NWARPS * 32, 1)
prefill_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const pf::Params p)
{
    using namespace pf;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *xs = base;                                       // STAGES x 16 KB, 1 KB aligned
    unsigned char *ws = xs + (size_t)STAGES * X_BYTES;              // STAGES x 4 KB
    __half *ys = reinterpret_cast<__half *>(ws + (size_t)STAGES * W_BYTES);
    Smem *sm = reinterpret_cast<Smem *>(reinterpret_cast<unsigned char *>(ys) + 32 * YS_PITCH * 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = p.tiles_n * p.tiles_m;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&sm->x_full[s], 1); mbar_init(&sm->x_empty[s], 1 + 4); }
        for (int s = 0; s < ASTAGES; s++) { mbar_init(&sm->a_full[s], 4); mbar_init(&sm->a_empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&sm->d_full[b], 1); mbar_init(&sm->d_empty[b], 4); }
        fence_mbar_init();
        prefetch_tensormap(&xmap);
        prefetch_tensormap(&wmap);
    }
    if (warp == 1) { tmem_alloc(&sm->tmem_base, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm->tmem_base;
    bool dead = false;
    auto wait = [&](uint64_t *bar, uint32_t parity) {
        if (dead) return;
        if (!mbar_wait(bar, parity, 1u << 24)) { dead = true; atomicExch(p.status, 1); }
    };

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
                const int nt = t % p.tiles_n, mt = t / p.tiles_n;
                for (int kb = 0; kb < p.kblocks; kb++) {
                    wait(&sm->x_empty[s], ph ^ 1u);
                    mbar_arrive_expect_tx(&sm->x_full[s], X_BYTES + W_BYTES);
                    tma_load_2d(xs + (size_t)s * X_BYTES, &xmap, &sm->x_full[s], kb * KB, mt * TM);
                    tma_load_2d(ws + (size_t)s * W_BYTES, &wmap, &sm->x_full[s], kb * (KB / 2), nt * TN);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(TN, TM);
            int s = 0, as = 0; uint32_t ph = 0, aph = 0;
            int it = 0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x, it++) {
                const int b = it & 1;
                wait(&sm->d_empty[b], (uint32_t)(((it >> 1) & 1) ^ 1));
                tc_fence_after();
                const uint32_t d_tmem = tmem + (uint32_t)(b * TM);
                for (int kb = 0; kb < p.kblocks; kb++) {
                    wait(&sm->x_full[s], ph);
                    wait(&sm->a_full[as], aph);
                    tc_fence_after();
                    const uint32_t a_tmem = tmem + (uint32_t)(A_COL0 + as * (KB / 2));
                    const uint32_t xaddr = smem_u32(xs + (size_t)s * X_BYTES);
#pragma unroll
                    for (int kk = 0; kk < KB / 16; kk++)
                        umma_f16_ts(d_tmem, a_tmem + (uint32_t)(kk * 8), umma_desc_sw128(xaddr + (uint32_t)(kk * 32)), idesc,
                                    (uint32_t)((kb | kk) != 0));
                    umma_commit(&sm->x_empty[s]);
                    umma_commit(&sm->a_empty[as]);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                    if (++as == ASTAGES) { as = 0; aph ^= 1u; }
                }
                umma_commit(&sm->d_full[b]);
            }
        }
    } else if (warp < 6) {
        // ================= converters: packed INT4 (smem) -> FP16 (TMEM, A operand) =================
        const int q = warp & 3;                        // TMEM lane quarter this warp may touch
        const int row = q * 32 + lane;                 // output row inside the tile == TMEM lane
        int s = 0, as = 0; uint32_t ph = 0, aph = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
            for (int kb = 0; kb < p.kblocks; kb++) {
                wait(&sm->x_full[s], ph);
                const uint4 *wrow = reinterpret_cast<const uint4 *>(ws + (size_t)s * W_BYTES + row * (KB / 2));
                const uint4 w0 = wrow[0], w1 = wrow[1];
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->x_empty[s]);
                uint32_t h[32];
                const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint32_t o[4];
                    int4x8_to_half2x4_natural(ww[j], o);
                    h[4 * j] = o[0]; h[4 * j + 1] = o[1]; h[4 * j + 2] = o[2]; h[4 * j + 3] = o[3];
                }
                wait(&sm->a_empty[as], aph ^ 1u);
                tc_fence_after();
                tmem_st_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(A_COL0 + as * (KB / 2)), h);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->a_full[as]);
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                if (++as == ASTAGES) { as = 0; aph ^= 1u; }
            }
        }
    } else {
        // ================= epilogue: TMEM -> scale -> FP16 -> shared (transpose) -> global =================
        const int q = warp & 3;
        const int et = (warp - 6) * 32 + lane;         // 0..127 among the epilogue threads
        const bool vec_ok = (p.N % 8) == 0;
        int it = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, it++) {
            const int nt = t % p.tiles_n, mt = t / p.tiles_n;
            const int b = it & 1;
            const int n = nt * TN + q * 32 + lane;
            const float sc = (n < p.N) ? __half2float(p.scales[n]) : 0.f;
            wait(&sm->d_full[b], (uint32_t)((it >> 1) & 1));
            tc_fence_after();
            for (int c = 0; c < TM / 32; c++) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TM + c * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) ys[j * YS_PITCH + q * 32 + lane] = __float2half_rn(__uint_as_float(r[j]) * sc);
                named_bar_sync(1, 128);
#pragma unroll
                for (int i2 = 0; i2 < 4; i2++) {
                    const int id = i2 * 128 + et, tok = id >> 4, part = id & 15;
                    const int m = mt * TM + c * 32 + tok, n0 = nt * TN + part * 8;
                    if (m < p.M && n0 < p.N) {
                        const __half *src = ys + tok * YS_PITCH + part * 8;
                        __half *dst = p.y + (size_t)m * p.N + n0;
                        if (vec_ok) {
                            *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
                        } else {
                            for (int e = 0; e < 8 && n0 + e < p.N; e++) dst[e] = src[e];
                        }
                    }
                }
                named_bar_sync(1, 128);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->d_empty[b]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

int64_t prefill_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }

static int launch_prefill_base(const FwdArgs &a)
{
    using namespace pf;
    CUtensorMap xmap, wmap;
    if (!make_tensor_map_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                            (uint64_t)a.K * 2, TM, KB, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    if (!make_tensor_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)a.N, (uint64_t)(a.K / 2),
                            (uint64_t)(a.K / 2), TN, KB / 2, CU_TENSOR_MAP_SWIZZLE_NONE))
        return ORTHO_B200_ERR_CUDA;
    Params p;
    p.scales = a.scales; p.y = a.y; p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N;
    p.tiles_n = (int)ceil_div(a.N, TN); p.tiles_m = (int)ceil_div(a.M, TM); p.kblocks = (int)ceil_div(a.K, KB);
    p.status = kernel_status_word();
    if (!p.status) return ORTHO_B200_ERR_CUDA;
    static bool attr_set = false;
    static int num_sms = 148;
    if (!attr_set) {
        OB_CUDA(cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        int dev = 0;
        OB_CUDA(cudaGetDevice(&dev));
        OB_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
        attr_set = true;
    }
    const int ntiles = p.tiles_n * p.tiles_m;
    const int grid = ntiles < num_sms ? ntiles : num_sms;
    prefill_kernel<<<grid, NWARPS * 32, kSmemBytes, a.stream>>>(xmap, wmap, p);
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}

int launch_prefill(const FwdArgs &a)
{
    if (!a.has_ortho) return launch_prefill_base(a);
    // sparse term not yet fused on the tensor-core path: token chunks through the streaming kernel
    for (int64_t m0 = 0; m0 < a.M; m0 += ORTHO_B200_DECODE_MAX_M) {
        FwdArgs b = a;
        b.M = (a.M - m0 < ORTHO_B200_DECODE_MAX_M) ? (a.M - m0) : ORTHO_B200_DECODE_MAX_M;
        b.x = a.x + m0 * a.K;
        b.y = a.y + m0 * a.N;
        int st = launch_decode(b);
        if (st != ORTHO_B200_OK) return st;
    }
    return ORTHO_B200_OK;
}

}  // namespace ob
