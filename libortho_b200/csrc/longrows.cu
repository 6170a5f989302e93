// Sparse sums of the plan's long rows for the prefill regime, computed ahead of the main tensor-core kernel:
//
//     OL[h][m] = sum over the entries i of long row hrow[h] of v_i * x[m, c_i]            (FP32)
//
// A layer whose entries pile up in a few rows (power-law row loads) has rows with hundreds to thousands of entries;
// inside the main kernel one warp walks a row with one 16-byte gather per entry and lane, so such a row would hold
// up its whole tile, and as gathers the long rows alone move nnz_long x M x 2 bytes through L2.  A row that long is
// better treated as what it nearly is, a dense row: the plan keeps the long rows as a zero-filled FP16 matrix
// HD[n_long (padded to 128)][K], and their sums are a small GEMM on the 5th-generation tensor cores,
//
//     OL = HD * X^T        (tcgen05.mma kind::f16, both operands K-major from shared memory via TMA, FP32 in TMEM)
//
// tile = 128 long rows x 256 tokens, K cut into `nsplit` shares so that the few tiles fill the GPU; every share
// leaves its FP32 sums in the workspace and the main kernel adds the shares, in share order, when it picks a long
// row's sums up (no atomics: the result does not depend on scheduling).  X is read in its own layout, the
// transposed copy is not needed here.  The main kernel is launched as a programmatic dependent of this one: its
// tensor-core pipeline starts while this kernel drains, only the warps that read the sums wait for it.
// The reference walks every coordinate serially per token (src/ortho.c:384-398).
#include <cstring>

#include "common.cuh"
#include "umma.cuh"

namespace ob {

int *kernel_status_word();

namespace lg {
constexpr int TR = 128;                 // long rows per tile (MMA M)
constexpr int TT = 256;                 // tokens per tile (MMA N)
constexpr int KB = 64;                  // k per stage: 128-byte rows, 128-byte swizzle
constexpr int ST = 4;
constexpr int A_BYTES = TR * KB * 2;    // 16 KB
constexpr int B_BYTES = TT * KB * 2;    // 32 KB
constexpr int NWARPS = 6;               // TMA, MMA, four epilogue warps
struct Smem {
    uint64_t full[ST], empty[ST], d_full;
    uint32_t tmem_base;
};
constexpr size_t kSmemBytes = 1024 + (size_t)ST * (A_BYTES + B_BYTES) + sizeof(Smem) + 64;
struct Params {
    float *part;                        // [nsplit][n_pad][Mp]
    int n_long, n_pad, Mp, kblocks, nsplit;
    int *status;
};
}  // namespace lg

__global__ void __launch_bounds__(lg::NWARPS * 32, 1)
long_gemm_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap xmap, const lg::Params p)
{
    using namespace lg;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *as = base, *bs = base + (size_t)ST * A_BYTES;
    Smem *sm = reinterpret_cast<Smem *>(base + (size_t)ST * (A_BYTES + B_BYTES));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.x, tok0 = blockIdx.y * TT, row0 = blockIdx.z * TR;
    const int kb0 = (int)((long long)p.kblocks * s / p.nsplit), kb1 = (int)((long long)p.kblocks * (s + 1) / p.nsplit);

    if (threadIdx.x == 0) {
        for (int i = 0; i < ST; i++) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], 1); }
        mbar_init(&sm->d_full, 1);
        fence_mbar_init();
        prefetch_tensormap(&amap);
        prefetch_tensormap(&xmap);
    }
    if (warp == 1) { tmem_alloc(&sm->tmem_base, TT); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the main kernel may start its own pipeline
    const uint32_t tmem = sm->tmem_base;
    bool dead = false;
    auto wait = [&](uint64_t *bar, uint32_t parity) {
        if (dead) return;
        if (!mbar_wait(bar, parity, 1u << 24)) { dead = true; atomicExch(p.status, 1); }
    };

    if (warp == 0) {
        if (lane == 0) {
            int st = 0; uint32_t ph = 0;
            for (int kb = kb0; kb < kb1; kb++) {
                wait(&sm->empty[st], ph ^ 1u);
                mbar_arrive_expect_tx(&sm->full[st], A_BYTES + B_BYTES);
                tma_load_2d(as + (size_t)st * A_BYTES, &amap, &sm->full[st], kb * KB, row0);
                tma_load_2d(bs + (size_t)st * B_BYTES, &xmap, &sm->full[st], kb * KB, tok0);
                if (++st == ST) { st = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(TR, TT);
            const uint64_t adesc0 = umma_desc_sw128(smem_u32(as)), bdesc0 = umma_desc_sw128(smem_u32(bs));
            int st = 0; uint32_t ph = 0;
            for (int kb = kb0; kb < kb1; kb++) {
                wait(&sm->full[st], ph);
                tc_fence_after();
                const uint64_t ad = adesc0 + (uint64_t)(st * (A_BYTES >> 4)), bd = bdesc0 + (uint64_t)(st * (B_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < KB / 16; kk++)
                    umma_f16_ss(tmem, ad + (uint64_t)(2 * kk), bd + (uint64_t)(2 * kk), idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
                umma_commit(&sm->empty[st]);
                if (++st == ST) { st = 0; ph ^= 1u; }
            }
            umma_commit(&sm->d_full);
        }
    } else {
        // epilogue: thread = long row (TMEM lane), columns = tokens; raw FP32 sums of this K share to the workspace
        const int q = warp & 3;
        const int row = row0 + q * 32 + lane;
        if (!dead) {
            bool ok = false;
            for (uint32_t i = 0; i < (1u << 22) && !ok; i++) {
                ok = mbar_try_wait(&sm->d_full, 0);
                if (!ok) __nanosleep(128);
            }
            if (!ok) { dead = true; atomicExch(p.status, 1); }
        }
        tc_fence_after();
        float *dst = p.part + ((size_t)s * p.n_pad + row) * p.Mp + tok0;
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
        for (int c = 0; c < TT / 32; c++) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
            tmem_ld_wait();
            if (row < p.n_long && !dead) {
                float4 *d4 = reinterpret_cast<float4 *>(dst + c * 32);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    d4[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                        __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TT); }
}

// ---- plan side: the dense copy of the long rows --------------------------------------------------------------
// One CTA per long row: writes the row's entries into the (zeroed) dense row and marks every column in a
// shared-memory bitmap; a column met twice (a CSR row that repeats a column, which the dense form cannot hold)
// raises *dup, and the plan then keeps no long rows at all.
__global__ void __launch_bounds__(256)
long_rows_densify_kernel(const uint32_t *__restrict__ entries, const int32_t *__restrict__ row_ptr,
                         const int32_t *__restrict__ hrow, int K, __half *__restrict__ dense, int *dup)
{
    __shared__ uint32_t seen[65536 / 32];
    const int h = blockIdx.x;
    for (int i = threadIdx.x; i < (K + 31) / 32; i += 256) seen[i] = 0;
    __syncthreads();
    const int n = hrow[h];
    const int e0 = row_ptr[n], e1 = row_ptr[n + 1];
    unsigned short *drow = reinterpret_cast<unsigned short *>(dense) + (size_t)h * K;
    for (int e = e0 + threadIdx.x; e < e1; e += 256) {
        const uint32_t pk = entries[e];
        const uint32_t c = pk & 0xFFFFu;
        if (atomicOr(&seen[c >> 5], 1u << (c & 31)) & (1u << (c & 31))) atomicExch(dup, 1);
        drow[c] = (unsigned short)(pk >> 16);
    }
}

static int64_t lr_mp(int64_t M) { return ceil_div(M, lg::TT) * lg::TT; }

// K shares per tile: enough CTAs to fill the GPU, at least four k blocks each
static int long_rows_splits(const Plan *pl, int64_t M)
{
    const int64_t base = (pl->n_pad / lg::TR) * (lr_mp(M) / lg::TT);
    const int64_t kblocks = ceil_div(pl->K, lg::KB);
    int64_t ns = device_sm_count(pl->device) / (base > 0 ? base : 1);
    if (ns > kblocks / 4) ns = kblocks / 4;
    if (ns > 32) ns = 32;
    return (int)(ns < 1 ? 1 : ns);
}

// Builds pl->hdense / pl->n_pad for the rows listed in pl->hrow (device) / n_long.  Returns a cudaError_t; on a
// repeated column *dup_out is set and the caller drops the long rows.
int plan_build_long_rows(Plan *pl, cudaStream_t st, bool *dup_out)
{
    *dup_out = false;
    pl->n_pad = ceil_div(pl->n_long, lg::TR) * lg::TR;
    const size_t bytes = (size_t)pl->n_pad * (size_t)pl->K * 2;
    int *d_dup = nullptr;
    cudaError_t e = cudaMalloc(&pl->hdense, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&d_dup, sizeof(int));
    if (e == cudaSuccess) e = cudaMemsetAsync(pl->hdense, 0, bytes, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_dup, 0, sizeof(int), st);
    if (e == cudaSuccess) {
        long_rows_densify_kernel<<<(unsigned)pl->n_long, 256, 0, st>>>(pl->entries, pl->row_ptr, pl->hrow, (int)pl->K,
                                                                       pl->hdense, d_dup);
        count_launch();
        e = cudaGetLastError();
    }
    int h_dup = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h_dup, d_dup, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (d_dup) cudaFree(d_dup);
    *dup_out = h_dup != 0;
    return (int)e;
}

// per-share sums: nsplit * n_pad * Mp floats
int64_t long_rows_workspace_bytes(const Plan *pl, int64_t M)
{
    if (!pl || pl->n_long == 0) return 0;
    const int64_t Mp = lr_mp(M);
    return (((int64_t)long_rows_splits(pl, M) * pl->n_pad * Mp * 4 + 255) / 256) * 256;
}

// ws: long_rows_workspace_bytes() bytes, 256-byte aligned; Mp = tokens rounded up to 256.  The sums of long row h for
// token m are  sum over s < *nsplit_out of  (*part_out)[(s * n_pad + h) * Mp + m].
int launch_long_rows(const FwdArgs &a, int Mp, void *ws, const float **part_out, int *nsplit_out)
{
    using namespace lg;
    const Plan *pl = a.plan;
    Params p;
    p.part = reinterpret_cast<float *>(ws);
    p.n_long = (int)pl->n_long; p.n_pad = (int)pl->n_pad; p.Mp = Mp;
    p.kblocks = (int)ceil_div(a.K, KB); p.nsplit = long_rows_splits(pl, a.M);
    p.status = kernel_status_word();
    if (!p.status) return ORTHO_B200_ERR_CUDA;
    CUtensorMap amap, xmap;
    if (!make_tensor_map_2d(&amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, pl->hdense, (uint64_t)pl->n_pad, (uint64_t)a.K,
                            (uint64_t)a.K * 2, TR, KB, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    if (!make_tensor_map_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                            (uint64_t)a.K * 2, TT, KB, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    static bool attr_set[kMaxDevices] = {};       // the attribute is per device
    const int dev = current_device_index();
    if (dev < 0) return ORTHO_B200_ERR_CUDA;
    if (!attr_set[dev]) {
        OB_CUDA(cudaFuncSetAttribute(long_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev] = true;
    }
    dim3 g1((unsigned)p.nsplit, (unsigned)(Mp / TT), (unsigned)(pl->n_pad / TR));
    long_gemm_kernel<<<g1, NWARPS * 32, kSmemBytes, a.stream>>>(amap, xmap, p);
    count_launch();
    OB_CUDA(cudaGetLastError());
    *part_out = p.part;
    *nsplit_out = p.nsplit;
    return ORTHO_B200_OK;
}

}  // namespace ob
