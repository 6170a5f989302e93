// Decode regime (M <= 64) on the 5th-generation tensor cores: the weight stream is converted once,
// by one thread per output row, straight into tensor memory, and one thread issues tcgen05.mma with
// a tiny token tile (N = 16/32/64).  Compared with the mma.sync streaming kernel this removes the
// per-warp MMA / B-fragment instructions and the 8-token granularity, so the cost per weight byte is
// essentially the INT4 unpack alone and does not grow with M.
//
// Decomposition: a tile is 128 output rows; a cluster of S CTAs splits K (each CTA keeps the token
// slab of its K range resident in shared memory, loaded once by TMA in the MMA's K-major 128-byte
// swizzled layout); clusters are persistent and walk the tiles round-robin.  Per CTA:
//   warp 0      TMA producer: token slab once, then a ring of packed-weight boxes (128 rows x 128 B)
//   warp 1      MMA issuer and TMEM allocator (accumulators double buffered: 2 x TM columns)
//   warps 2-9   converters: packed INT4 (smem) -> exact FP16 integers -> TMEM A operand ring;
//               two groups of four warps alternate over the 64-wide k blocks
//   warps 10-13 epilogue: tcgen05.ld the partial sums, push every row's TM partials into the shared
//               memory of the CTA that owns the row (distributed shared memory + cluster-scope
//               mbarrier), and, as owner, add the S partials in rank order, apply scale[n], add
//               alpha * O (sparse term computed by ortho_rows_kernel just before) and store FP16.
// Fixed summation order, no atomics: bitwise reproducible; alpha <= 0 or nnz == 0 skips the sparse
// kernel entirely.  Every wait is bounded and reports through the device status word.
#include "common.cuh"
#include "umma.cuh"

namespace ob {

int *kernel_status_word();

namespace dt {
constexpr int TH = 128;
constexpr int KB = 64;
constexpr int WKB = 4;                   // k blocks per packed-weight box (128 bytes per row)
constexpr int W_BYTES = TH * 128;        // 16 KB
constexpr int ASLOTS = 4;                // A-operand ring in TMEM: slots of 128 k (64 columns)
constexpr int NISSUE = 4;                // MMA issuer warps, one accumulator each
constexpr int NCG = 2;                   // converter groups: group g converts the g-th 128-k half of a weight box
constexpr int CONV_WARPS = 4 * NCG;
constexpr int CONV_WARP0 = 1 + NISSUE;
constexpr int EPI_WARP0 = CONV_WARP0 + CONV_WARPS;
constexpr int NWARPS = EPI_WARP0 + 4;

struct Params {
    const __half *scales; __half *y;
    const float *o;          // sparse term O[n][TM] (FP32) or nullptr
    float alpha;
    int M, K, N;
    long long ldy;           // elements between token rows of y
    int ntiles, nboxes;      // ceil(N/128), ceil(K/256)
    int wstages;
    int rb;                  // rows of a tile owned (finalized) by one CTA of the cluster: ceil(128 / S)
    int *status;
};

struct Bars {
    uint64_t x_ready, x_perm;
    uint64_t w_full[8], w_empty[8];
    uint64_t a_full[ASLOTS], a_empty[ASLOTS];
    uint64_t d_full[2], d_empty[2];
    uint64_t inbox_full[2], inbox_free[2];
    uint32_t tmem_base;
};
}  // namespace dt

// sparse term for the decode regime: O[n][m] = sum_i v_i x[m][c_i], one warp per output row, lanes
// stride over the row's entries, butterfly reduction per token (same scheme as the streaming kernel)
template <int TM>
__global__ void __launch_bounds__(256)
ortho_rows_kernel(OrthoView ov, const __half *__restrict__ x, float *__restrict__ o, int M, int K, int N)
{
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const int e0 = ov.row_ptr[n], e1 = ov.row_ptr[n + 1];
    float acc[TM];
#pragma unroll
    for (int m = 0; m < TM; m++) acc[m] = 0.f;
    for (int e = e0 + lane; e < e1; e += 32) {
        int c; float v;
        if (ov.entries) {
            const uint32_t pk = ov.entries[e];
            c = (int)(pk & 0xFFFFu);
            v = __half2float(__ushort_as_half((unsigned short)(pk >> 16)));
        } else {
            c = ov.col[e];
            v = __half2float(ov.val[e]);
            if ((unsigned)c >= (unsigned)K) { c = 0; v = 0.f; }
        }
#pragma unroll
        for (int m = 0; m < TM; m++)
            if (m < M) acc[m] = fmaf(v, __half2float(x[(size_t)m * K + c]), acc[m]);
    }
#pragma unroll
    for (int m = 0; m < TM; m++) {
        float s = acc[m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == (m & 31)) o[(size_t)n * TM + m] = s;
    }
}

template <int TM>
__global__ void __launch_bounds__(dt::NWARPS * 32, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const dt::Params p)
{
    using namespace dt;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = (int)cluster_nctarank(), rank = (int)cluster_ctarank();
    const int cid = blockIdx.y, G = gridDim.y;

    // this CTA's K range, in packed-weight boxes of 256 k
    const int b0 = (p.nboxes * rank) / S, b1 = (p.nboxes * (rank + 1)) / S;
    const int nbox = b1 - b0;
    const int nkb = nbox * WKB;
    const int my_tiles = (p.ntiles - cid + G - 1) / G;

    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *wring = base;                                            // wstages x 16 KB
    unsigned char *xslab = wring + (size_t)p.wstages * W_BYTES;             // nkb x (TM x 128 B)
    float *inbox = reinterpret_cast<float *>(xslab + (size_t)(((p.nboxes + S - 1) / S) * WKB) * TM * 128);   // [2][S][rb][TM]
    Bars *bar = reinterpret_cast<Bars *>(reinterpret_cast<unsigned char *>(inbox) + (size_t)2 * S * p.rb * TM * 4);

    const int rows_mine = max(0, min(p.rb, TH - rank * p.rb));              // rows of a tile this CTA finalizes

    if (threadIdx.x == 0) {
        mbar_init(&bar->x_ready, 1);
        mbar_init(&bar->x_perm, CONV_WARPS);
        for (int s = 0; s < p.wstages; s++) { mbar_init(&bar->w_full[s], 1); mbar_init(&bar->w_empty[s], CONV_WARPS); }
        for (int s = 0; s < ASLOTS; s++) { mbar_init(&bar->a_full[s], 4); mbar_init(&bar->a_empty[s], NISSUE); }
        for (int b = 0; b < 2; b++) {
            mbar_init(&bar->d_full[b], NISSUE);
            mbar_init(&bar->d_empty[b], 4);
            mbar_init(&bar->inbox_full[b], (uint32_t)max(1, S * rows_mine));
            mbar_init(&bar->inbox_free[b], (uint32_t)S);
        }
        fence_mbar_init();
        prefetch_tensormap(&xmap);
        prefetch_tensormap(&wmap);
    }
    if (warp == 1) { tmem_alloc(&bar->tmem_base, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    if (S > 1) { cluster_arrive(); cluster_wait(); }      // every CTA's barriers exist before any remote arrive
    tc_fence_after();
    const uint32_t tmem = bar->tmem_base;
    // TMEM columns: [2 buffers][NISSUE accumulators][TM], then the A ring (ASLOTS x 64 columns).  Every
    // MMA issuer owns one accumulator, so issuers never order their MMAs against each other; the
    // epilogue adds the NISSUE partial accumulators.
    const uint32_t A_COL0 = 2 * NISSUE * TM;
    bool dead = false;
    auto wait = [&](uint64_t *b, uint32_t parity) {
        if (dead) return;
        if (mbar_try_wait(b, parity)) return;
        if (!mbar_wait(b, parity, 1u << 20)) { dead = true; atomicExch(p.status, 1); }
    };

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0 && nbox > 0) {
            // weights do not depend on the previous kernel: start them before the grid dependency resolves
            int ws = 0; uint32_t wph = 0;
            int issued = 0, ti = 0, bi = 0;
            const int total = my_tiles * nbox;
            auto issue_w = [&]() {
                wait(&bar->w_empty[ws], wph ^ 1u);
                mbar_arrive_expect_tx(&bar->w_full[ws], W_BYTES);
                tma_load_2d(wring + (size_t)ws * W_BYTES, &wmap, &bar->w_full[ws], (b0 + bi) * 128, (cid + ti * G) * TH);
                if (++ws == p.wstages) { ws = 0; wph ^= 1u; }
                if (++bi == nbox) { bi = 0; ++ti; }
                issued++;
            };
            for (int i = 0; i < p.wstages && issued < total; i++) issue_w();
            asm volatile("griddepcontrol.wait;" ::: "memory");
            mbar_arrive_expect_tx(&bar->x_ready, (uint32_t)(nkb * TM * 128));
            for (int kb = 0; kb < nkb; kb++)
                tma_load_2d(xslab + (size_t)kb * TM * 128, &xmap, &bar->x_ready, (b0 * WKB + kb) * KB, 0);
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            while (issued < total) issue_w();
        } else if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
    } else if (warp < 1 + NISSUE) {
        // ================= MMA issuers: issuer j takes k steps j and j+4 of every 128-wide slot =================
        const int j = warp - 1;
        if (lane == 0 && nbox > 0) {
            const uint32_t idesc = umma_idesc_f16(TH, TM);
            const uint64_t desc0 = umma_desc_sw128(smem_u32(xslab));
            wait(&bar->x_perm, 0);                        // slab landed and was put into unpack pair order
            tc_fence_after();
            int as = 0; uint32_t aph = 0;
            const int nslots = nkb / 2;                   // slots of 128 k per tile
            for (int it = 0; it < my_tiles; it++) {
                const int b = it & 1;
                wait(&bar->d_empty[b], (uint32_t)(((it >> 1) & 1) ^ 1));
                tc_fence_after();
                const uint32_t d_tmem = tmem + (uint32_t)((b * NISSUE + j) * TM);
                for (int sl = 0; sl < nslots; sl++) {
                    wait(&bar->a_full[as], aph);
                    tc_fence_after();
                    const uint32_t a_tmem = tmem + A_COL0 + (uint32_t)(as * KB);          // 64 columns per slot
                    const uint64_t bdesc = desc0 + (uint64_t)((2 * sl) * ((TM * 128) >> 4));
                    // k step j of the slot's first k block, k step j of its second k block
                    umma_f16_ts(d_tmem, a_tmem + (uint32_t)(j * 8), bdesc + (uint64_t)(2 * j), idesc, sl != 0 ? 1u : 0u);
                    umma_f16_ts(d_tmem, a_tmem + (uint32_t)(32 + j * 8), bdesc + (uint64_t)(((TM * 128) >> 4) + 2 * j), idesc, 1u);
                    umma_commit(&bar->a_empty[as]);
                    if (++as == ASLOTS) { as = 0; aph ^= 1u; }
                }
                umma_commit(&bar->d_full[b]);
            }
        }
    } else if (warp < EPI_WARP0) {
        // ================= converters =================
        const int cw = warp - CONV_WARP0;                 // 0 .. CONV_WARPS-1
        const int q = warp & 3, grp = cw >> 2;            // TMEM lane quarter, converter group (half of a weight box)
        const int row = q * 32 + lane;
        const uint32_t swz = (uint32_t)(row & 7);
        // one-time: put the token slab into the pair order the unpack produces.  Inside every 16-byte
        // chunk (8 consecutive k of one token) (x0..x7) becomes (x0,x4,x1,x5,x2,x6,x3,x7); the 128-byte
        // swizzle only moves whole chunks, so the permutation can be applied in place, chunk by chunk.
        if (nbox > 0) {
            wait(&bar->x_ready, 0);
            uint4 *slab = reinterpret_cast<uint4 *>(xslab);
            const int nchunks = nkb * TM * 8;
            for (int i = cw * 32 + lane; i < nchunks; i += CONV_WARPS * 32) {
                const uint4 v = slab[i];
                uint4 o;
                asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o.x) : "r"(v.x), "r"(v.z));
                asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o.y) : "r"(v.x), "r"(v.z));
                asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o.z) : "r"(v.y), "r"(v.w));
                asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o.w) : "r"(v.y), "r"(v.w));
                slab[i] = o;
            }
            fence_proxy_async();                          // generic-proxy writes -> visible to the MMA's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->x_perm);
        }
        // group g converts the g-th half (128 k = 64 bytes per row) of every weight box into one A slot
        const int iters = my_tiles * nbox;
        int ws = 0; uint32_t wph = 0;
        int as = grp; uint32_t aph = 0;                   // slots alternate between the two groups
        for (int i = 0; i < iters; i++) {
            wait(&bar->w_full[ws], wph);
            const unsigned char *wrow = wring + (size_t)ws * W_BYTES + row * 128;
            uint4 wv[4];
#pragma unroll
            for (int c = 0; c < 4; c++) wv[c] = *reinterpret_cast<const uint4 *>(wrow + ((((uint32_t)(4 * grp + c)) ^ swz) << 4));
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->w_empty[ws]);
            if (++ws == p.wstages) { ws = 0; wph ^= 1u; }
            uint32_t h[64];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t ww[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
#pragma unroll
                for (int j2 = 0; j2 < 4; j2++) {
                    uint32_t o4[4];
                    int4x8_to_half2x4(ww[j2], o4);           // pair order (e0,e4)(e1,e5)(e2,e6)(e3,e7)
                    h[16 * c + 4 * j2] = o4[0]; h[16 * c + 4 * j2 + 1] = o4[1];
                    h[16 * c + 4 * j2 + 2] = o4[2]; h[16 * c + 4 * j2 + 3] = o4[3];
                }
            }
            wait(&bar->a_empty[as], aph ^ 1u);
            tc_fence_after();
            const uint32_t a_tmem = tmem + ((uint32_t)(q * 32) << 16) + A_COL0 + (uint32_t)(as * KB);
            tmem_st_32x32b_x32(a_tmem, *reinterpret_cast<const uint32_t (*)[32]>(&h[0]));
            tmem_st_32x32b_x32(a_tmem + 32, *reinterpret_cast<const uint32_t (*)[32]>(&h[32]));
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->a_full[as]);
            as += NCG;
            if (as >= ASLOTS) { as -= ASLOTS; aph ^= 1u; }
        }
    } else {
        // ================= epilogue: partial sums -> owner's inbox -> reduce, scale, sparse term, store =====
        const int q = warp & 3;
        const int row = q * 32 + lane;                      // row of the tile held by this thread (TMEM lane)
        const int et = (warp - EPI_WARP0) * 32 + lane;      // 0..127
        const int owner = row / p.rb, orow = row - owner * p.rb;
        const uint32_t inbox_base = smem_u32(inbox);
        asm volatile("griddepcontrol.wait;" ::: "memory");   // O (previous kernel) is read and Y written below
        for (int it = 0; it < my_tiles; it++) {
            const int b = it & 1;
            const uint32_t u = (uint32_t)(it >> 1);
            float d[TM];
            if (nbox > 0) {
                wait(&bar->d_full[b], u & 1u);
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < TM; j++) d[j] = 0.f;
#pragma unroll
                for (int a = 0; a < NISSUE; a++) {
#pragma unroll
                    for (int c = 0; c < TM / 16; c++) {
                        uint32_t r[16];
                        tmem_ld_32x32b_x16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)((b * NISSUE + a) * TM + c * 16), r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) d[c * 16 + j] += __uint_as_float(r[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar->d_empty[b]);
            } else {
#pragma unroll
                for (int j = 0; j < TM; j++) d[j] = 0.f;
            }
            // push this row's partials into its owner's inbox slot [b][rank][orow][:]
            if (!dead && !mbar_wait_cluster(&bar->inbox_free[b], (u & 1u) ^ 1u, 1u << 20)) { dead = true; atomicExch(p.status, 1); }
            {
                const uint32_t dst = mapa_shared(inbox_base + (uint32_t)((((b * S + rank) * p.rb + orow) * TM) * 4), (uint32_t)owner);
#pragma unroll
                for (int j = 0; j < TM; j += 4) st_dsmem_v4(dst + (uint32_t)(j * 4), make_float4(d[j], d[j + 1], d[j + 2], d[j + 3]));
                mbar_arrive_remote(mapa_shared(smem_u32(&bar->inbox_full[b]), (uint32_t)owner));
            }
            // owner side: rows [rank*rb, rank*rb + rows_mine) of this tile
            if (rows_mine > 0) {
                if (!dead && !mbar_wait_cluster(&bar->inbox_full[b], u & 1u, 1u << 20)) { dead = true; atomicExch(p.status, 1); }
                if (et < rows_mine) {
                    const int n = (cid + it * G) * TH + rank * p.rb + et;
                    if (n < p.N) {
                        const float sc = __half2float(p.scales[n]);
                        const float *ib = inbox + (size_t)(b * S) * p.rb * TM + (size_t)et * TM;
                        for (int m = 0; m < p.M; m++) {
                            float s = 0.f;
                            for (int r2 = 0; r2 < S; r2++) s += ib[(size_t)r2 * p.rb * TM + m];
                            float v = sc * s;
                            if (p.o) v = fmaf(p.alpha, p.o[(size_t)n * TM + m], v);
                            p.y[(size_t)m * (size_t)p.ldy + n] = __float2half_rn(v);
                        }
                    }
                }
            }
            named_bar_sync(1, 128);                          // all owner reads of inbox[b] are done
            if (et == 0 && rows_mine > 0) {
                for (int r2 = 0; r2 < S; r2++) mbar_arrive_remote(mapa_shared(smem_u32(&bar->inbox_free[b]), (uint32_t)r2));
            } else if (et == 0) {
                // a CTA that owns no rows never consumes its inbox: release the senders right away
                for (int r2 = 0; r2 < S; r2++) mbar_arrive_remote(mapa_shared(smem_u32(&bar->inbox_free[b]), (uint32_t)r2));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (S > 1) { cluster_arrive(); cluster_wait(); }      // nobody leaves while a peer may still write or signal here
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ---- host ----------------------------------------------------------------------------------------
static size_t tc_smem_bytes(int TM, int S, int nboxes, int wstages)
{
    const int rb = (dt::TH + S - 1) / S;
    return 1024 + (size_t)wstages * dt::W_BYTES + (size_t)((nboxes + S - 1) / S) * dt::WKB * TM * 128 +
           (size_t)2 * S * rb * TM * 4 + sizeof(dt::Bars) + 128;
}

int64_t decode_tc_workspace_bytes(int64_t M, int64_t N)
{
    const int64_t TM = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    return N * TM * 4;
}

static int g_tc_cfg[2] = {0, 0};   // {k split, weight stages}; 0 = built-in choice
void set_tc_config(int s, int stages) { g_tc_cfg[0] = s; g_tc_cfg[1] = stages; }

// picks the cluster size: the token slab must fit, every CTA needs at least one weight box, and the
// persistent grid should fill the 148 SMs in as few, as full waves as possible
static int tc_choose_split(int TM, int ntiles, int nboxes, int wstages)
{
    int best = 0; double best_eff = -1.0;
    for (int s = 1; s <= 8; s++) {
        if (s > nboxes) break;
        if (tc_smem_bytes(TM, s, nboxes, wstages) > 220 * 1024) continue;
        const int clusters = 148 / s;
        const int waves = (ntiles + clusters - 1) / clusters;
        const double eff = (double)ntiles * s / ((double)waves * 148.0);
        if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    }
    return best;
}

template <int TM>
static int launch_tc(const FwdArgs &a, int S, int wstages)
{
    using namespace dt;
    Params p;
    p.scales = a.scales; p.y = a.y; p.alpha = a.alpha; p.o = nullptr;
    p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.pitch_y();
    p.ntiles = (int)ceil_div(a.N, TH); p.nboxes = (int)ceil_div(a.K, 256);
    p.wstages = wstages; p.rb = (TH + S - 1) / S;
    p.status = kernel_status_word();
    if (!p.status) return ORTHO_B200_ERR_CUDA;
    if (a.has_ortho) {
        if (!a.workspace || a.workspace_bytes < decode_tc_workspace_bytes(a.M, a.N)) return ORTHO_B200_ERR_WORKSPACE;
        float *o = reinterpret_cast<float *>(a.workspace);
        ortho_rows_kernel<TM><<<(unsigned)ceil_div(a.N, 8), 256, 0, a.stream>>>(a.ortho, a.x, o, (int)a.M, (int)a.K, (int)a.N);
        count_launch();
        OB_CUDA(cudaGetLastError());
        p.o = o;
    }
    CUtensorMap xmap, wmap;
    if (!make_tensor_map_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                            (uint64_t)a.K * 2, TM, KB, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    if (!make_tensor_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)a.N, (uint64_t)(a.K / 2),
                            (uint64_t)(a.K / 2), TH, 128, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    const size_t smem = tc_smem_bytes(TM, S, p.nboxes, wstages);
    auto kern = decode_tc_kernel<TM>;
    static bool attr_set = false;
    if (!attr_set) {
        OB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NWARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    // persistent grid: only as many clusters as the hardware can keep resident at once (a cluster has
    // to fit inside one GPC, so this is usually fewer than 148 / S)
    static struct { int s; size_t smem; int n; } cache[16];
    static int cache_n = 0;
    int clusters = 0;
    for (int i = 0; i < cache_n; i++)
        if (cache[i].s == S && cache[i].smem == smem) clusters = cache[i].n;
    if (clusters == 0) {
        cfg.gridDim = dim3((unsigned)S, 148, 1);
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = 148 / S; }
        cfg.numAttrs = 2;
        clusters = n;
        cache[cache_n % 16] = {S, smem, n};
        if (cache_n < 16) cache_n++;
    }
    if (clusters > p.ntiles) clusters = p.ntiles;
    cfg.gridDim = dim3((unsigned)S, (unsigned)clusters, 1);
    OB_CUDA(cudaLaunchKernelEx(&cfg, kern, xmap, wmap, p));
    count_launch();
    return ORTHO_B200_OK;
}

// returns ORTHO_B200_ERR_SHAPE when the shape does not fit this kernel (caller falls back)
int launch_decode_tc(const FwdArgs &a)
{
    // 2 buffers x 4 accumulators x TM columns plus the 256-column A ring must fit 512 TMEM columns
    if (a.M > 32 || (a.K % 256) != 0) return ORTHO_B200_ERR_SHAPE;
    const int TM = a.M <= 16 ? 16 : 32;
    const int ntiles = (int)ceil_div(a.N, dt::TH), nboxes = (int)ceil_div(a.K, 256);
    int wstages = g_tc_cfg[1] > 0 ? g_tc_cfg[1] : 5;
    if (wstages > 8) wstages = 8;
    int S = g_tc_cfg[0] > 0 ? g_tc_cfg[0] : tc_choose_split(TM, ntiles, nboxes, wstages);
    while (S == 0 && wstages > 2) { wstages--; S = tc_choose_split(TM, ntiles, nboxes, wstages); }
    if (S <= 0 || S > 8 || S > nboxes || tc_smem_bytes(TM, S, nboxes, wstages) > 227 * 1024) return ORTHO_B200_ERR_SHAPE;
    if (TM == 16) return launch_tc<16>(a, S, wstages);
    return launch_tc<32>(a, S, wstages);
}

}  // namespace ob
