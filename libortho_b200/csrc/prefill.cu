// Prefill-regime (large M) OrthoLinear forward for sm_100a on the 5th-generation tensor cores.
//
// Replaces the reference's WMMA kernels (src/dual_gemm_tensor_core.cu:70-174, 215-337), which
// quantise activations to int8 and scan the whole coordinate list per output element.  Here the
// base term is a real FP16 contraction with FP32 accumulation in tensor memory:
//
//     D[n, m] = sum_k  w_int[n, k] * x[m, k]          (tcgen05.mma, kind::f16)
//     y[m, n] = scale[n] * D[n, m] + bias[n] + alpha * O[n, m]
//
// The weight tile is the M operand of the MMA and lives in TENSOR MEMORY: TMA brings the packed
// INT4 bytes (128 bytes = 256 k per row and load) into shared memory, eight converter warps (two threads per
// output row, 32 k of a block each) unpack them in registers to exact small-integer halves and write them with
// tcgen05.st, so the converted weights never touch shared memory.  The token tile (256 tokens x
// 64 k, FP16, 128-byte swizzle) is the N operand and goes from global to shared memory by TMA and
// from there straight into the MMA.  A tile is 128 output rows x 256 tokens (one 256-column FP32
// accumulator); one elected thread issues the MMAs.  The per-row scale is applied in the FP32 epilogue (it
// factors out of the K sum, src/ortho.c:356,363); outputs are transposed through shared memory and stored
// coalesced.
//
// The sparse ortho term (the reference intends its fusion into this kernel, src/dual_gemm_tensor_core.cu:324-332,
// but scans the whole coordinate list per output element) takes one of two forms:
//  * With a plan whose rows list their columns in ascending order it is FOLDED INTO THE WEIGHT TILE: as the
//    converters walk along K, each thread walks the entries of its row with them and adds v * alpha / scale[n]
//    (FP16) to the integer weight it has just unpacked, so the MMAs compute base and sparse term in one go
//    (scale[n] * (w + v alpha / scale[n]) = scale[n] w + alpha v).  No transposed activations, no gathers, no
//    extra traffic.  Rows whose corrections FP16 cannot hold (zero or tiny scale, huge values) are gathered by
//    the epilogue warps straight from X, rows a plan marks as long get their sums from the tensor-core pre-pass
//    of longrows.cu; a tile without such rows does nothing else.
//  * Otherwise (raw CSR, unordered plan) the epilogue warps compute it while the tile's MMAs run: a warp walks one
//    output row at a time with the tile's 256 tokens across its lanes and gathers 16 bytes per entry and lane
//    from the once-transposed activations Xt[k][m], eight entries in flight.
// In both forms the sums the epilogue warps produce are collected, 32 rows at a time, as FP16 in the (then idle)
// output staging tiles and moved, thread = row, into the 128 tensor-memory columns that the accumulator and the
// weight ring leave free; the FP32 epilogue adds alpha * O.
//
// TMEM columns: [0,256) accumulator, [256,384) ring of 4 converted weight stages, [384,512) sparse term.
// Warp roles (CTA = 1 SM, persistent over tiles):
//   warp 0       TMA producer           warp 1       MMA issuer, TMEM allocator
//   warps 2-9    INT4 -> FP16 (+ sparse entries) -> TMEM
//   warps 10-17  sparse term where needed, then epilogue (TMEM -> scale -> FP16 -> global): two sets of four warps
//                that take alternate 32-token chunks
//   warps 18-19  N-sharded layer only: copy each finished output tile from the local buffer to the peers' buffers
//                (plain loads and stores over NVLink) while the next tile is being computed
#include <cstring>

#include "common.cuh"
#include "gather.cuh"
#include "umma.cuh"

namespace ob {

int launch_decode(const FwdArgs &a);
int *kernel_status_word();

namespace pf {
constexpr int TH = 128;            // output rows per MMA (one TMEM accumulator, MMA M)
constexpr int NH = 1;              // accumulators per tile that share one token tile
constexpr int TN = TH * NH;        // output rows per tile
constexpr int TM = 256;            // tokens per tile        (MMA N)
constexpr int KB = 64;             // k per pipeline stage
constexpr int STAGES = 4;
constexpr int ASTAGES = 4;
constexpr int X_BYTES = TM * KB * 2;     // 32 KB
constexpr int WKB = 4;                   // k-blocks covered by one packed-weight load (128 bytes per row)
constexpr int WSTAGES = 3;
constexpr int W_BYTES = TN * 128;        // 32 KB: 256 rows x 128 B (256 k), 128-byte swizzle
constexpr int YS_PITCH = TH + 8;         // halves per staged token row (pad against bank conflicts)
constexpr int YS_BYTES = 32 * YS_PITCH * 2;
constexpr int CONV_WARPS = 8;            // two converter threads per output row of the tile (32 k of a block each)
static_assert(NH == 1, "the converter and epilogue warp layouts are written for one accumulator");
constexpr int EPI_WARP0 = 2 + CONV_WARPS;
constexpr int ESETS = 2;                 // epilogue warp sets per accumulator: set e drains the 32-token chunks c = e, e + 2, ...
constexpr int EPI_WARPS = 4 * NH * ESETS;
constexpr int PUSH_WARP0 = EPI_WARP0 + EPI_WARPS;
constexpr int PUSH_WARPS = 2;            // N-sharded layer: copy every finished output tile to the peers while the next tile runs
constexpr int NWARPS = PUSH_WARP0 + PUSH_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int A_COL0 = NH * TM;          // accumulators occupy [0, NH*TM); converted weights follow
constexpr int A_STAGE_COLS = NH * (KB / 2);
constexpr int O_COL0 = A_COL0 + ASTAGES * A_STAGE_COLS;   // sparse term: 256 tokens as FP16 pairs = 128 columns
static_assert(O_COL0 + TM / 2 <= TMEM_COLS, "tensor memory layout");
constexpr int OB_PITCH = TM + 8;         // halves per row of the sparse term's 32-row batch buffer (pad against bank conflicts)
static_assert(32 * OB_PITCH * 2 <= NH * ESETS * YS_BYTES, "the batch buffer lives in the staging tiles");

struct Params {
    const __half *scales; __half *y;
    const float *bias;      // optional FP32 [N], added in the FP32 epilogue
    int M, K, N;
    long long ldy;          // elements between token rows of y
    int tiles_n, tiles_m, kblocks;
    int *status;
    // sparse term: CSR view (plan entries or raw arrays) and the transposed activations Xt[k][Mp] (zero for m >= M)
    OrthoView ov; const __half *xt; int Mp; float alpha; int has_ortho;
    // long rows of the plan: the pre-pass of longrows.cu leaves their sums as ol_splits FP32 shares,
    // ol[(s * ol_pad + h) * Mp + m] for share s, long row h, token m
    const float *ol; int ol_splits, ol_pad; const int32_t *hrow; int n_long, heavy;
    // patch != 0 (a plan whose rows list their columns in ascending order): the converters add the sparse entries
    // to the weight tile itself (see the kernel's header); row_max[n] = largest |value| of row n, x = the
    // activations in their own layout for the rows that cannot be patched
    int patch; const float *row_max; const __half *x;
    // split-K of the last, partial wave: tiles [full_tiles, full_tiles + n_split) are each worked on by two
    // CTAs (k-blocks [0, kh) and [kh, kblocks)); the second one leaves its raw FP32 accumulators in
    // part[j][128][TM] and raises flags[j], the first one adds them in its epilogue
    int full_tiles, n_split, kh;
    float *part; int *flags;
    // N-sharded layer: the epilogue stores every output tile into all ranks' buffers (peer stores over NVLink,
    // overlapped tile by tile with the MMAs of the following tiles) and the last CTA exchanges the flags
    int gather;
    GatherView gv;
};

struct Unit { int t, kb0, kb1, role, j; };      // role 0: whole tile, 1: first K half (final), 2: second K half (partial)
__device__ __forceinline__ Unit unit_of(const Params &p, int u) {
    Unit r;
    if (u < p.full_tiles) { r.t = u; r.kb0 = 0; r.kb1 = p.kblocks; r.role = 0; r.j = 0; return r; }
    const int v = u - p.full_tiles;
    r.j = v >> 1; r.t = p.full_tiles + r.j;
    if (v & 1) { r.kb0 = p.kh; r.kb1 = p.kblocks; r.role = 2; } else { r.kb0 = 0; r.kb1 = p.kh; r.role = 1; }
    return r;
}
constexpr int kMaxSplit = 74;                               // at most half of the SMs' worth of split tiles
constexpr size_t kSplitPartBytes = (size_t)kMaxSplit * TH * TM * 4;
constexpr size_t kSplitBytes = kSplitPartBytes + 1024;      // partial tiles, then the flag words

struct Smem {
    uint64_t x_full[STAGES], x_empty[STAGES];
    uint64_t w_full[WSTAGES], w_empty[WSTAGES];
    uint64_t a_full[ASTAGES], a_empty[ASTAGES];
    uint64_t d_full, d_empty;
    uint64_t y_done;            // the epilogue warps have stored a tile to the local output (gathering forward)
    uint32_t tmem_base;
};

constexpr int DL_BYTES = TN * KB * 2;     // 16 KB: one row of 64 FP16 weight corrections per converter thread
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * X_BYTES + (size_t)WSTAGES * W_BYTES + NH * ESETS * YS_BYTES + DL_BYTES + sizeof(Smem) + 256;
static_assert(kSmemBytes <= 232448, "shared memory per CTA");

}  // namespace pf

__global__ void __launch_bounds__(pf::NWARPS * 32, 1)
prefill_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const pf::Params p)
{
    using namespace pf;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *xs = base;                                       // STAGES x 16 KB, 1 KB aligned
    unsigned char *ws = xs + (size_t)STAGES * X_BYTES;              // WSTAGES x 32 KB, 1 KB aligned
    unsigned char *ys_base = ws + (size_t)WSTAGES * W_BYTES;        // NH staging tiles for the transposed store
    unsigned char *dl_base = ys_base + NH * ESETS * YS_BYTES;       // weight corrections of the current k block
    Smem *sm = reinterpret_cast<Smem *>(dl_base + DL_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nunits = p.full_tiles + 2 * p.n_split;       // work units of the grid (a split tile counts twice)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&sm->x_full[s], 1); mbar_init(&sm->x_empty[s], 1); }
        for (int s = 0; s < WSTAGES; s++) { mbar_init(&sm->w_full[s], 1); mbar_init(&sm->w_empty[s], CONV_WARPS); }
        for (int s = 0; s < ASTAGES; s++) { mbar_init(&sm->a_full[s], CONV_WARPS); mbar_init(&sm->a_empty[s], 1); }
        mbar_init(&sm->d_full, 1);
        mbar_init(&sm->d_empty, EPI_WARPS);
        mbar_init(&sm->y_done, EPI_WARPS);
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
            int s = 0, wsi = 0; uint32_t ph = 0, wph = 0;
            for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
                const Unit un = unit_of(p, u);
                const int nt = un.t % p.tiles_n, mt = un.t / p.tiles_n;
                for (int kb = un.kb0; kb < un.kb1; kb++) {
                    if ((kb % WKB) == 0) {      // packed weights: one 128-byte-wide load per WKB k-blocks
                        wait(&sm->w_empty[wsi], wph ^ 1u);
                        mbar_arrive_expect_tx(&sm->w_full[wsi], W_BYTES);
                        tma_load_2d(ws + (size_t)wsi * W_BYTES, &wmap, &sm->w_full[wsi], kb * (KB / 2), nt * TN);
                        if (++wsi == WSTAGES) { wsi = 0; wph ^= 1u; }
                    }
                    wait(&sm->x_empty[s], ph ^ 1u);
                    mbar_arrive_expect_tx(&sm->x_full[s], X_BYTES);
                    tma_load_2d(xs + (size_t)s * X_BYTES, &xmap, &sm->x_full[s], kb * KB, mt * TM);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(TH, TM);
            const uint64_t desc0 = umma_desc_sw128(smem_u32(xs));     // stage s, k step kk: + s*X_BYTES/16 + 2*kk
            int s = 0, as = 0; uint32_t ph = 0, aph = 0;
            int it = 0;
            for (int u = blockIdx.x; u < nunits; u += gridDim.x, it++) {
                const Unit un = unit_of(p, u);
                wait(&sm->d_empty, (uint32_t)((it & 1) ^ 1));     // the epilogue has drained the accumulators
                tc_fence_after();
                for (int kb = un.kb0; kb < un.kb1; kb++) {
                    wait(&sm->x_full[s], ph);
                    wait(&sm->a_full[as], aph);
                    tc_fence_after();
                    const uint32_t a_tmem = tmem + (uint32_t)(A_COL0 + as * A_STAGE_COLS);
                    const uint64_t bdesc = desc0 + (uint64_t)(s * (X_BYTES >> 4));
                    const uint32_t acc0 = (uint32_t)(kb != un.kb0);
#pragma unroll
                    for (int kk = 0; kk < KB / 16; kk++) {
#pragma unroll
                        for (int h = 0; h < NH; h++)
                            umma_f16_ts(tmem + (uint32_t)(h * TM), a_tmem + (uint32_t)(h * (KB / 2) + kk * 8),
                                        bdesc + (uint64_t)(2 * kk), idesc, kk == 0 ? acc0 : 1u);
                    }
                    umma_commit(&sm->x_empty[s]);
                    umma_commit(&sm->a_empty[as]);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                    if (++as == ASTAGES) { as = 0; aph ^= 1u; }
                }
                umma_commit(&sm->d_full);
            }
        }
    } else if (warp < EPI_WARP0) {
        // ================= converters: packed INT4 (smem) -> FP16 (TMEM, A operand) =================
        // two threads per output row: thread (row, half) converts k [32 half, 32 half + 32) of every k block
        const int q = warp & 3;                        // TMEM lane quarter this warp may touch
        const int half = (warp - 2) >> 2;              // which 32 k of the block's 64
        const int row = q * 32 + lane;                 // output row inside the tile
        int wsi = 0, as = 0; uint32_t wph = 0, aph = 0;
        const uint32_t swz = (uint32_t)(row & 7);      // 128-byte swizzle: 16-byte chunk c sits at c ^ (row & 7)
        // Patch mode: this thread walks the sparse entries of its row in column order along the k blocks (both
        // threads of a row walk all of them and each keeps those of its own half), a window of four entries in
        // registers.  An entry v becomes the FP16 correction v * alpha / scale[row], dropped into this thread's private
        // 32 corrections in shared memory and added to the converted weights (no synchronisation: nobody else
        // touches them).
        __half *dlrow = reinterpret_cast<__half *>(dl_base) + half * (TN * 32) + row * 32;     // four 16-byte chunks, swizzled
        const uint32_t dsw = (uint32_t)((row >> 1) & 3);
        if (p.patch) {
#pragma unroll
            for (int j = 0; j < 4; j++) reinterpret_cast<uint4 *>(dlrow)[j] = make_uint4(0, 0, 0, 0);
        }
        int pend_as = -1;                                                // stage whose tcgen05.st is still on its way
        for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
            const Unit un = unit_of(p, u);
            int e_cur = 0, e_end = 0; float rsc = 0.f;
            uint32_t w0 = 0, w1 = 0, w2 = 0, w3 = 0;
            if (p.patch) {
                const int n = (un.t % p.tiles_n) * TN + row;
                if (n < p.N) {
                    const int e0 = p.ov.row_ptr[n], e1 = p.ov.row_ptr[n + 1];
                    if (e1 > e0 && !(p.n_long > 0 && e1 - e0 > p.heavy)) {
                        rsc = patch_rscale(p.alpha, __half2float(p.scales[n]), p.row_max[n]);
                        if (rsc != 0.f) { e_cur = e0; e_end = e1; }
                    }
                }
                if (un.kb0 > 0 && e_cur < e_end) {          // second K half of a split tile: first entry at or past its start
                    int lo = e_cur, hi = e_end;
                    const uint32_t c0 = (uint32_t)(un.kb0 * KB);
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if ((p.ov.entries[mid] & 0xFFFFu) < c0) lo = mid + 1; else hi = mid;
                    }
                    e_cur = lo;
                }
                if (e_cur < e_end) w0 = p.ov.entries[e_cur];
                if (e_cur + 1 < e_end) w1 = p.ov.entries[e_cur + 1];
                if (e_cur + 2 < e_end) w2 = p.ov.entries[e_cur + 2];
                if (e_cur + 3 < e_end) w3 = p.ov.entries[e_cur + 3];
            }
            for (int kb4 = un.kb0; kb4 < un.kb1; kb4 += WKB) {
                // one packed-weight stage = four k blocks (kb0 is a multiple of four): this thread's four 16-byte slices
                // go to registers at once and the stage is handed back right away, so that its next load has the
                // time of three more k blocks to arrive
                wait(&sm->w_full[wsi], wph);
                const unsigned char *wrow = ws + (size_t)wsi * W_BYTES + row * 128;
                uint4 wq[WKB];
#pragma unroll
                for (int sub = 0; sub < WKB; sub++)
                    wq[sub] = *reinterpret_cast<const uint4 *>(wrow + ((((uint32_t)(2 * sub + half)) ^ swz) << 4));
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->w_empty[wsi]);
                if (++wsi == WSTAGES) { wsi = 0; wph ^= 1u; }
#pragma unroll
                for (int sub = 0; sub < WKB; sub++) {
                const int kb = kb4 + sub;
                if (kb >= un.kb1) break;
                const uint4 wa = wq[sub];
                uint32_t hreg[16];
                const uint32_t ww[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t o[4];
                    int4x8_to_half2x4_natural(ww[j], o);
                    hreg[4 * j] = o[0]; hreg[4 * j + 1] = o[1]; hreg[4 * j + 2] = o[2]; hreg[4 * j + 3] = o[3];
                }
                if (p.patch) {
                    // entries of this row inside the k block: w_int + v * alpha / scale, as FP16
                    const int kend = (kb + 1) * KB;
                    bool mine = false;
                    while (e_cur < e_end && (int)(w0 & 0xFFFFu) < kend) {
                        const int c = (int)(w0 & 0xFFFFu) - kb * KB;
                        if ((c >> 5) == half) {
                            const float d = __half2float(__ushort_as_half((unsigned short)(w0 >> 16))) * rsc;
                            dlrow[(((((uint32_t)c >> 3) & 3u) ^ dsw) << 3) + (c & 7)] = __float2half_rn(d);
                            mine = true;
                        }
                        e_cur++;
                        w0 = w1; w1 = w2; w2 = w3;
                        w3 = (e_cur + 3 < e_end) ? p.ov.entries[e_cur + 3] : 0u;
                    }
                    if (__any_sync(0xffffffffu, mine)) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint4 dv = *reinterpret_cast<const uint4 *>(dlrow + ((((uint32_t)j) ^ dsw) << 3));
                            const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const __half2 sum = __hadd2(*reinterpret_cast<const __half2 *>(&hreg[4 * j + i]),
                                                            *reinterpret_cast<const __half2 *>(&dw[i]));
                                hreg[4 * j + i] = *reinterpret_cast<const uint32_t *>(&sum);
                            }
                        }
                        if (mine) {
#pragma unroll
                            for (int j = 0; j < 4; j++) reinterpret_cast<uint4 *>(dlrow)[j] = make_uint4(0, 0, 0, 0);
                        }
                    }
                }
                // the store of the previous k block has had this block's conversion to complete: publish it now,
                // then start this block's store (its completion is awaited one block later)
                if (pend_as >= 0) {
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->a_full[pend_as]);
                }
                wait(&sm->a_empty[as], aph ^ 1u);
                tc_fence_after();
                tmem_st_32x32b_x16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(A_COL0 + as * A_STAGE_COLS + half * (KB / 4)), hreg);
                pend_as = as;
                if (++as == ASTAGES) { as = 0; aph ^= 1u; }
                }
            }
        }
        if (pend_as >= 0) {
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->a_full[pend_as]);
        }
    } else if (warp < PUSH_WARP0) {
        // ================= epilogue: TMEM -> scale -> FP16 -> shared (transpose) -> global =================
        // these warps alone read what the long-row pre-pass wrote: they wait for it here, the other warps do not
        if (p.n_long > 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        const int q = warp & 3;
        const int h = 0;                               // accumulator handled by this warp set (NH == 1)
        const int eset = (warp - EPI_WARP0) >> 2;      // which set of four warps: it drains chunks eset, eset + ESETS, ...
        const int et = ((warp - EPI_WARP0) & 3) * 32 + lane;   // 0..127 inside the set
        __half *ys = reinterpret_cast<__half *>(ys_base + eset * YS_BYTES);
        static_assert(NH == 1, "the epilogue warp sets are laid out for one accumulator");
        const bool vec_ok = (p.N % 8) == 0 && (p.ldy % 8) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0;
        // N-sharded layer: with 16-byte alignment the epilogue stores to the local buffer only (p.y) and the push warps
        // copy the finished tile to the peers while the next tile is being computed; otherwise the epilogue stores to
        // every rank itself
        const bool push_split = p.gather && vec_ok;
        int it = 0;
        for (int u = blockIdx.x; u < nunits; u += gridDim.x, it++) {
            const Unit un = unit_of(p, u);
            const int nt = un.t % p.tiles_n, mt = un.t / p.tiles_n;
            const int nbase = nt * TN + h * TH;
            if (un.role == 2) {
                // second K half of a split tile: raw accumulators to the partial buffer, then the flag
                float *prow = p.part + ((size_t)un.j * TH + (size_t)(q * 32 + lane)) * TM;
                wait(&sm->d_full, (uint32_t)(it & 1));
                tc_fence_after();
                for (int c = eset; c < TM / 32; c += ESETS) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * TM + c * 32), r);
                    tmem_ld_wait();
                    float4 *dst = reinterpret_cast<float4 *>(prow + c * 32);
#pragma unroll
                    for (int j4 = 0; j4 < 8; j4++)
                        dst[j4] = make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]),
                                              __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->d_empty);
                __threadfence();
                named_bar_sync(1 + eset, 128);
                // every set counts itself in; the partner waits for all ESETS of them
                if (et == 0) asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p.flags + un.j), "r"(1) : "memory");
                continue;
            }
            const int n = nbase + q * 32 + lane;
            const float sc = (n < p.N) ? __half2float(p.scales[n]) : 0.f;
            const float bs = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            // ---- sparse term of this tile, computed while its MMAs run: O[row][token] -> FP16 -> tensor memory ----
            // A warp walks one row at a time with the 256 tokens of the tile across its lanes (8 per lane, one 16-byte
            // gather per entry and lane, eight entries in flight).  The eight warps fill a 32-row batch (one
            // tensor-memory lane quarter) in the staging tiles, then the two warps of that quarter, which alone may
            // touch those lanes, move it into tensor memory with thread = row.
            bool with_o = p.has_ortho != 0;
            const int ew = warp - EPI_WARP0;
            // Patch mode: the converters fold the entries of ordinary rows into the weight tile, which leaves two kinds
            // of rows to this pass: long rows of the plan (their sums exist already) and rows whose corrections FP16
            // cannot hold (gathered here, straight from X).  Lane l < 16 classifies this warp's row l of the tile
            // (batch l / 4, row l % 4 of the batch); a tile without such rows skips the pass altogether.
            int my_e0 = 0, my_e1 = 0, my_li = -1, my_mode = 0;       // mode 1: long row, 2: gather from X
            if (with_o && p.patch) {
                if (lane < 16) {
                    const int nrow = nbase + (lane >> 2) * 32 + ew * 4 + (lane & 3);
                    if (nrow < p.N) { my_e0 = p.ov.row_ptr[nrow]; my_e1 = p.ov.row_ptr[nrow + 1]; }
                    if (my_e1 > my_e0) {
                        if (p.n_long > 0 && my_e1 - my_e0 > p.heavy) {
                            int lo = 0, hi = p.n_long - 1;
                            while (lo < hi) {
                                const int mid = (lo + hi) >> 1;
                                if (p.hrow[mid] < nrow) lo = mid + 1; else hi = mid;
                            }
                            my_li = lo; my_mode = 1;
                        } else if (patch_rscale(p.alpha, __half2float(p.scales[nrow]), p.row_max[nrow]) == 0.f) {
                            my_mode = 2;
                        }
                    }
                }
                uint32_t any_row;
                asm volatile(
                    "{\n\t.reg .pred pi, po;\n\t"
                    "setp.ne.u32 pi, %1, 0;\n\t"
                    "bar.red.or.pred po, 3, %2, pi;\n\t"
                    "selp.u32 %0, 1, 0, po;\n\t}"
                    : "=r"(any_row) : "r"((uint32_t)(my_mode != 0)), "r"(EPI_WARPS * 32) : "memory");
                with_o = any_row != 0;
            }
            if (with_o) {
                __half *obuf = reinterpret_cast<__half *>(ys_base);          // [32][OB_PITCH]
                const __half *xtile = p.xt + (size_t)mt * TM + lane * 8;       // + col * Mp
                for (int qq = 0; qq < 4; qq++) {
                    for (int i = 0; i < 4; i++) {
                        const int r = ew * 4 + i;                              // row inside the quarter
                        const int nrow = nbase + qq * 32 + r;
                        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        int e0 = 0, e1 = 0, li = -1;
                        if (p.patch) {
                            const int mode = __shfl_sync(0xffffffffu, my_mode, qq * 4 + i);
                            li = __shfl_sync(0xffffffffu, my_li, qq * 4 + i);
                            if (mode == 2) {
                                // a row outside the FP16 range of the weight tile: every entry against the lane's eight
                                // tokens of X in its own layout (uncoalesced; such rows are rare)
                                const int ea = __shfl_sync(0xffffffffu, my_e0, qq * 4 + i), eb2 = __shfl_sync(0xffffffffu, my_e1, qq * 4 + i);
                                for (int e = ea; e < eb2; e++) {
                                    int c; float v;
                                    ortho_entry(p.ov, e, p.K, c, v);
#pragma unroll
                                    for (int t = 0; t < 8; t++) {
                                        const int m = mt * TM + lane * 8 + t;
                                        if (m < p.M) acc[t] = fmaf(v, __half2float(p.x[(size_t)m * p.K + c]), acc[t]);
                                    }
                                }
                            }
                        } else {
                            if (nrow < p.N) { e0 = p.ov.row_ptr[nrow]; e1 = p.ov.row_ptr[nrow + 1]; }
                            if (p.n_long > 0 && e1 - e0 > p.heavy) {           // a long row of the plan: its sums were computed ahead
                                int lo = 0, hi = p.n_long - 1;
                                while (lo < hi) {
                                    const int mid = (lo + hi) >> 1;
                                    if (p.hrow[mid] < nrow) lo = mid + 1; else hi = mid;
                                }
                                if (p.hrow[lo] == nrow) li = lo;
                            }
                        }
                        if (li >= 0) {
                            const float *src = p.ol + (size_t)li * p.Mp + (size_t)mt * TM + lane * 8;
                            const size_t sstride = (size_t)p.ol_pad * p.Mp;
                            for (int s2 = 0; s2 < p.ol_splits; s2 += 4) {             // four shares in flight, added in share order
                                float4 a0[4], a1[4];
#pragma unroll
                                for (int i2 = 0; i2 < 4; i2++) {
                                    if (s2 + i2 < p.ol_splits) {
                                        const float4 *sp = reinterpret_cast<const float4 *>(src + (size_t)(s2 + i2) * sstride);
                                        a0[i2] = __ldcg(sp); a1[i2] = __ldcg(sp + 1);
                                    }
                                }
#pragma unroll
                                for (int i2 = 0; i2 < 4; i2++) {
                                    if (s2 + i2 < p.ol_splits) {
                                        acc[0] += a0[i2].x; acc[1] += a0[i2].y; acc[2] += a0[i2].z; acc[3] += a0[i2].w;
                                        acc[4] += a1[i2].x; acc[5] += a1[i2].y; acc[6] += a1[i2].z; acc[7] += a1[i2].w;
                                    }
                                }
                            }
                        } else {
                            for (int eb = e0; eb < e1; eb += 32) {
                                int cl = 0; float vl = 0.f;
                                if (eb + lane < e1) ortho_entry(p.ov, eb + lane, p.K, cl, vl);
                                const int nb = min(32, e1 - eb);
                                for (int j0 = 0; j0 < nb; j0 += 8) {
                                    uint4 xv[8]; float vv[8];
#pragma unroll
                                    for (int j = 0; j < 8; j++) {
                                        const int cc = __shfl_sync(0xffffffffu, cl, (j0 + j) & 31);
                                        vv[j] = __shfl_sync(0xffffffffu, vl, (j0 + j) & 31);      // slots past the row hold v = 0, c = 0
                                        xv[j] = __ldg(reinterpret_cast<const uint4 *>(xtile + (size_t)cc * p.Mp));
                                    }
#pragma unroll
                                    for (int j = 0; j < 8; j++) {
                                        const __half2 *h = reinterpret_cast<const __half2 *>(&xv[j]);
#pragma unroll
                                        for (int q2 = 0; q2 < 4; q2++) {
                                            const float2 f = __half22float2(h[q2]);
                                            acc[2 * q2] = fmaf(vv[j], f.x, acc[2 * q2]);
                                            acc[2 * q2 + 1] = fmaf(vv[j], f.y, acc[2 * q2 + 1]);
                                        }
                                    }
                                }
                            }
                        }
                        const __half2 h0 = __floats2half2_rn(acc[0], acc[1]), h1 = __floats2half2_rn(acc[2], acc[3]);
                        const __half2 h2 = __floats2half2_rn(acc[4], acc[5]), h3 = __floats2half2_rn(acc[6], acc[7]);
                        *reinterpret_cast<uint4 *>(obuf + r * OB_PITCH + lane * 8) =
                            make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                                       *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
                    }
                    named_bar_sync(3, EPI_WARPS * 32);           // the batch is complete
                    if (q == qq) {
                        for (int c = eset; c < TM / 32; c += ESETS) {
                            const uint4 *src = reinterpret_cast<const uint4 *>(obuf + lane * OB_PITCH + c * 32);
                            uint32_t hp[16];
#pragma unroll
                            for (int j4 = 0; j4 < 4; j4++) {
                                const uint4 u = src[j4];
                                hp[4 * j4] = u.x; hp[4 * j4 + 1] = u.y; hp[4 * j4 + 2] = u.z; hp[4 * j4 + 3] = u.w;
                            }
                            tmem_st_32x32b_x16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(O_COL0 + c * 16), hp);
                        }
                    }
                    named_bar_sync(3, EPI_WARPS * 32);           // the batch buffer is free again
                }
                tmem_st_wait();
            }
            wait(&sm->d_full, (uint32_t)(it & 1));
            tc_fence_after();
            const float *prow = nullptr;               // first K half of a split tile: the partner's partial sums
            if (un.role == 1) {
                if (et == 0 && !dead) {                // bounded wait for the partner's flag
                    int seen = 0;
                    for (unsigned spin = 0; spin < (1u << 22); spin++) {
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.flags + un.j) : "memory");
                        if (seen >= ESETS) break;
                        __nanosleep(64);
                    }
                    if (seen < ESETS) atomicExch(p.status, 1);
                }
                named_bar_sync(1 + eset, 128);
                prow = p.part + ((size_t)un.j * TH + (size_t)(q * 32 + lane)) * TM;
            }
            // the partner's partial sums are fetched one chunk ahead, like the sparse term
            float4 pv[8];
            auto load_p = [&](int c) {
                const float4 *p4 = reinterpret_cast<const float4 *>(prow + c * 32);
#pragma unroll
                for (int j4 = 0; j4 < 8; j4++) pv[j4] = __ldcg(p4 + j4);
            };
            if (prow) load_p(eset);
            for (int c = eset; c < TM / 32; c += ESETS) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * TM + c * 32), r);
                tmem_ld_wait();
                if (prow) {
#pragma unroll
                    for (int j4 = 0; j4 < 8; j4++) {
                        r[4 * j4 + 0] = __float_as_uint(__uint_as_float(r[4 * j4 + 0]) + pv[j4].x);
                        r[4 * j4 + 1] = __float_as_uint(__uint_as_float(r[4 * j4 + 1]) + pv[j4].y);
                        r[4 * j4 + 2] = __float_as_uint(__uint_as_float(r[4 * j4 + 2]) + pv[j4].z);
                        r[4 * j4 + 3] = __float_as_uint(__uint_as_float(r[4 * j4 + 3]) + pv[j4].w);
                    }
                    if (c + ESETS < TM / 32) load_p(c + ESETS);
                }
                if (with_o) {                          // y = scale * D + bias + alpha * O
                    uint32_t ho[16];
                    tmem_ld_32x32b_x16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(O_COL0 + c * 16), ho);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float2 o2 = __half22float2(*reinterpret_cast<const __half2 *>(&ho[j]));
                        ys[(2 * j) * YS_PITCH + q * 32 + lane] = __float2half_rn(fmaf(p.alpha, o2.x, fmaf(__uint_as_float(r[2 * j]), sc, bs)));
                        ys[(2 * j + 1) * YS_PITCH + q * 32 + lane] = __float2half_rn(fmaf(p.alpha, o2.y, fmaf(__uint_as_float(r[2 * j + 1]), sc, bs)));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) ys[j * YS_PITCH + q * 32 + lane] = __float2half_rn(fmaf(__uint_as_float(r[j]), sc, bs));
                }
                named_bar_sync(1 + eset, 128);
#pragma unroll
                for (int i2 = 0; i2 < 4; i2++) {
                    const int id = i2 * 128 + et, tok = id >> 4, part = id & 15;
                    const int m = mt * TM + c * 32 + tok, n0 = nbase + part * 8;
                    if (m < p.M && n0 < p.N) {
                        const __half *src = ys + tok * YS_PITCH + part * 8;
                        __half *dst = p.y + (size_t)m * (size_t)p.ldy + n0;
                        if (!p.gather || push_split) {
                            if (vec_ok) {
                                *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
                            } else {
                                for (int e = 0; e < 8 && n0 + e < p.N; e++) dst[e] = src[e];
                            }
                        } else {
                            const size_t at = (size_t)m * (size_t)p.ldy + n0;
                            if (vec_ok) {
                                const uint4 v = *reinterpret_cast<const uint4 *>(src);
                                for (int r = 0; r < p.gv.world; r++) *reinterpret_cast<uint4 *>(p.gv.y[r] + at) = v;
                            } else {
                                for (int r = 0; r < p.gv.world; r++)
                                    for (int e = 0; e < 8 && n0 + e < p.N; e++) p.gv.y[r][at + e] = src[e];
                            }
                        }
                    }
                }
                named_bar_sync(1 + eset, 128);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->d_empty);
            if (push_split) {                          // this warp's share of the tile is in the local buffer
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->y_done);
            }
        }
    } else if (warp >= PUSH_WARP0) {
        // ================= push warps (gathering forward): local output tile -> every peer, over NVLink =================
        // plain 16-byte loads (through L2) and stores; the tile of unit u travels while unit u + 1 is being computed
        const bool vec_ok = (p.N % 8) == 0 && (p.ldy % 8) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0;
        if (p.gather && vec_ok) {
            const int pt = (warp - PUSH_WARP0) * 32 + lane;       // 0..63: token row pt / 16 of a group, 16-byte piece pt % 16
            int done = 0;
            for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
                const Unit un = unit_of(p, u);
                if (un.role == 2) continue;                        // the second K half of a split tile writes no output
                const int nt = un.t % p.tiles_n, mt = un.t / p.tiles_n;
                wait(&sm->y_done, (uint32_t)(done & 1));
                done++;
                const int n0 = nt * TN + (pt & 15) * 8;
                if (n0 >= p.N) continue;
                constexpr int PU = 4;                              // loads in flight per lane
                for (int r0 = 0; r0 < TM; r0 += PUSH_WARPS * 2 * PU) {
                    uint4 v[PU];
#pragma unroll
                    for (int i = 0; i < PU; i++) {
                        const int m = mt * TM + r0 + i * PUSH_WARPS * 2 + (pt >> 4);
                        if (m < p.M) v[i] = __ldcg(reinterpret_cast<const uint4 *>(p.y + (size_t)m * (size_t)p.ldy + n0));
                    }
#pragma unroll
                    for (int i = 0; i < PU; i++) {
                        const int m = mt * TM + r0 + i * PUSH_WARPS * 2 + (pt >> 4);
                        if (m >= p.M) continue;
                        const size_t at = (size_t)m * (size_t)p.ldy + n0;
                        for (int r = 0; r < p.gv.world; r++)
                            if (r != p.gv.rank) *reinterpret_cast<uint4 *>(p.gv.y[r] + at) = v[i];
                    }
                }
            }
        }
    }

    if (p.gather) {
        if (!gather_signal_and_wait(p.gv, gridDim.x)) atomicExch(p.status, 2);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

int launch_transpose_x(const __half *x, __half *xt, int M, int K, int Mp, cudaStream_t stream);   // transpose.cu

// workspace layout: [ Xt : K * Mp halves, Mp = M rounded up to 256 ][ split-K partial tiles + flags ]
static int64_t prefill_mp(int64_t M) { return ceil_div(M, pf::TM) * pf::TM; }
static int64_t prefill_xt_bytes(int64_t M, int64_t K) { return ((K * prefill_mp(M) * 2 + 255) / 256) * 256; }
// what the sparse term needs (the forward refuses less when the ortho term is active) ...
int64_t prefill_min_workspace_bytes(int64_t M, int64_t K, int64_t N) { (void)N; return prefill_xt_bytes(M, K); }
// ... and what ortho_b200_workspace_bytes() reports: room behind it for the split-K partial tiles, which the
// forward uses when it is there (also for base-only calls) and does without otherwise
int64_t prefill_workspace_bytes(int64_t M, int64_t K, int64_t N)
{
    (void)N;
    return prefill_xt_bytes(M, K) + (int64_t)pf::kSplitBytes;
}

int launch_prefill(const FwdArgs &a)
{
    using namespace pf;
    Params p;
    memset(&p, 0, sizeof(p));
    p.alpha = a.alpha; p.has_ortho = 0; p.K = (int)a.K;
    if (a.has_ortho) {
        const int Mp = (int)prefill_mp(a.M);
        p.ov = a.ortho; p.Mp = Mp; p.has_ortho = 1;
        // With a plan whose rows are in column order the sparse entries are folded into the weight tile by the
        // converters; otherwise the activations are transposed once per forward (Xt[k][m]) so that one sparse entry
        // touches a contiguous run of tokens, and the epilogue warps gather the term.
        p.patch = (a.plan && a.ortho.entries && a.plan->ordered && a.plan->row_max && tuning_snapshot().patch_weights) ? 1 : 0;
        if (p.patch) {
            p.row_max = a.plan->row_max; p.x = a.x;
        } else {
            if (!a.workspace || a.workspace_bytes < prefill_xt_bytes(a.M, a.K)) return ORTHO_B200_ERR_WORKSPACE;
            if (((uintptr_t)a.workspace & 255u) != 0) return ORTHO_B200_ERR_ALIGN;
            __half *xt = reinterpret_cast<__half *>(a.workspace);
            const int st = launch_transpose_x(a.x, xt, (int)a.M, (int)a.K, Mp, a.stream);
            if (st != ORTHO_B200_OK) return st;
            p.xt = xt;
        }
        if (a.plan && a.ortho.entries && a.plan->n_long > 0) {
            // the long rows' pre-pass keeps its place behind the (in patch mode unused) transposed activations
            const int64_t lr = long_rows_workspace_bytes(a.plan, a.M);
            if (!a.workspace || a.workspace_bytes < prefill_xt_bytes(a.M, a.K) + lr) return ORTHO_B200_ERR_WORKSPACE;
            if (((uintptr_t)a.workspace & 255u) != 0) return ORTHO_B200_ERR_ALIGN;
            p.hrow = a.plan->hrow; p.n_long = (int)a.plan->n_long; p.heavy = a.plan->heavy; p.ol_pad = (int)a.plan->n_pad;
        }
    }
    CUtensorMap xmap, wmap;
    if (!make_tensor_map_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                            (uint64_t)a.K * 2, TM, KB, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    if (!make_tensor_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)a.N, (uint64_t)(a.K / 2),
                            (uint64_t)(a.K / 2), TN, 128, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    p.scales = a.scales; p.y = a.y; p.bias = a.bias; p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.pitch_y();
    p.tiles_n = (int)ceil_div(a.N, TN); p.tiles_m = (int)ceil_div(a.M, TM); p.kblocks = (int)ceil_div(a.K, KB);
    p.status = kernel_status_word();
    if (!p.status) return ORTHO_B200_ERR_CUDA;
    p.gather = 0;
    if (a.gv && a.gv->world > 1) {
        p.gv = *a.gv;
        p.gather = 1;
        if (a.gather_fused) *a.gather_fused = true;
    }
    static bool attr_set[kMaxDevices] = {};       // the attribute is per device
    const int dev = current_device_index();
    if (dev < 0) return ORTHO_B200_ERR_CUDA;
    if (!attr_set[dev]) {
        OB_CUDA(cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev] = true;
    }
    const int num_sms = device_sm_count(dev);
    // split-K of the last partial wave: worth it when the leftover tiles occupy at most half of the SMs
    // and the caller's workspace has room for their partial sums behind the sparse pre-pass's part
    {
        const int T = p.tiles_n * p.tiles_m;
        const int G = T < num_sms ? T : num_sms;
        const int L = T % G == 0 ? (T < num_sms ? T : 0) : T % G;       // tiles of the last wave
        const int64_t off = a.has_ortho ? prefill_xt_bytes(a.M, a.K) + (p.n_long > 0 ? long_rows_workspace_bytes(a.plan, a.M) : 0) : 0;
        p.full_tiles = T; p.n_split = 0; p.kh = 0; p.part = nullptr; p.flags = nullptr;
        const int kh = (p.kblocks / 2 / WKB) * WKB;
        if (L > 0 && 2 * L <= num_sms && L <= kMaxSplit && kh >= WKB && a.workspace &&
            ((uintptr_t)a.workspace & 255u) == 0 && a.workspace_bytes >= off + (int64_t)kSplitBytes) {
            unsigned char *base = reinterpret_cast<unsigned char *>(a.workspace) + off;
            p.full_tiles = T - L; p.n_split = L; p.kh = kh;
            p.part = reinterpret_cast<float *>(base);
            p.flags = reinterpret_cast<int *>(base + kSplitPartBytes);
            OB_CUDA(cudaMemsetAsync(p.flags, 0, (size_t)L * sizeof(int), a.stream));
        }
    }
    const int nunits = p.full_tiles + 2 * p.n_split;
    const int grid = nunits < num_sms ? nunits : num_sms;
    if (p.n_long > 0) {
        // The pre-pass goes right in front of the main kernel, which is launched as its programmatic dependent: the
        // main kernel's CTAs move in as the pre-pass's CTAs leave, and only its epilogue warps wait for the sums.
        const int st2 = launch_long_rows(a, p.Mp, reinterpret_cast<unsigned char *>(a.workspace) + prefill_xt_bytes(a.M, a.K),
                                         &p.ol, &p.ol_splits);
        if (st2 != ORTHO_B200_OK) return st2;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(NWARPS * 32); cfg.dynamicSmemBytes = kSmemBytes;
        cfg.stream = a.stream; cfg.attrs = attr; cfg.numAttrs = 1;
        OB_CUDA(cudaLaunchKernelEx(&cfg, prefill_kernel, xmap, wmap, p));
    } else {
        prefill_kernel<<<grid, NWARPS * 32, kSmemBytes, a.stream>>>(xmap, wmap, p);
    }
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}

}  // namespace ob
