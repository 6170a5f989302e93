// Forward for a few tokens up to 128 on the 5th-generation tensor cores, with the operand roles of prefill.cu
// exchanged: the TOKENS are the M operand of the MMA (128 TMEM lanes, zero rows beyond the real token
// count) and the WEIGHT rows are its N operand (256 per instruction).
//
// Why: on this part one tcgen05.mma (kind::f16, K = 16) occupies the tensor pipe for about 185 cycles whatever
// its M and N are, so the weight bytes a kernel can push through the pipe depend only on how many weight rows
// one instruction covers: 128 as the M operand (prefill.cu: ~1.6 TB/s of packed INT4 per GPU), 256 as the N
// operand (here: ~3.2 TB/s), against ~2.3 / 1.2 TB/s for legacy mma.sync at 32 / 64 tokens.  Replaces, for
// this token range, the reference's one-thread-per-output kernel (src/dual_gemm.cu:176-225) and its WMMA
// variant (src/dual_gemm_tensor_core.cu:215-337).
//
//     D[m, n] = sum_k x[m, k] * w_int[n, k]        (tcgen05.mma, A and B from shared memory, FP32 in TMEM)
//     y[m, n] = scale[n] * D[m, n] + alpha * O[m, n] + bias[n]
//
// The packed INT4 bytes come in by TMA (256 rows x 128 B = 256 k per load, 128-byte swizzle); eight converter
// warps (one thread per weight row) unpack them to exact small-integer FP16 and write the K-major, 128-byte
// swizzled B tile (256 rows x 64 k) straight into shared memory; the token tile (128 x 64 k) is a plain TMA load.
// Two 256-column accumulators alternate, so the epilogue of one unit runs under the MMAs of the next.
// Epilogue thread = token (TMEM lane), columns = weight rows: every thread stores runs of 32 consecutive
// outputs of its own token row, no transposition.
//
// Work split (stream-K): the sequence of all (row tile, k block) pairs is cut into one contiguous share per
// CTA, so every SM does the same number of MMAs however few row tiles the layer has.  A CTA whose share starts
// inside a row tile leaves that tile's partial FP32 sums in its slot of the workspace and raises a flag; the CTA
// that holds the tile's first k block adds the partials of the CTAs behind it, in CTA order (fixed order:
// reproducible), in its epilogue.  A share's only partial piece is processed first and the piece that collects
// partials last, so the bounded flag wait does not normally wait at all.
//
// The sparse term.  With a plan whose rows are in column order and that lists no long rows, the converters fold it
// into the weight tile: each converter thread walks the entries of its row along K and adds v * alpha / scale[n] (FP16)
// to the weights it has just written to shared memory, so the MMAs compute base and sparse term together; a row
// whose corrections FP16 cannot hold (zero or tiny scale, huge values) is gathered from x by the epilogue thread of
// each token (rare).  Otherwise it is computed ahead into O[m][n] (token-major FP32, in the workspace) by
// ortho_tokens_kernel from the once-transposed activations (a warp per 8 weight rows, lanes = tokens) and added in
// the FP32 epilogue.
#include <cstring>

#include "common.cuh"
#include "gather.cuh"
#include "umma.cuh"

namespace ob {

int *kernel_status_word();
int launch_transpose_x(const __half *x, __half *xt, int M, int K, int Mp, cudaStream_t stream);   // transpose.cu

namespace md {
constexpr int TN = 256;                 // weight rows per tile (MMA N)
constexpr int TMK = 128;                // token lanes (MMA M)
constexpr int KB = 64;                  // k per pipeline stage
constexpr int WKB = 4;                  // k blocks covered by one packed-weight load
constexpr int W_BYTES = TN * 128;       // 32 KB
constexpr int X_BYTES = TMK * KB * 2;   // 16 KB: a full token stage (fewer tokens use smaller stages, see Params::xstage)
constexpr int B_BYTES = TN * KB * 2;    // 32 KB
constexpr int BST = 3;                  // converted-weight stages (the converters work one k block ahead of the MMAs)
constexpr int WST_MAX = 4, XST_MAX = 12;
// The packed weights come from HBM: at the rate the tensor pipe can consume them (8 KB per ~0.4 us and SM) and a
// loaded latency of 2-3 us, two 32 KB stages in flight per SM are the least that keeps the pipe fed, so the
// shared memory left by the two B stages goes to packed-weight stages first (Params::wst) and the token stages
// (which come from L2 and are small for few tokens) take the rest.
constexpr int kSmemData = 214 * 1024;   // packed-weight + token + converted-weight stages
constexpr int CONV_WARPS = 16;          // two threads per weight row: each converts 32 of the 64 k of a stage
constexpr int EPI_WARP0 = 2 + CONV_WARPS;
constexpr int EPI_WARPS = 4;
constexpr int NWARPS = EPI_WARP0 + EPI_WARPS;
constexpr int TMEM_COLS = 512;

struct Params {
    const __half *scales; const float *bias; __half *y;
    int M, K, N;
    long long ldy;
    int tiles_n, kblocks;
    long long total;            // tiles_n * kblocks
    int mrows;                  // token rows kept per partial slot (M rounded up to 32)
    int xbox_bytes;             // bytes one token-tile load delivers (token rows of the TMA box x 128)
    int xstage, xst;            // bytes between token stages (xbox_bytes rounded up to 1 KB) and how many there are
    int wst;                    // packed-weight stages
    float *slots; int *flags;   // slots[2 * cta + which][mrows][256] (which = 0: sums handed to another CTA, 1: this
                                // CTA's own sums of a tile it finishes), flags[cta]
    const float *o; float alpha; int has_ortho;    // O[m][n], row pitch N
    // patch != 0 (a plan with ordered rows and no long rows): the converters add the sparse entries to the weight tile
    // (v * alpha / scale[n], FP16) instead; rows that FP16 cannot hold are gathered from x by the epilogue
    int patch; OrthoView ov; const float *row_max; const __half *x;
    int *status;
    int gather;
    GatherView gv;
};

struct Smem {
    uint64_t w_full[WST_MAX], w_empty[WST_MAX];
    uint64_t x_full[XST_MAX], x_empty[XST_MAX];
    uint64_t b_full[BST], b_empty[BST];
    uint64_t d_full[2], d_empty[2];
    uint64_t fin_bar;           // bulk copies of partial-sum slots into shared memory (the collecting piece)
    uint32_t tmem_base;
    float sc[TN], bs[TN];
    alignas(16) unsigned char fb[TN];    // patch mode: 1 = this row of the tile is gathered by the epilogue
};
constexpr size_t kSmemBytes = 1024 + (size_t)kSmemData + sizeof(Smem) + 256;

struct Seg { int t, kb0, kb1; };
}  // namespace md

__global__ void __launch_bounds__(md::NWARPS * 32, 1)
mid_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const md::Params p)
{
    using namespace md;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *ws = base;
    unsigned char *xs = ws + (size_t)p.wst * W_BYTES;            // token stages; an MMA reads 128 token rows from a stage's
    unsigned char *bsm = base + (size_t)kSmemData - (size_t)BST * B_BYTES;   // base, i.e. on into what follows it
    Smem *sm = reinterpret_cast<Smem *>(base + (size_t)kSmemData);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const long long r_begin = p.total * cta / G, r_end = p.total * (cta + 1) / G;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WST_MAX; s++) { mbar_init(&sm->w_full[s], 1); mbar_init(&sm->w_empty[s], CONV_WARPS); }
        for (int s = 0; s < XST_MAX; s++) { mbar_init(&sm->x_full[s], 1); mbar_init(&sm->x_empty[s], 1); }
        for (int s = 0; s < BST; s++) { mbar_init(&sm->b_full[s], CONV_WARPS); mbar_init(&sm->b_empty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&sm->d_full[s], 1); mbar_init(&sm->d_empty[s], EPI_WARPS); }
        mbar_init(&sm->fin_bar, 1);
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
    // A converter warp waits with one polling lane (the warp shuffle hands the result and the ordering on to the
    // others) when it has nothing else in flight: 6-7 % faster than 512 threads polling one word.  With the sparse
    // entries folded in (their loads in flight across the wait) all lanes polling measured 5 % faster, so that form
    // keeps it.
    auto wait_warp = [&](uint64_t *bar, uint32_t parity) {
        if (p.patch) { wait(bar, parity); return; }
        if (lane == 0) wait(bar, parity);
        dead = __shfl_sync(0xffffffffu, (int)dead, 0) != 0;
    };
    // the pieces of this CTA's share, in order: (row tile, k blocks [kb0, kb1))
    auto next_seg = [&](long long &pos, Seg &sg) -> bool {
        if (pos >= r_end) return false;
        sg.t = (int)(pos / p.kblocks);
        sg.kb0 = (int)(pos - (long long)sg.t * p.kblocks);
        const long long left = r_end - pos;
        sg.kb1 = (int)((long long)(p.kblocks - sg.kb0) < left ? p.kblocks : sg.kb0 + left);
        pos += sg.kb1 - sg.kb0;
        return true;
    };

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            int xi = 0, wi = 0; uint32_t xph = 0, wph = 0;
            long long pos = r_begin; Seg sg;
            while (next_seg(pos, sg)) {
                for (int kb = sg.kb0; kb < sg.kb1; kb++) {
                    if ((kb % WKB) == 0 || kb == sg.kb0) {
                        wait(&sm->w_empty[wi], wph ^ 1u);
                        mbar_arrive_expect_tx(&sm->w_full[wi], W_BYTES);
                        tma_load_2d(ws + (size_t)wi * W_BYTES, &wmap, &sm->w_full[wi], (kb / WKB) * 128, sg.t * TN);
                        if (++wi == p.wst) { wi = 0; wph ^= 1u; }
                    }
                    wait(&sm->x_empty[xi], xph ^ 1u);
                    mbar_arrive_expect_tx(&sm->x_full[xi], (uint32_t)p.xbox_bytes);
                    tma_load_2d(xs + (size_t)xi * p.xstage, &xmap, &sm->x_full[xi], kb * KB, 0);
                    if (++xi == p.xst) { xi = 0; xph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(TMK, TN);
            const uint64_t adesc0 = umma_desc_sw128(smem_u32(xs));
            const uint64_t bdesc0 = umma_desc_sw128(smem_u32(bsm));
            int xi = 0, bi = 0; uint32_t xph = 0, bph = 0;
            long long pos = r_begin; Seg sg; int it = 0;
            while (next_seg(pos, sg)) {
                const int a = it & 1;
                wait(&sm->d_empty[a], (uint32_t)(((it >> 1) & 1) ^ 1));      // the epilogue has drained this accumulator
                tc_fence_after();
                const uint32_t d_tmem = tmem + (uint32_t)(a * TN);
                for (int kb = sg.kb0; kb < sg.kb1; kb++) {
                    wait(&sm->x_full[xi], xph);
                    wait(&sm->b_full[bi], bph);
                    tc_fence_after();
                    const uint64_t ad = adesc0 + (uint64_t)(xi * (p.xstage >> 4));
                    const uint64_t bd = bdesc0 + (uint64_t)(bi * (B_BYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < KB / 16; kk++)
                        umma_f16_ss(d_tmem, ad + (uint64_t)(2 * kk), bd + (uint64_t)(2 * kk), idesc, (kb != sg.kb0 || kk != 0) ? 1u : 0u);
                    umma_commit(&sm->x_empty[xi]);
                    umma_commit(&sm->b_empty[bi]);
                    if (++xi == p.xst) { xi = 0; xph ^= 1u; }
                    if (++bi == BST) { bi = 0; bph ^= 1u; }
                }
                umma_commit(&sm->d_full[a]);
                it++;
            }
        }
    } else if (warp < EPI_WARP0) {
        // ================= converters: packed INT4 (smem) -> FP16 B tile (smem, K-major, 128-byte swizzle) =================
        const int cw = warp - 2;
        const int row = (cw & 7) * 32 + lane;            // weight row inside the tile
        const int half = cw >> 3;                        // which 32 k of the stage's 64 this thread converts
        const uint32_t swz = (uint32_t)(row & 7);
        int wi = 0, bi = 0; uint32_t wph = 0, bph = 0;
        long long pos = r_begin; Seg sg;
        // Patch mode: this thread walks the sparse entries of its weight row in column order along the k blocks (both
        // threads of a row walk all of them, each applies those of its own 32 k), a window of four packed entries in
        // registers.  Only a share's first piece can start inside a row (kb0 > 0): one binary search per CTA, under
        // the ramp-up of the weight pipeline; the row's extent, scale and largest value for the next piece (the next
        // tile) are fetched a piece ahead.
        int nx_e0 = 0, nx_e1 = 0; float nx_sc = 0.f, nx_rm = 0.f;
        auto fetch_row = [&](int t) {
            nx_e0 = nx_e1 = 0; nx_sc = 0.f; nx_rm = 0.f;
            const int n = t * TN + row;
            if (t < p.tiles_n && n < p.N) {
                nx_e0 = p.ov.row_ptr[n]; nx_e1 = p.ov.row_ptr[n + 1];
                nx_sc = __half2float(p.scales[n]); nx_rm = p.row_max[n];
            }
        };
        if (p.patch && r_begin < r_end) fetch_row((int)(r_begin / p.kblocks));
        while (next_seg(pos, sg)) {
            int e_cur = 0, e_end = 0; float rsc = 0.f;
            uint32_t q0 = 0, q1 = 0, q2 = 0, q3 = 0;
            if (p.patch) {
                if (nx_e1 > nx_e0) {
                    rsc = patch_rscale(p.alpha, nx_sc, nx_rm);
                    if (rsc != 0.f) { e_cur = nx_e0; e_end = nx_e1; }
                }
                fetch_row(sg.t + 1);
                if (sg.kb0 > 0 && e_cur < e_end) {           // first entry at or past the piece's first column
                    int lo = e_cur, hi = e_end;
                    const uint32_t c0 = (uint32_t)(sg.kb0 * KB);
                    while (lo < hi) {
                        const int mid2 = (lo + hi) >> 1;
                        if ((p.ov.entries[mid2] & 0xFFFFu) < c0) lo = mid2 + 1; else hi = mid2;
                    }
                    e_cur = lo;
                }
                if (e_cur < e_end) q0 = p.ov.entries[e_cur];
                if (e_cur + 1 < e_end) q1 = p.ov.entries[e_cur + 1];
                if (e_cur + 2 < e_end) q2 = p.ov.entries[e_cur + 2];
                if (e_cur + 3 < e_end) q3 = p.ov.entries[e_cur + 3];
            }
            for (int kb = sg.kb0; kb < sg.kb1; kb++) {
                const int sub = kb % WKB;
                if (sub == 0 || kb == sg.kb0) wait_warp(&sm->w_full[wi], wph);
                const unsigned char *wrow = ws + (size_t)wi * W_BYTES + row * 128;
                const uint4 w0 = *reinterpret_cast<const uint4 *>(wrow + ((((uint32_t)(2 * sub + half)) ^ swz) << 4));
                if (sub == WKB - 1 || kb == sg.kb1 - 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->w_empty[wi]);
                    if (++wi == p.wst) { wi = 0; wph ^= 1u; }
                }
                const uint32_t ww[4] = {w0.x, w0.y, w0.z, w0.w};
                uint32_t o[4][4];
#pragma unroll
                for (int j = 0; j < 4; j++) int4x8_to_half2x4_natural(ww[j], o[j]);
                wait_warp(&sm->b_empty[bi], bph ^ 1u);
                unsigned char *brow = bsm + (size_t)bi * B_BYTES + row * 128;
#pragma unroll
                for (int j = 0; j < 4; j++)
                    *reinterpret_cast<uint4 *>(brow + ((((uint32_t)(4 * half + j)) ^ swz) << 4)) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
                if (p.patch) {
                    // entries of this row inside the k block: w_int + v * alpha / scale, as FP16, in the tile just written
                    const int kend = (kb + 1) * KB;
                    while (e_cur < e_end && (int)(q0 & 0xFFFFu) < kend) {
                        const uint32_t c = (q0 & 0xFFFFu) - (uint32_t)(kb * KB);
                        if ((int)(c >> 5) == half) {
                            __half *hp = reinterpret_cast<__half *>(brow + (((c >> 3) ^ swz) << 4)) + (c & 7u);
                            const float d = __half2float(__ushort_as_half((unsigned short)(q0 >> 16))) * rsc;
                            *hp = __hadd(*hp, __float2half_rn(d));
                        }
                        e_cur++;
                        q0 = q1; q1 = q2; q2 = q3;
                        q3 = (e_cur + 3 < e_end) ? p.ov.entries[e_cur + 3] : 0u;
                    }
                }
                fence_proxy_async();                     // the tensor core reads shared memory through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->b_full[bi]);
                if (++bi == BST) { bi = 0; bph ^= 1u; }
            }
        }
    } else {
        // ================= epilogue: TMEM -> (+ partials) -> scale, sparse term, bias -> FP16 -> global =================
        const int q = warp & 3;                          // TMEM lane quarter of this warp
        const int tok = q * 32 + lane;                   // token of this thread
        const int et = (warp - EPI_WARP0) * 32 + lane;   // 0..127 among the epilogue threads
        const bool warp_on = q * 32 < p.M;               // this warp's lanes hold real tokens
        const bool vec_ok = (p.ldy % 8) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0;
        const int nranks = p.gather ? p.gv.world : 1;
        // patch mode, a row the converters could not fold: its sparse sum for one token, straight from x
        auto gathered = [&](int n, int m) -> float {
            float acc = 0.f;
            const int e0 = p.ov.row_ptr[n], e1 = p.ov.row_ptr[n + 1];
            for (int e = e0; e < e1; e++) {
                int c; float v;
                ortho_entry(p.ov, e, p.K, c, v);
                acc = fmaf(v, __half2float(p.x[(size_t)m * p.K + c]), acc);
            }
            return acc;
        };
        long long pos = r_begin; Seg sg; int it = 0;
        while (next_seg(pos, sg)) {
            const int a = it & 1;
            const int n0 = sg.t * TN;
            const bool owner = sg.kb0 == 0;
            const bool whole = owner && sg.kb1 == p.kblocks;
            // contributors: the CTAs behind this one whose share starts inside the same row tile
            int c_first = cta + 1, c_last = cta;
            if (owner && !whole) {
                const long long tile_end = (long long)(sg.t + 1) * p.kblocks;
                while (c_last + 1 < G && p.total * (c_last + 1) / G < tile_end) c_last++;
            }
            if (owner) {
                for (int i = et; i < TN; i += EPI_WARPS * 32) {
                    const int n = n0 + i;
                    const float scn = n < p.N ? __half2float(p.scales[n]) : 0.f;
                    sm->sc[i] = scn;
                    sm->bs[i] = (p.bias && n < p.N) ? p.bias[n] : 0.f;
                    unsigned char f = 0;
                    if (p.patch && n < p.N && p.ov.row_ptr[n + 1] > p.ov.row_ptr[n] &&
                        patch_rscale(p.alpha, scn, p.row_max[n]) == 0.f)
                        f = 1;                       // the converters leave this row's entries alone: gathered below
                    sm->fb[i] = f;
                }
            }
            if (!dead) {                                 // a long wait (a whole piece of MMAs): poll with pauses
                bool ok = false;
                for (uint32_t i = 0; i < (1u << 22) && !ok; i++) {
                    ok = mbar_try_wait(&sm->d_full[a], (uint32_t)((it >> 1) & 1));
                    if (!ok) __nanosleep(256);
                }
                if (!ok) { dead = true; atomicExch(p.status, 1); }
            }
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * TN);
            if (!whole) {
                // a piece of a split tile: the raw FP32 sums go to this CTA's slot
                if (warp_on) {
                    float *dst = p.slots + ((size_t)(2 * cta + (owner ? 1 : 0)) * p.mrows + tok) * TN;
                    for (int c = 0; c < TN / 32; c++) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
                        tmem_ld_wait();
                        float4 *d4 = reinterpret_cast<float4 *>(dst + c * 32);
#pragma unroll
                        for (int j4 = 0; j4 < 8; j4++)
                            d4[j4] = make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]),
                                                 __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3]));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->d_empty[a]);          // the accumulator is free again
                __threadfence();
                if (owner && et == 0 && !dead) {                       // bounded wait for the contributors' flags
                    for (int c = c_first; c <= c_last; c++) {
                        int seen = 0;
                        for (unsigned spin = 0; spin < (1u << 22); spin++) {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.flags + c) : "memory");
                            if (seen) break;
                            __nanosleep(64);
                        }
                        if (!seen) { atomicExch(p.status, 1); break; }
                    }
                }
                named_bar_sync(1, EPI_WARPS * 32);       // own sums written, scales staged, flags seen
                if (!owner) {
                    if (et == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.flags + cta), "r"(1) : "memory");
                } else {
                    // the tile's pieces are added in CTA order (this CTA's first) by all epilogue threads: a unit is
                    // one token x 4 consecutive weight rows, consecutive threads take consecutive units
                    // The slots (this CTA's own first, then the contributors') are brought into shared memory 32 token
                    // rows at a time by bulk copies -- the pipeline stages are idle by now: the piece that collects
                    // partial sums is the last of a CTA's share -- and added from there.
                    const int ncon = c_last - c_first + 1;
                    constexpr int kFinRows = 32;
                    constexpr uint32_t kFinBytes = kFinRows * TN * 4;            // one slot, one group of rows: 32 KB
                    // (a tile cut into more pieces than fit takes several passes: the running sums stay in the first
                    // buffer, every pass brings the next contributors in beside it)
                    constexpr int kGroup = kSmemData / (int)kFinBytes - 1;       // contributors per pass
                    const bool staged = !dead;
                    float4 *fs4 = reinterpret_cast<float4 *>(base);
                    const size_t cstride = (size_t)2 * p.mrows * TN;
                    uint32_t fin_phase = 0;
                    for (int r0 = 0; r0 < p.mrows && r0 < p.M; r0 += kFinRows) {
                    const int rows_here = p.M - r0 < kFinRows ? p.M - r0 : kFinRows;
                    const int units = rows_here * (TN / 4);
                    int nb = ncon;                                               // contributors beside the running sums in this pass
                    if (staged) {
                        for (int done = 0;; done += nb) {
                            nb = ncon - done < kGroup ? ncon - done : kGroup;
                            if (et == 0) {
                                asm volatile("fence.proxy.async;" ::: "memory");   // the slots were written through the generic proxy
                                mbar_arrive_expect_tx(&sm->fin_bar, (uint32_t)((done == 0 ? 1 : 0) + nb) * kFinBytes);
                                if (done == 0)
                                    bulk_load_1d(base, p.slots + ((size_t)(2 * cta + 1) * p.mrows + r0) * TN, kFinBytes, &sm->fin_bar);
                                for (int s2 = 0; s2 < nb; s2++)
                                    bulk_load_1d(base + (size_t)(1 + s2) * kFinBytes,
                                                 p.slots + ((size_t)(2 * (c_first + done + s2)) * p.mrows + r0) * TN, kFinBytes, &sm->fin_bar);
                            }
                            wait(&sm->fin_bar, fin_phase & 1u);
                            fin_phase++;
                            if (done + nb >= ncon) break;                          // the last pass is finished off below
                            for (int u = et; u < units; u += EPI_WARPS * 32) {
                                float4 acc = fs4[u];
                                for (int s2 = 0; s2 < nb; s2++) {                  // added in CTA order
                                    const float4 t4 = fs4[(size_t)(1 + s2) * (kFinBytes / 16) + u];
                                    acc.x += t4.x; acc.y += t4.y; acc.z += t4.z; acc.w += t4.w;
                                }
                                fs4[u] = acc;
                            }
                            named_bar_sync(1, EPI_WARPS * 32);                     // before the next pass overwrites the contributors
                        }
                    }
                    for (int u = et; u < units; u += EPI_WARPS * 32) {
                        const int m = r0 + u / (TN / 4), c4 = (u % (TN / 4)) * 4;
                        const int n = n0 + c4;
                        if (n >= p.N) continue;
                        float4 acc;
                        if (staged) {
                            acc = fs4[u];
                            for (int s2 = 0; s2 < nb; s2++) {                    // added in CTA order
                                const float4 t4 = fs4[(size_t)(1 + s2) * (kFinBytes / 16) + u];
                                acc.x += t4.x; acc.y += t4.y; acc.z += t4.z; acc.w += t4.w;
                            }
                        } else {
                            const float *mine = p.slots + ((size_t)(2 * cta + 1) * p.mrows + m) * TN + c4;
                            const float *theirs = p.slots + ((size_t)(2 * cta) * p.mrows + m) * TN + c4;     // + (cc - cta) * cstride
                            acc = __ldcg(reinterpret_cast<const float4 *>(mine));
                            int cc = c_first;
                            for (; cc + 3 <= c_last; cc += 4) {            // four loads in flight, added in CTA order
                                float4 t4[4];
#pragma unroll
                                for (int i = 0; i < 4; i++) t4[i] = __ldcg(reinterpret_cast<const float4 *>(theirs + (size_t)(cc + i - cta) * cstride));
#pragma unroll
                                for (int i = 0; i < 4; i++) { acc.x += t4[i].x; acc.y += t4[i].y; acc.z += t4[i].z; acc.w += t4[i].w; }
                            }
                            for (; cc <= c_last; cc++) {
                                const float4 t4 = __ldcg(reinterpret_cast<const float4 *>(theirs + (size_t)(cc - cta) * cstride));
                                acc.x += t4.x; acc.y += t4.y; acc.z += t4.z; acc.w += t4.w;
                            }
                        }
                        float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) v[j] = fmaf(v[j], sm->sc[c4 + j], sm->bs[c4 + j]);
                        if (p.has_ortho) {
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                if (n + j < p.N) v[j] = fmaf(p.alpha, p.o[(size_t)m * p.N + n + j], v[j]);
                        }
                        if (p.patch && *reinterpret_cast<const uint32_t *>(&sm->fb[c4]) != 0u) {
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                if (sm->fb[c4 + j]) v[j] = fmaf(p.alpha, gathered(n + j, m), v[j]);
                        }
                        const __half2 h01 = __floats2half2_rn(v[0], v[1]), h23 = __floats2half2_rn(v[2], v[3]);
                        const size_t at = (size_t)m * (size_t)p.ldy + n;
                        for (int rk = 0; rk < nranks; rk++) {
                            __half *dst = (p.gather ? p.gv.y[rk] : p.y) + at;
                            if (vec_ok && n + 4 <= p.N) {
                                *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&h01),
                                                                             *reinterpret_cast<const uint32_t *>(&h23));
                            } else {
                                const __half hs[4] = {__low2half(h01), __high2half(h01), __low2half(h23), __high2half(h23)};
                                for (int j = 0; j < 4 && n + j < p.N; j++) dst[j] = hs[j];
                            }
                        }
                    }
                    if (staged) named_bar_sync(1, EPI_WARPS * 32);     // before the next rows overwrite the staging area
                    }
                }
                named_bar_sync(1, EPI_WARPS * 32);       // the staged scales are rewritten by the next piece
                it++;
                continue;
            }
            // the whole tile was accumulated here: straight from tensor memory to the output
            named_bar_sync(1, EPI_WARPS * 32);           // scales staged
            if (warp_on) {
                for (int c = 0; c < TN / 32; c++) {
                    const int nc = n0 + c * 32;
                    if (nc >= p.N) break;
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
                    tmem_ld_wait();
                    if (tok < p.M) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = fmaf(__uint_as_float(r[j]), sm->sc[c * 32 + j], sm->bs[c * 32 + j]);
                        const bool full = nc + 32 <= p.N;
                        if (p.has_ortho) {
                            const float *orow = p.o + (size_t)tok * p.N + nc;
                            if (full && (p.N % 4) == 0) {
#pragma unroll
                                for (int j4 = 0; j4 < 8; j4++) {
                                    const float4 o4 = *reinterpret_cast<const float4 *>(orow + 4 * j4);
                                    v[4 * j4] = fmaf(p.alpha, o4.x, v[4 * j4]); v[4 * j4 + 1] = fmaf(p.alpha, o4.y, v[4 * j4 + 1]);
                                    v[4 * j4 + 2] = fmaf(p.alpha, o4.z, v[4 * j4 + 2]); v[4 * j4 + 3] = fmaf(p.alpha, o4.w, v[4 * j4 + 3]);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (nc + j < p.N) v[j] = fmaf(p.alpha, orow[j], v[j]);
                            }
                        }
                        if (p.patch) {
                            const uint4 *fw = reinterpret_cast<const uint4 *>(&sm->fb[c * 32]);
                            const uint4 f0 = fw[0], f1 = fw[1];
                            if ((f0.x | f0.y | f0.z | f0.w | f1.x | f1.y | f1.z | f1.w) != 0u) {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (sm->fb[c * 32 + j]) v[j] = fmaf(p.alpha, gathered(nc + j, tok), v[j]);
                            }
                        }
                        uint32_t h[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const __half2 hh = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                            h[j] = *reinterpret_cast<const uint32_t *>(&hh);
                        }
                        const size_t at = (size_t)tok * (size_t)p.ldy + nc;
                        for (int rk = 0; rk < nranks; rk++) {
                            __half *dst = (p.gather ? p.gv.y[rk] : p.y) + at;
                            if (vec_ok && full && (nc % 8) == 0) {
#pragma unroll
                                for (int j4 = 0; j4 < 4; j4++)
                                    reinterpret_cast<uint4 *>(dst)[j4] = make_uint4(h[4 * j4], h[4 * j4 + 1], h[4 * j4 + 2], h[4 * j4 + 3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; j++) {
                                    const __half2 hh = *reinterpret_cast<const __half2 *>(&h[j]);
                                    if (nc + 2 * j < p.N) dst[2 * j] = __low2half(hh);
                                    if (nc + 2 * j + 1 < p.N) dst[2 * j + 1] = __high2half(hh);
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->d_empty[a]);
            named_bar_sync(1, EPI_WARPS * 32);           // the staged scales are rewritten by the next piece
            it++;
        }
    }

    if (p.gather) {
        if (!gather_signal_and_wait(p.gv, gridDim.x)) atomicExch(p.status, 2);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// O[m][n] = sum over the entries of row n of v * x[m, c]   (FP32, token-major with row pitch N; alpha is applied
// in the epilogue).  A warp takes 8 consecutive weight rows; a lane holds TPL consecutive tokens (Mp = 32 * TPL) and
// reads them from the transposed activations Xt[k][Mp] with one load per entry, up to 32 / TPL entries in flight;
// entries are fetched 32 at a time with one coalesced load and broadcast by shuffles.
template <int TPL>
__global__ void __launch_bounds__(256)
ortho_tokens_kernel(const OrthoView ov, const __half *__restrict__ xt, float *__restrict__ o, int M, int K, int N)
{
    constexpr int Mp = 32 * TPL;
    constexpr int U = 32 / TPL;                          // activation loads in flight per lane
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_first = (blockIdx.x * 8 + warp) * 8;     // a warp takes 8 consecutive weight rows, one after the other
    if (n_first >= N) return;
    float res[8][TPL];
#pragma unroll
    for (int r = 0; r < 8; r++) {
#pragma unroll
        for (int i = 0; i < TPL; i++) res[r][i] = 0.f;
        const int n = n_first + r;
        if (n >= N) continue;
        const int e0 = ov.row_ptr[n], e1 = ov.row_ptr[n + 1];
        float acc[TPL];
#pragma unroll
        for (int i = 0; i < TPL; i++) acc[i] = 0.f;
        for (int eb = e0; eb < e1; eb += 32) {
            int cl = 0; float vl = 0.f;
            if (eb + lane < e1) ortho_entry(ov, eb + lane, K, cl, vl);
            const int nb = min(32, e1 - eb);
            for (int j0 = 0; j0 < nb; j0 += U) {
                float vv[U];
                if constexpr (TPL == 1) {
                    __half h[U];
#pragma unroll
                    for (int j = 0; j < U; j++) {
                        const int c = __shfl_sync(0xffffffffu, cl, (j0 + j) & 31);
                        vv[j] = __shfl_sync(0xffffffffu, vl, (j0 + j) & 31);      // slots past the row hold v = 0, c = 0
                        h[j] = xt[(size_t)c * Mp + lane];
                    }
#pragma unroll
                    for (int j = 0; j < U; j++) acc[0] = fmaf(vv[j], __half2float(h[j]), acc[0]);
                } else if constexpr (TPL == 2) {
                    __half2 h[U];
#pragma unroll
                    for (int j = 0; j < U; j++) {
                        const int c = __shfl_sync(0xffffffffu, cl, (j0 + j) & 31);
                        vv[j] = __shfl_sync(0xffffffffu, vl, (j0 + j) & 31);
                        h[j] = *reinterpret_cast<const __half2 *>(xt + (size_t)c * Mp + lane * 2);
                    }
#pragma unroll
                    for (int j = 0; j < U; j++) {
                        const float2 f = __half22float2(h[j]);
                        acc[0] = fmaf(vv[j], f.x, acc[0]); acc[1] = fmaf(vv[j], f.y, acc[1]);
                    }
                } else {
                    uint2 u[U];
#pragma unroll
                    for (int j = 0; j < U; j++) {
                        const int c = __shfl_sync(0xffffffffu, cl, (j0 + j) & 31);
                        vv[j] = __shfl_sync(0xffffffffu, vl, (j0 + j) & 31);
                        u[j] = *reinterpret_cast<const uint2 *>(xt + (size_t)c * Mp + lane * 4);
                    }
#pragma unroll
                    for (int j = 0; j < U; j++) {
                        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&u[j].x));
                        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&u[j].y));
                        acc[0] = fmaf(vv[j], f0.x, acc[0]); acc[1] = fmaf(vv[j], f0.y, acc[1]);
                        acc[2] = fmaf(vv[j], f1.x, acc[2]); acc[3] = fmaf(vv[j], f1.y, acc[3]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < TPL; i++) res[r][i] = acc[i];
    }
    // a lane writes the 8 rows' sums of each of its tokens as one 32-byte run
    const bool vec = (N % 4) == 0 && n_first + 8 <= N;
#pragma unroll
    for (int i = 0; i < TPL; i++) {
        const int m = lane * TPL + i;
        if (m >= M) continue;
        float *dst = o + (size_t)m * N + n_first;
        if (vec) {
            reinterpret_cast<float4 *>(dst)[0] = make_float4(res[0][i], res[1][i], res[2][i], res[3][i]);
            reinterpret_cast<float4 *>(dst)[1] = make_float4(res[4][i], res[5][i], res[6][i], res[7][i]);
        } else {
#pragma unroll
            for (int r = 0; r < 8; r++)
                if (n_first + r < N) dst[r] = res[r][i];
        }
    }
}

// workspace: [ Xt : K * Mp halves ][ O : M * N floats ][ partial slots : SMs * mrows * 256 floats ][ flags ]
constexpr int kMidMaxSms = 148;         // the partial-sum slots are sized for this many CTAs; the grid never exceeds it
static int64_t mid_mp(int64_t M) { return M <= 32 ? 32 : M <= 64 ? 64 : 128; }
static int64_t mid_xt_bytes(int64_t M, int64_t K) { return ((K * mid_mp(M) * 2 + 255) / 256) * 256; }
static int64_t mid_o_bytes(int64_t M, int64_t N) { return ((M * N * 4 + 255) / 256) * 256; }
static int64_t mid_slot_bytes(int64_t M, int sms) { return (int64_t)2 * sms * ((M + 31) / 32 * 32) * md::TN * 4; }
int64_t mid_workspace_bytes(int64_t M, int64_t K, int64_t N)
{
    return mid_xt_bytes(M, K) + mid_o_bytes(M, N) + mid_slot_bytes(M, kMidMaxSms) + 1024;
}

int launch_mid(const FwdArgs &a)
{
    using namespace md;
    if (a.M > TMK || a.M < 1) return ORTHO_B200_ERR_SHAPE;
    if (!a.workspace || a.workspace_bytes < mid_workspace_bytes(a.M, a.K, a.N)) return ORTHO_B200_ERR_WORKSPACE;
    if (((uintptr_t)a.workspace & 255u) != 0) return ORTHO_B200_ERR_ALIGN;
    const int dev = current_device_index();
    if (dev < 0) return ORTHO_B200_ERR_CUDA;
    const int num_sms = device_sm_count(dev);
    unsigned char *wsb = reinterpret_cast<unsigned char *>(a.workspace);
    __half *xt = reinterpret_cast<__half *>(wsb);
    float *o = reinterpret_cast<float *>(wsb + mid_xt_bytes(a.M, a.K));
    float *slots = reinterpret_cast<float *>(wsb + mid_xt_bytes(a.M, a.K) + mid_o_bytes(a.M, a.N));
    int *flags = reinterpret_cast<int *>(wsb + mid_xt_bytes(a.M, a.K) + mid_o_bytes(a.M, a.N) + mid_slot_bytes(a.M, kMidMaxSms));

    Params p;
    memset(&p, 0, sizeof(p));
    p.scales = a.scales; p.bias = a.bias; p.y = a.y; p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.pitch_y();
    p.tiles_n = (int)ceil_div(a.N, TN); p.kblocks = (int)ceil_div(a.K, KB);
    p.total = (long long)p.tiles_n * p.kblocks;
    p.mrows = (int)((a.M + 31) / 32 * 32);
    // Only the token rows that exist are fetched (rounded up to the 8-row period of the swizzle).  The MMA still
    // reads 128 rows of the stage: what the rows beyond the box hold only reaches accumulator rows nobody reads.
    const int xbox_rows = (int)((a.M + 7) / 8 * 8);
    p.xbox_bytes = xbox_rows * 128;
    p.xstage = (p.xbox_bytes + 1023) / 1024 * 1024;
    {
        const int room = kSmemData - BST * B_BYTES;           // for packed-weight and token stages
        p.wst = WST_MAX;
        while (p.wst > 2 && (room - p.wst * W_BYTES) / p.xstage < 3) p.wst--;
        const int xroom = room - p.wst * W_BYTES;
        p.xst = xroom / p.xstage < XST_MAX ? xroom / p.xstage : XST_MAX;
    }
    p.slots = slots; p.flags = flags;
    p.alpha = a.alpha; p.has_ortho = 0; p.o = nullptr;
    p.status = kernel_status_word();
    if (!p.status) return ORTHO_B200_ERR_CUDA;
    if (a.has_ortho && a.plan && a.ortho.entries && a.plan->ordered && a.plan->row_max && a.plan->n_long == 0 &&
        tuning_snapshot().patch_weights) {
        // the sparse entries are folded into the weight tile by the converters: no transposed activations, no O
        p.patch = 1; p.ov = a.ortho; p.row_max = a.plan->row_max; p.x = a.x;
    } else if (a.has_ortho) {
        const int Mp = (int)mid_mp(a.M);
        int st = launch_transpose_x(a.x, xt, (int)a.M, (int)a.K, Mp, a.stream);
        if (st != ORTHO_B200_OK) return st;
        const unsigned blocks = (unsigned)ceil_div(a.N, 64);
        if (Mp == 32) ortho_tokens_kernel<1><<<blocks, 256, 0, a.stream>>>(a.ortho, xt, o, (int)a.M, (int)a.K, (int)a.N);
        else if (Mp == 64) ortho_tokens_kernel<2><<<blocks, 256, 0, a.stream>>>(a.ortho, xt, o, (int)a.M, (int)a.K, (int)a.N);
        else ortho_tokens_kernel<4><<<blocks, 256, 0, a.stream>>>(a.ortho, xt, o, (int)a.M, (int)a.K, (int)a.N);
        count_launch();
        OB_CUDA(cudaGetLastError());
        p.o = o; p.has_ortho = 1;
    }
    CUtensorMap xmap, wmap;
    if (!make_tensor_map_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                            (uint64_t)a.K * 2, (uint32_t)xbox_rows, KB, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    if (!make_tensor_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)a.N, (uint64_t)(a.K / 2),
                            (uint64_t)(a.K / 2), TN, 128, CU_TENSOR_MAP_SWIZZLE_128B))
        return ORTHO_B200_ERR_CUDA;
    p.gather = 0;
    if (a.gv && a.gv->world > 1) {
        p.gv = *a.gv;
        p.gather = 1;
        if (a.gather_fused) *a.gather_fused = true;
    }
    static bool attr_set[kMaxDevices] = {};
    if (!attr_set[dev]) {
        OB_CUDA(cudaFuncSetAttribute(mid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev] = true;
    }
    // every CTA gets at least kMinShare k blocks: a narrow layer cut into shares of a few k blocks would spend its time
    // adding dozens of partial tiles
    constexpr long long kMinShare = 16;
    long long grid = (p.total + kMinShare - 1) / kMinShare;
    if (grid > num_sms) grid = num_sms;
    if (grid > kMidMaxSms) grid = kMidMaxSms;
    if (grid < 1) grid = 1;
    OB_CUDA(cudaMemsetAsync(flags, 0, (size_t)grid * sizeof(int), a.stream));
    mid_kernel<<<(unsigned)grid, NWARPS * 32, kSmemBytes, a.stream>>>(xmap, wmap, p);
    count_launch();
    OB_CUDA(cudaGetLastError());
    return ORTHO_B200_OK;
}

}  // namespace ob
