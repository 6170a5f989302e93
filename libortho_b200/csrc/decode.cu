// Decode-regime (small M) OrthoLinear forward for sm_100a: a memory-bound streaming kernel.
//
// Replaces dual_gemm_kernel_csr and its helpers (src/dual_gemm.cu:30-40,55-92,106-130,176-225 of
// the reference), where one thread walks a whole weight row byte by byte.  Here the packed INT4
// base is streamed exactly once with 128-bit coalesced loads that are all put in flight before
// any arithmetic, unpacked in registers, and contracted on the tensor pipe with the weight tile
// as the 16-row operand and the token block as the 8-column operand (FP32 accumulate).  The
// per-row scale has no zero point and no groups (src/ortho.c:356,363), so it factors out of the
// K sum and is applied once in the FP32 epilogue:
//     y[m,n] = scale[n] * sum_k x[m,k] * w_int[n,k]  +  alpha * sum_i v_i * x[m, c_i].
// The alpha-scaled sparse term is computed by the same CTAs, one warp per output row with
// shuffle reductions, from the plan's packed {col16|f16} entries (or raw CSR when no plan is
// given), while the base loads are in flight.  alpha <= 0 or nnz == 0 skips that stream entirely.
//
// Work decomposition: grid.y = tiles of R = 16*WR output rows; the K range is split over the
// S CTAs of a thread-block cluster (grid.x) and again over the WK k-groups of warps inside a
// CTA.  Partial sums meet in shared memory inside a CTA and through distributed shared memory
// across the cluster, so there is no global scratch and the result is deterministic.
#include <cooperative_groups.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ob {

struct DecodeParams {
    const uint8_t *w; const __half *scales; const __half *x; __half *y;
    const float *bias;   // optional FP32 [N]
    OrthoView ov; int has_ortho; float alpha;
    int M, K, N;
    long long ldy;    // elements between token rows of y
    int T;            // ceil(K / 128): k steps of 128 elements (64 packed bytes per row)
    int pass_steps;   // k steps staged in shared memory per pass
    int pitch;        // bytes between token rows of the staged X slab (== pass_steps*256 + 64)
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

template <int MT, int WR, int WK, int U>
__global__ void __launch_bounds__(WR * WK * 32)
decode_kernel(const DecodeParams p)
{
    constexpr int R = 16 * WR;       // output rows per CTA
    constexpr int TOK = 8 * MT;      // token slots (multiple of the mma n=8)
    constexpr int NW = WR * WK;
    constexpr int NT = NW * 32;

    extern __shared__ __align__(128) unsigned char smem[];
    // [ X slab: M rows * pitch ][ red: WK * R * TOK floats ][ O: R * TOK floats ]
    unsigned char *xs = smem;
    float *red = reinterpret_cast<float *>(smem + (size_t)p.M * p.pitch);
    float *osm = red + WK * R * TOK;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wr = warp / WK, wk = warp % WK;
    const int g = lane >> 2, t = lane & 3;

    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();

    const int row_tile0 = blockIdx.y * R;
    const int cs0 = (int)(((long long)p.T * rank) / S);
    const int cs1 = (int)(((long long)p.T * (rank + 1)) / S);

    const int K = p.K, N = p.N, M = p.M;
    const size_t row_bytes = (size_t)K >> 1;
    const int row0 = row_tile0 + 16 * wr + g, row1 = row0 + 8;
    const unsigned char *wp0 = p.w + (size_t)row0 * row_bytes + t * 16;
    const unsigned char *wp1 = p.w + (size_t)row1 * row_bytes + t * 16;
    const bool r0ok = row0 < N, r1ok = row1 < N;

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

    uint4 wa[U], wb[U];
    auto load_batch = [&](int s, int s_end) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int ss = s + u;
            const bool in = (ss < s_end) && (ss * 128 + t * 32 < K);
            wa[u] = (in && r0ok) ? ldg_stream(wp0 + (size_t)ss * 64) : make_uint4(0, 0, 0, 0);
            wb[u] = (in && r1ok) ? ldg_stream(wp1 + (size_t)ss * 64) : make_uint4(0, 0, 0, 0);
        }
    };

    // sparse ortho term: warp per output row, lanes stride over the row's entries, shuffle
    // reduction per token.  Runs once per CTA, while the first base loads are in flight.
    auto ortho_rows = [&]() {
        const int RB = R / S;                // rows of this tile owned by this CTA
        for (int ii = warp; ii < RB; ii += NW) {
            const int i = rank * RB + ii;
            const int n = row_tile0 + i;
            int e0 = 0, e1 = 0;
            if (n < N) { e0 = p.ov.row_ptr[n]; e1 = p.ov.row_ptr[n + 1]; }
#pragma unroll 1
            for (int tc = 0; tc < MT; tc++) {
                if (tc * 8 >= M) break;
                float a8[8];
#pragma unroll
                for (int jj = 0; jj < 8; jj++) a8[jj] = 0.f;
                for (int e = e0 + lane; e < e1; e += 32) {
                    int c; float v;
                    if (p.ov.entries) {
                        const uint32_t pk = p.ov.entries[e];
                        c = (int)(pk & 0xFFFFu);
                        v = __half2float(__ushort_as_half((unsigned short)(pk >> 16)));
                    } else {
                        c = p.ov.col[e];
                        v = __half2float(p.ov.val[e]);
                        if ((unsigned)c >= (unsigned)K) { c = 0; v = 0.f; }
                    }
#pragma unroll
                    for (int jj = 0; jj < 8; jj++) {
                        const int m = tc * 8 + jj;
                        if (m < M) a8[jj] = fmaf(v, __half2float(p.x[(size_t)m * K + c]), a8[jj]);
                    }
                }
#pragma unroll
                for (int jj = 0; jj < 8; jj++) {
                    float s = a8[jj];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                    if (lane == 0) osm[i * TOK + tc * 8 + jj] = s;
                }
            }
        }
    };

    for (int pass0 = cs0; pass0 < cs1; pass0 += p.pass_steps) {
        const int pass1 = min(pass0 + p.pass_steps, cs1);
        const int np = pass1 - pass0;
        const int ws0 = pass0 + (np * wk) / WK;
        const int ws1 = pass0 + (np * (wk + 1)) / WK;

        // put the first batch of weight loads in flight before anything else
        load_batch(ws0, ws1);

        if (pass0 != cs0) __syncthreads();   // everyone finished reading the previous slab

        // stage X[:, pass k-range] into shared memory in the pair order the unpack produces:
        // each 16-byte chunk (x0..x7) is stored as (x0,x4,x1,x5,x2,x6,x3,x7); inside a k step the
        // 16 chunks are laid out [j][t] so that the 4 lanes sharing a row read 64 contiguous bytes.
        {
            const int chunks_per_row = np * 16;
            const int total = M * chunks_per_row;
            for (int idx = tid; idx < total; idx += NT) {
                const int r = idx / chunks_per_row, q = idx - r * chunks_per_row;
                const int k = pass0 * 128 + q * 8;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (k < K) v = *reinterpret_cast<const uint4 *>(p.x + (size_t)r * K + k);
                uint4 o;
                o.x = prmt(v.x, v.z, 0x5410);   // (x0,x4)
                o.y = prmt(v.x, v.z, 0x7632);   // (x1,x5)
                o.z = prmt(v.y, v.w, 0x5410);   // (x2,x6)
                o.w = prmt(v.y, v.w, 0x7632);   // (x3,x7)
                const int sl = q >> 4, c16 = q & 15, tt = c16 >> 2, j = c16 & 3;
                *reinterpret_cast<uint4 *>(xs + (size_t)r * p.pitch + sl * 256 + j * 64 + tt * 16) = o;
            }
        }

        if (pass0 == cs0 && p.has_ortho) ortho_rows();

        __syncthreads();   // X slab staged

        for (int s = ws0; s < ws1; s += U) {
            uint4 ca[U], cb[U];
#pragma unroll
            for (int u = 0; u < U; u++) { ca[u] = wa[u]; cb[u] = wb[u]; }
            if (s + U < ws1) load_batch(s + U, ws1);   // next batch in flight during the math
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (s + u < ws1) {
                    const int sl = s + u - pass0;
                    const uint32_t wwa[4] = {ca[u].x, ca[u].y, ca[u].z, ca[u].w};
                    const uint32_t wwb[4] = {cb[u].x, cb[u].y, cb[u].z, cb[u].w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint32_t ha[4], hb[4];
                        int4x8_to_half2x4(wwa[j], ha);
                        int4x8_to_half2x4(wwb[j], hb);
                        const uint32_t A0[4] = {ha[0], hb[0], ha[1], hb[1]};
                        const uint32_t A1[4] = {ha[2], hb[2], ha[3], hb[3]};
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            const int tok = 8 * mt + g;
                            uint4 xb = make_uint4(0, 0, 0, 0);
                            if (tok < M)
                                xb = *reinterpret_cast<const uint4 *>(
                                    xs + (size_t)tok * p.pitch + sl * 256 + j * 64 + t * 16);
                            mma_16816(acc[mt], A0, xb.x, xb.y);
                            mma_16816(acc[mt], A1, xb.z, xb.w);
                        }
                    }
                }
            }
        }
    }

    if (cs0 >= cs1 && p.has_ortho) ortho_rows();   // a CTA without k steps still owns ortho rows

    // ---- reduce the WK k-groups of this CTA in shared memory -------------------------------
    {
        float *mine = red + (size_t)wk * R * TOK;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int col = 8 * mt + 2 * t;
            *reinterpret_cast<float2 *>(mine + (16 * wr + g) * TOK + col) = make_float2(acc[mt][0], acc[mt][1]);
            *reinterpret_cast<float2 *>(mine + (16 * wr + g + 8) * TOK + col) = make_float2(acc[mt][2], acc[mt][3]);
        }
    }
    __syncthreads();
    if (WK > 1) {
        for (int idx = tid; idx < R * TOK; idx += NT) {
            float s = red[idx];
#pragma unroll
            for (int k2 = 1; k2 < WK; k2++) s += red[(size_t)k2 * R * TOK + idx];
            red[idx] = s;
        }
    }
    if (S > 1) cluster.sync(); else __syncthreads();

    // ---- finalize the rows this CTA owns: sum cluster partials, scale, add ortho, store f16 ----
    {
        const int RB = R / S;
        const int total = RB * M;
        for (int idx = tid; idx < total; idx += NT) {
            const int m = idx / RB, ii = idx - m * RB;
            const int i = rank * RB + ii;
            const int n = row_tile0 + i;
            if (n < N) {
                float s = 0.f;
                if (S > 1) {
                    for (int r2 = 0; r2 < S; r2++) {
                        const float *peer = cluster.map_shared_rank(red, r2);
                        s += peer[i * TOK + m];
                    }
                } else {
                    s = red[i * TOK + m];
                }
                float v = __half2float(p.scales[n]) * s;
                if (p.has_ortho) v = fmaf(p.alpha, osm[i * TOK + m], v);
                if (p.bias) v += p.bias[n];
                p.y[(size_t)m * (size_t)p.ldy + n] = __float2half_rn(v);
            }
        }
    }
    if (S > 1) cluster.sync();   // keep shared memory alive until every peer has read it
}

// ---- host side ------------------------------------------------------------------------------

struct DecodeCfg { int wr, wk, u, s; };

// Tuning hook state.  prefill_above: forwards with more tokens go to the tcgen05 kernels.  Measured on
// 8192->8192 / 8192->57344 / 28672->8192: at 32 tokens the 128 x 256 tensor-core tile (mostly padding) takes
// 97 / 370 / 300 us where the mma.sync kernel below takes 146 / 972 / 479 us; at 17 tokens the two are within a
// few per cent.
static std::mutex g_tune_mu;
static Tuning g_tune;
Tuning tuning_snapshot()
{
    std::lock_guard<std::mutex> lock(g_tune_mu);
    return g_tune;
}

// Which regime a forward runs in.  Above the token threshold the tensor-core kernel wins unless the layer (or
// the shard of it that this GPU holds) has so few 128-row tiles that most SMs would idle for a whole K sweep:
// measured at K = 8192, M = 32: N = 1024 / 2048 / 4096 take 24 / 27 / 51 us here against 96 / 96 / 93 us there
// (141 against 95 us at N = 7168); M = 64: 63 against 98 us at N = 1024, 117 against 96 us at N = 2048.  With a
// long K the balance tips back (K = 28672, N = 4096, M = 32: 272 against 216 us), hence the bound on N * K.
// The narrow-layer exception only applies to the built-in threshold, so that the tuning hook can still force
// either kernel.
static bool decode_regime_of(const Tuning &t, int64_t M, int64_t N, int64_t K)
{
    if (M <= t.prefill_above) return true;
    if (t.prefill_above != kPrefillAboveBuiltin || M > ORTHO_B200_DECODE_MAX_M) return false;
    if (N * K > (int64_t)4096 * 8192) return false;
    return (M <= 32 && N <= 4096) || N <= 1024;
}
bool decode_regime(int64_t M, int64_t N, int64_t K) { return decode_regime_of(tuning_snapshot(), M, N, K); }
bool mid_token_range(int64_t M)
{
    const Tuning t = tuning_snapshot();
    return M > t.mid_lo && M <= t.mid_hi && M <= 128;
}
// Measured on one B200 (us, 0.3 % ortho, alpha = 1, folded sparse term): 32 tokens on 8192->8192 / 8192->10240 /
// 8192->57344 / 28672->8192 take 49 / 54 / 183 / 107 with the tokens-as-M kernel against 95 / 108 / 370 / 218 with the
// 128 x 256-token tile of prefill.cu; at 16 tokens the streaming kernel is level on the largest layer (205) and ahead
// on K = 4096 layers (33 against 68 on 4096->22016).  From 17 tokens on the mma.sync kernel of this file falls behind
// quickly (20 / 24 tokens: 8192->10240 113 / 147 against 51 / 52, 8192->57344 497 / 797 against 182, 11008->4096 50 / 54
// against 43 / 44), hence the built-in range (16, 128].
// Narrow layers (a GPU's shard of a layer, say), tokens-as-M kernel against the mma.sync kernel of this file:
//   32 tokens: 8192->1024 39 / 25, 8192->1280 39 / 25, 4096->2048 34 / 17, 4096->4096 35 / 33, 11008->512 41 / 25, but
//              8192->2560 40 / 48, 8192->4096 42 / 52, 28672->1024 66 / 107, 28672->2048 64 / 86;
//   64 tokens: 8192->1024 53 / 63, 8192->1280 53 / 166, 8192->2560 54 / 109, 4096->4096 45 / 80, 4096->2048 44 / 117,
//              28672->1024 98 / 175 (only 4096->1024 loses: 43 / 38).
//   17 .. 24 tokens on layers of at most 4096 x 4096 weights: the mma.sync kernel stays ahead (4096->4096 25-27 against
//              31-33, 8192->2048 19-21 against 35-37, 4096->1024 13-14 against 31).
// So with its workspace the tokens-as-M kernel takes everything above 16 tokens except up to 32 tokens on layers of at
// most 4096 x 4096 weights; without the workspace the older rule between the mma.sync kernel and the prefill tile
// (decode_regime_of) stands.
Route route_of(int64_t M, int64_t N, int64_t K, const void *workspace, int64_t workspace_bytes)
{
    const Tuning t = tuning_snapshot();
    const bool mid_ok = M > t.mid_lo && M <= t.mid_hi && M <= 128 && workspace && ((uintptr_t)workspace & 255u) == 0 &&
                        workspace_bytes >= mid_workspace_bytes(M, K, N);
    if (mid_ok && t.mid_first) return kRouteMid;
    if (mid_ok) {
        if (t.prefill_above == kPrefillAboveBuiltin && M <= 32 && N * K <= (int64_t)4096 * 4096) return kRouteDecode;
        return kRouteMid;
    }
    if (decode_regime_of(t, M, N, K)) return kRouteDecode;
    return kRoutePrefill;
}

int launch_decode_stream(const FwdArgs &a, int S, int stages);          // decode_stream.cu
int launch_decode_stream_multi(const FwdArgs *layers, int nl, int S, int stages);

int set_decode_config(int wr, int wk, int u, int s)
{
    std::lock_guard<std::mutex> lock(g_tune_mu);
    Tuning &t = g_tune;
    if (wr == -3) {       // forwards with more than s tokens (0 <= s <= 64) go to the tensor-core prefill kernel
        if (s < 0 || s > ORTHO_B200_DECODE_MAX_M) return ORTHO_B200_ERR_SHAPE;
        t.prefill_above = s;
        return ORTHO_B200_OK;
    }
    if (wr == -4) {       // forwards with u < tokens <= s (s <= 128) use the tokens-as-M tensor-core kernel whatever the
                          // other rules say (u == s: never); u == s == 0 restores the built-in rule
        if (u < 0 || s < 0 || s > 128 || u > s) return ORTHO_B200_ERR_SHAPE;
        if (u == 0 && s == 0) { t.mid_lo = 16; t.mid_hi = 128; t.mid_first = false; }
        else { t.mid_lo = u; t.mid_hi = s; t.mid_first = true; }
        return ORTHO_B200_OK;
    }
    if (wr == -7) {       // s = 1: per-CTA signalling in the peer exchange (every rank of a group must use the same setting)
        if (s != 0 && s != 1) return ORTHO_B200_ERR_SHAPE;
        t.gather_per_cta = s == 1;
        return ORTHO_B200_OK;
    }
    if (wr == -6) {       // s = 0: the tensor-core kernels compute the sparse term as gathers even with an ordered plan
        if (s != 0 && s != 1) return ORTHO_B200_ERR_SHAPE;
        t.patch_weights = s == 1;
        return ORTHO_B200_OK;
    }
    if (wr == -5) {       // plans created from now on treat rows of more than max(s, 4 x the mean row) entries as long
        if (s != 0 && (s < 8 || s > 65536)) return ORTHO_B200_ERR_SHAPE;
        t.long_row_min = s ? s : kLongRowMin;
        return ORTHO_B200_OK;
    }
    if (wr == -1) {
        if ((s != 0 && s != 1 && s != 2 && s != 4 && s != 8) || u < 0 || u > 12 || u == 1) return ORTHO_B200_ERR_SHAPE;
        t.wr = t.wk = t.u = t.s = 0;
        t.force_stream = true;
        t.stream_s = s; t.stream_stages = u;
        return ORTHO_B200_OK;
    }
    if (wr < 0) return ORTHO_B200_ERR_SHAPE;
    t.force_stream = false;
    t.stream_s = t.stream_stages = 0;
    if (wr <= 0 || wk <= 0 || u <= 0 || s <= 0) { t.wr = t.wk = t.u = t.s = 0; return ORTHO_B200_OK; }
    const bool shape_ok = (wr == 1 && wk == 8) || (wr == 2 && wk == 4) || (wr == 4 && wk == 2) ||
                          (wr == 8 && wk == 1) || (wr == 1 && wk == 4) || (wr == 2 && wk == 2);
    if (!shape_ok || (u != 2 && u != 4) || (s != 1 && s != 2 && s != 4 && s != 8))
        return ORTHO_B200_ERR_SHAPE;
    t.wr = wr; t.wk = wk; t.u = u; t.s = s;
    return ORTHO_B200_OK;
}

static DecodeCfg choose(const Tuning &t, int64_t M, int64_t K, int64_t N)
{
    if (t.wr > 0) return DecodeCfg{t.wr, t.wk, t.u, t.s};
    DecodeCfg c;
    if (M <= 8) { c.wr = 1; c.wk = 8; }
    else if (M <= 16) { c.wr = 2; c.wk = 4; }
    else if (M <= 32) { c.wr = 4; c.wk = 2; }
    else { c.wr = 8; c.wk = 1; }
    c.u = 4;
    const int64_t T = ceil_div(K, 128);
    int s = 1;
    while (s < 8 && T / (int64_t)(s * c.wk) > 2 * c.u) s *= 2;
    // enough CTAs to cover the machine at least ~twice when the layer is small
    while (s < 8 && ceil_div(N, 16 * c.wr) * s < 2 * 148 && T / (int64_t)(s * 2 * c.wk) >= 1) s *= 2;
    c.s = s;
    return c;
}

template <int MT, int WR, int WK, int U>
static int launch_cfg(const FwdArgs &a, int S)
{
    DecodeParams p;
    p.w = a.w; p.scales = a.scales; p.x = a.x; p.y = a.y; p.bias = a.bias;
    p.ov = a.ortho; p.has_ortho = a.has_ortho; p.alpha = a.alpha;
    p.M = (int)a.M; p.K = (int)a.K; p.N = (int)a.N; p.ldy = a.pitch_y();
    p.T = (int)ceil_div(a.K, 128);
    constexpr int R = 16 * WR, TOK = 8 * MT;
    const int steps_per_cta = (int)ceil_div(p.T, S);
    // X slab budget: keep a pass under ~96 KB so that two CTAs still fit one SM
    int pass_steps = (int)((96 * 1024 / a.M - 64) / 256);
    if (pass_steps < 1) pass_steps = 1;
    if (pass_steps > steps_per_cta) pass_steps = steps_per_cta;
    p.pass_steps = pass_steps;
    p.pitch = pass_steps * 256 + 64;
    const size_t smem = (size_t)a.M * p.pitch + (size_t)(WK + 1) * R * TOK * sizeof(float);

    auto kern = decode_kernel<MT, WR, WK, U>;
    static bool smem_set[kMaxDevices] = {};       // the attribute is per device
    const int dev = current_device_index();
    if (dev < 0) return ORTHO_B200_ERR_CUDA;
    if (!smem_set[dev]) {
        OB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        smem_set[dev] = true;
    }
    if (smem > 227 * 1024) return ORTHO_B200_ERR_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)S, (unsigned)ceil_div(a.N, R), 1);
    cfg.blockDim = dim3(WR * WK * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OB_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    count_launch();
    return ORTHO_B200_OK;
}

template <int MT>
static int launch_mt(const FwdArgs &a, const DecodeCfg &c)
{
#define OB_CASE(WR_, WK_)                                                      \
    if (c.wr == WR_ && c.wk == WK_) {                                          \
        return c.u == 2 ? launch_cfg<MT, WR_, WK_, 2>(a, c.s)                  \
                        : launch_cfg<MT, WR_, WK_, 4>(a, c.s);                 \
    }
    OB_CASE(1, 8) OB_CASE(2, 4) OB_CASE(4, 2) OB_CASE(8, 1) OB_CASE(1, 4) OB_CASE(2, 2)
#undef OB_CASE
    return ORTHO_B200_ERR_SHAPE;
}

// M <= 16: persistent TMA streaming kernel, unless another kernel was asked for explicitly
// (its TMA view needs whole 128-byte column blocks per row: K a multiple of 256)
static bool stream_selected(const Tuning &t, int64_t M, int64_t K)
{
    return M <= 16 && (K % 256) == 0 && (t.force_stream || t.wr == 0);
}
bool stream_kernel_selected(int64_t M, int64_t K)
{
    const Tuning t = tuning_snapshot();
    return M <= t.prefill_above && stream_selected(t, M, K);
}

int launch_decode_multi(const FwdArgs *layers, int nl)
{
    const Tuning t = tuning_snapshot();
    return launch_decode_stream_multi(layers, nl, t.stream_s, t.stream_stages);
}

int launch_decode(const FwdArgs &a)
{
    if (a.M > ORTHO_B200_DECODE_MAX_M) return ORTHO_B200_ERR_SHAPE;
    const Tuning t = tuning_snapshot();
    if (stream_selected(t, a.M, a.K)) return launch_decode_stream(a, t.stream_s, t.stream_stages);
    const DecodeCfg c = choose(t, a.M, a.K, a.N);
    if (a.M <= 8) return launch_mt<1>(a, c);
    if (a.M <= 16) return launch_mt<2>(a, c);
    if (a.M <= 32) return launch_mt<4>(a, c);
    return launch_mt<8>(a, c);
}

}  // namespace ob
