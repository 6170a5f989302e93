// Persistent streaming kernel for the decode regime (M <= 16): the kernel that has to run at HBM
// speed.  Same arithmetic as decode.cu (weights as the 16-row operand of mma.sync m16n8k16, token
// block as the 8-column operand, exact small-integer weights, per-row scale applied once in the
// FP32 epilogue, ortho term from packed entries), but organised around memory-level parallelism:
//
//  * the packed INT4 base is fetched by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) in boxes of
//    16 rows x 256 bytes (512 weights per row); every warp owns a private ring of such boxes with
//    one mbarrier per slot and keeps `stages` boxes in flight, across tile boundaries;
//  * a cluster of S CTAs (8 warps each) owns a 16-row output tile; the K range is split over the
//    8*S warps.  Clusters are persistent and walk the tiles round-robin; the activation slab of a
//    CTA's fixed K range is staged in shared memory once, in the pair order the unpack produces;
//  * partial sums are exchanged through distributed shared memory with a split-phase cluster
//    barrier: a tile's arrive is followed by the next tile's main loop, and the wait + finalize of
//    tile i happen after tile i+1 has been accumulated, so no warp idles at a barrier;
//  * the sparse stream is software-pipelined the same way: row pointers are fetched two tiles
//    ahead, packed entries one tile ahead, so that the dependent row_ptr -> entry -> activation
//    chain never sits on the critical path.  One warp handles one output row at a time; the
//    per-token sums are combined with a halving butterfly of warp shuffles (fixed order).
//
// No global scratch, no atomics: results are bitwise reproducible, and with alpha <= 0 or nnz == 0
// the sparse stream is not touched at all, so the output equals the base-only output exactly.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "gather.cuh"
#include "tma.cuh"

namespace ob {

// One TMA box is 16 rows x KBX column blocks of 128 packed bytes (KBX is a kernel template
// parameter: 2 for M <= 8, 1 for M = 9..16 where the activation slab limits the K range per CTA).
constexpr int kWarps = 8;

// One launch may walk the tiles of several layers that share the activations (same X, same K): the tile
// sequence is the concatenation of the layers' 16-row tiles, layer l owning tiles [tile0, next tile0).
constexpr int kMaxLayers = 4;
struct StreamLayer {
    const __half *scales; __half *y; const float *bias;   // bias: optional FP32 [N], added before the FP16 rounding
    OrthoView ov; int has_ortho; float alpha;
    int N;         // output rows of this layer
    int ldy;       // elements between token rows of y
    int tile0;     // first tile of this layer in the launch's tile sequence
};
struct StreamMaps { CUtensorMap m[kMaxLayers]; };
struct StreamParams {
    StreamLayer L[kMaxLayers];
    int nl;        // layers in this launch
    int any_ortho; // some layer has an active sparse term
    const __half *x;
    int M, K;
    int nboxes;    // ceil(K / weights per box row)
    int ntiles;    // 16-row tiles of all layers together
    int pitch;     // bytes between token rows of the staged activation slab
    int stages;    // ring depth per warp
    int red_bufs;  // 2: partial sums double-buffered; 1 (S == 1 only): one buffer and a group barrier per tile
    int *status;   // device word: set to 1 if a bounded wait gave up (2: a peer's gather flag)
};
// extra kernel argument of the GATHER instantiation (the plain one takes an empty struct)
struct StreamGather {
    int ldy;       // elements between token rows of y
    GatherView gv; // the finalized values are stored into every rank's output buffer
};
struct StreamNoGather {};
template <bool G> struct StreamGatherArg { using type = StreamNoGather; };
template <> struct StreamGatherArg<true> { using type = StreamGather; };

__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// MV = token slots kept per output row (M <= MV, power of two).  One CTA = 8 warps that split the
// CTA's K range of a 16-row tile; a cluster of S CTAs splits K further.
// GATHER: instantiation with a pitched output, peer stores and the flag exchange; the plain one
// (output pitch N, one GPU) carries none of it
// NG = warp groups per CTA.  A group is the 8-warp unit described above, with its own rings, tile barrier
// and reduction buffers; the groups of a CTA work on different tiles and share one activation slab, which
// is what limits residency for 8 and 16 tokens (NG = 2: one CTA of 16 warps per SM instead of one of 8).
// NL = 1: one layer (every per-layer lookup is resolved at compile time); NL = kMaxLayers: up to that many.
template <int NL>
__device__ __forceinline__ int layer_of(const StreamParams &p, int tile)
{
    int l = 0;
    if constexpr (NL > 1) {
#pragma unroll
        for (int i = 1; i < NL; i++)
            if (i < p.nl && tile >= p.L[i].tile0) l = i;
    }
    return l;
}

template <int MV, int KBX, bool GATHER, int NG, int NL>
__global__ void __launch_bounds__(NG * kWarps * 32, NG == 2 ? 1 : 2)
decode_stream_kernel(const __grid_constant__ StreamMaps maps, const StreamParams p,
                     const typename StreamGatherArg<GATHER>::type gp)
{
    constexpr int kKbx = KBX;
    constexpr int kBoxBytes = 16 * KBX * 128;
    constexpr int kBoxK = 256 * KBX;
    constexpr int MT = (MV + 7) / 8;              // mma n=8 token blocks
    constexpr int NCH = 2;                        // independent accumulator chains
    constexpr int LPG = 32 / MV;                  // lanes per token index after the butterfly
    extern __shared__ __align__(1024) unsigned char smem[];

    // tid / warp are relative to the warp group; cid / G index warp groups, not CTAs
    const int grp = (NG == 1) ? 0 : (int)(threadIdx.x >> 8);
    const int tid = threadIdx.x & 255, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = (int)cluster_nctarank();
    const int rank = (int)cluster_ctarank();
    const int cid = blockIdx.y * NG + grp, G = gridDim.y * NG;
    const int K = p.K, M = p.M;

    // ---- shared memory carve-up ----------------------------------------------------------------
    // the 128-byte TMA swizzle is a function of the shared-memory address: ring slots sit on 1 KB
    // one region per warp group (rounded to 1 KB), then the activation slab shared by the groups
    const size_t region = ((size_t)kWarps * p.stages * kBoxBytes + (((kWarps * p.stages + 1) * 8 + 127) & ~127) +
                           (size_t)p.red_bufs * kWarps * 16 * MV * 4 + (size_t)2 * 16 * MV * 4 + 1023) & ~(size_t)1023;
    unsigned char *base = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
    unsigned char *ring = base + (size_t)grp * region;                            // kWarps * stages boxes
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + (size_t)kWarps * p.stages * kBoxBytes);
    uint64_t *tbar = bars + kWarps * p.stages;                                    // tile barrier (S == 1)
    float *red = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(bars) + (((kWarps * p.stages + 1) * 8 + 127) & ~127));
    float *osm = red + p.red_bufs * kWarps * 16 * MV;                             // [2][16*MV]
    unsigned char *xs = base + (size_t)NG * region;                               // M * pitch

    // ---- this warp's share of the K range, in boxes of 256 weights -----------------------------
    const int cb0 = (p.nboxes * rank) / S, cb1 = (p.nboxes * (rank + 1)) / S;
    const int wb0 = cb0 + ((cb1 - cb0) * warp) / kWarps, wb1 = cb0 + ((cb1 - cb0) * (warp + 1)) / kWarps;
    const int nbw = wb1 - wb0;
    const int nt = cid < p.ntiles ? (p.ntiles - cid + G - 1) / G : 0;   // tiles walked by this warp group
    // every group of every CTA of the cluster goes through the same number of tile barriers
    const int nt_loop = ((int)blockIdx.y * NG < p.ntiles) ? (p.ntiles - (int)blockIdx.y * NG + G - 1) / G : 0;
    const int total = nt * nbw;                           // boxes this warp consumes
    const int k_lo = cb0 * kBoxK, k_hi = min(cb1 * kBoxK, K); // activation slab of this CTA

    unsigned char *my_ring = ring + (size_t)warp * p.stages * kBoxBytes;
    uint64_t *my_bars = bars + warp * p.stages;

    // producer cursor (meaningful in lane 0): next box to fetch = (tile i_ti, box i_bi) into slot i_st.
    // All ring indices advance by increment-and-wrap; there is no division in the steady state.
    int i_ti = 0, i_bi = 0, i_st = 0, i_left = total;
    auto issue = [&]() {   // lane 0 only
        mbar_arrive_expect_tx(&my_bars[i_st], kBoxBytes);
        const int T = cid + i_ti * G, l = layer_of<NL>(p, T);
        tma_load_3d(my_ring + (size_t)i_st * kBoxBytes, &maps.m[l], &my_bars[i_st], 0, (wb0 + i_bi) * kKbx, (T - p.L[l].tile0) * 16);
        if (++i_bi == nbw) { i_bi = 0; ++i_ti; }
        if (++i_st == p.stages) i_st = 0;
        --i_left;
    };

    // weights and the sparse structure are constants of the layer: they are prefetched before the
    // grid dependency is resolved; activations are only touched after griddep_wait()
    if (lane == 0) {
        for (int l = 0; l < (NL == 1 ? 1 : p.nl); l++) prefetch_tensormap(&maps.m[l]);
        for (int s = 0; s < p.stages; s++) mbar_init(&my_bars[s], 1);
        if (warp == 0) mbar_init(tbar, kWarps * 32);
        fence_mbar_init();
        const int pre = min(p.stages, total);
        for (int i = 0; i < pre; i++) issue();
    }

    // ---- sparse stream prologue: row pointers of the first two tiles, entries of the first ------
    // every CTA walks all 16 rows of a tile (2 per warp) and keeps the entries inside its K range
    int rp_cur[2][2] = {{0, 0}, {0, 0}}, rp_nxt[2][2] = {{0, 0}, {0, 0}};
    uint32_t ent[2][2] = {{0, 0}, {0, 0}};
    auto load_rp = [&](int ti, int (&rp)[2][2]) {
        const int T = cid + ti * G;
        const StreamLayer &Ly = p.L[layer_of<NL>(p, T)];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int n = (T - Ly.tile0) * 16 + warp + 8 * r;
            rp[r][0] = rp[r][1] = 0;
            if (ti < nt && Ly.has_ortho && n < Ly.N) { rp[r][0] = Ly.ov.row_ptr[n]; rp[r][1] = Ly.ov.row_ptr[n + 1]; }
        }
    };
    auto load_entry = [&](const OrthoView &ov, int e) -> uint32_t {
        if (ov.entries) return ov.entries[e];
        const int c = ov.col[e];
        const unsigned short vb = __half_as_ushort(ov.val[e]);
        return ((unsigned)c >= (unsigned)K) ? 0u : (((uint32_t)vb << 16) | (uint32_t)c);
    };
    // entries of local tile ti (whose row pointers are rp); rows without entries load nothing
    auto load_ent = [&](int ti, const int (&rp)[2][2], uint32_t (&en)[2][2]) {
        const OrthoView &ov = p.L[layer_of<NL>(p, cid + ti * G)].ov;
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int e = rp[r][0] + q * 32 + lane;
                en[r][q] = (e < rp[r][1]) ? load_entry(ov, e) : 0u;
            }
    };
    if (p.any_ortho) {
        load_rp(0, rp_cur);
        load_rp(1, rp_nxt);
        load_ent(0, rp_cur, ent);
    }

    griddep_wait();
    if constexpr (GATHER) {   // deferred exchange: the previous forward's slices must have arrived before X is read
        if (!gather_wait_previous(gp.gv)) atomicExch(p.status, 2);
    }

    // ---- stage X[:, k_lo:k_hi) once, in unpack pair order ---------------------------------------
    // 16-byte chunk (x0..x7) is stored as (x0,x4,x1,x5,x2,x6,x3,x7); inside a 128-element step the 16
    // chunks are laid out [j][t] so that the 4 lanes of a row group read 64 contiguous bytes.
    {
        const int chunks_per_row = (cb1 - cb0) * (kBoxK / 8);
        const int totalc = M * chunks_per_row;
        for (int idx = (int)threadIdx.x; idx < totalc; idx += NG * kWarps * 32) {
            const int r = idx / chunks_per_row, q = idx - r * chunks_per_row;
            const int k = k_lo + q * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (k < K) v = *reinterpret_cast<const uint4 *>(p.x + (size_t)r * K + k);
            uint4 o;
            o.x = prmt_b32(v.x, v.z, 0x5410);
            o.y = prmt_b32(v.x, v.z, 0x7632);
            o.z = prmt_b32(v.y, v.w, 0x5410);
            o.w = prmt_b32(v.y, v.w, 0x7632);
            const int sl = q >> 4, c16 = q & 15, tt = c16 >> 2, j = c16 & 3;
            *reinterpret_cast<uint4 *>(xs + (size_t)r * p.pitch + sl * 256 + j * 64 + tt * 16) = o;
        }
    }
    __syncthreads();
    griddep_launch();
    // A box is laid out [row][column block][128 B]; the 128-byte swizzle XORs the 16-byte chunk index
    // with bits 7..9 of the shared-memory address, i.e. with (row * kKbx + block) & 7.  mma row g is
    // mapped to box row rho(g) = g with bits 0 and 1 swapped, so that the two rows met in one
    // shared-memory phase (g = 2q, 2q+1) differ in bit 2 of that XOR term: every phase is conflict free
    // (for one column block per box the XOR term is row & 7 and rho rotates the low three bits instead).
    const int brow0 = (KBX == 2) ? ((g & 4) | ((g & 1) << 1) | ((g >> 1) & 1)) : ((g >> 1) | ((g & 1) << 2));
    const int brow1 = brow0 + 8;
    // token row read by this lane for the mma column g of block mt.  Columns >= M are never stored,
    // and mma columns are independent, so those lanes may read any valid row: clamp, no predicate.
    const unsigned char *xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) xrow[mt] = xs + (size_t)min(8 * mt + g, M - 1) * p.pitch + t * 16;

    // split-phase tile barrier: mbarrier inside one CTA, hardware cluster barrier across CTAs
    auto tile_arrive = [&]() { if (S == 1) mbar_arrive(tbar); else cluster_arrive(); };
    auto tile_wait = [&](int ti) -> bool {
        if (S == 1) return mbar_wait(tbar, (uint32_t)(ti & 1));
        cluster_wait();
        return true;
    };

    bool dead = false;
    int c_st = 0;              // consumer cursor: ring slot and its phase parity
    uint32_t c_ph = 0;
    float acc[NCH][MT][4];

    // element of a tile finalized by this thread (fixed for the whole kernel)
    const int RB = 16 / S;
    const bool fin_on = tid < RB * M;
    const int fin_m = fin_on ? tid / RB : 0;
    const int fin_i = rank * RB + (fin_on ? tid - fin_m * RB : 0);

    // the row scale a finalizing thread needs is fetched one tile early, so that the finalize of
    // tile i (executed while tile i+1 is in flight) never waits on global memory
    float sc_prev = 0.f, bias_prev = 0.f;
    const int rmask = p.red_bufs - 1;          // 1: alternate the partial-sum buffers, 0: single buffer
    auto finalize = [&](int ti) {
        const int buf = ti & 1, rbuf = ti & rmask;
        if (fin_on) {
            const int m = fin_m, i = fin_i;
            const int T = cid + ti * G;
            const StreamLayer &Ly = p.L[layer_of<NL>(p, T)];
            const int n = (T - Ly.tile0) * 16 + i;
            if (n < Ly.N) {
                const uint32_t red_base = smem_u32(red + (size_t)rbuf * kWarps * 16 * MV);
                const uint32_t osm_base = smem_u32(osm + (size_t)buf * 16 * MV);
                float s = 0.f, o = 0.f;
                if (S == 1) {
                    const float *rb = red + (size_t)rbuf * kWarps * 16 * MV + i * MV + m;
#pragma unroll
                    for (int w = 0; w < kWarps; w++) s += rb[w * 16 * MV];
                    if (Ly.has_ortho) o = osm[(size_t)buf * 16 * MV + i * MV + m];
                } else {
                    for (int r2 = 0; r2 < S; r2++) {
                        const uint32_t rb = mapa_shared(red_base, (uint32_t)r2);
#pragma unroll
                        for (int w = 0; w < kWarps; w++) s += ld_dsmem_f32(rb + (uint32_t)((w * 16 * MV + i * MV + m) * 4));
                        if (Ly.has_ortho) o += ld_dsmem_f32(mapa_shared(osm_base, (uint32_t)r2) + (uint32_t)((i * MV + m) * 4));
                    }
                }
                float v = sc_prev * s;
                if (Ly.has_ortho) v = fmaf(Ly.alpha, o, v);
                v += bias_prev;                                  // 0 when the layer has no bias
                if constexpr (!GATHER) {
                    Ly.y[(size_t)m * Ly.ldy + n] = __float2half_rn(v);
                } else {
                    const __half hv = __float2half_rn(v);
                    const size_t at = (size_t)m * gp.ldy + n;
                    for (int r = 0; r < gp.gv.world; r++) gp.gv.y[r][at] = hv;
                }
            }
        }
    };

    for (int ti = 0; ti < nt_loop; ti++) {
        float sc_new = 0.f, bias_new = 0.f;
        const int l_cur = layer_of<NL>(p, cid + ti * G);
        if (fin_on) {
            const StreamLayer &Ly = p.L[l_cur];
            const int n = (cid + ti * G - Ly.tile0) * 16 + fin_i;
            if (ti < nt && n < Ly.N) {
                sc_new = __half2float(Ly.scales[n]);
                if (Ly.bias) bias_new = Ly.bias[n];
            }
        }
#pragma unroll
        for (int c = 0; c < NCH; c++)
#pragma unroll
            for (int i = 0; i < MT; i++) { acc[c][i][0] = acc[c][i][1] = acc[c][i][2] = acc[c][i][3] = 0.f; }

        // sparse stream, pipeline stages A/B: row pointers two tiles ahead, entries one tile ahead
        int rp_fut[2][2] = {{0, 0}, {0, 0}};
        uint32_t ent_nxt[2][2] = {{0, 0}, {0, 0}};
        if (p.any_ortho) {
            load_rp(ti + 2, rp_fut);
            load_ent(ti + 1, rp_nxt, ent_nxt);
        }

        // ---- base: consume this warp's boxes of the tile ---------------------------------------
        for (int bi = 0; bi < (ti < nt ? nbw : 0); bi++) {
            if (!mbar_try_wait(&my_bars[c_st], c_ph)) {
                if (!dead && !mbar_wait(&my_bars[c_st], c_ph)) { dead = true; if (lane == 0) atomicExch(p.status, 1); }
            }
            const unsigned char *box = my_ring + (size_t)c_st * kBoxBytes;
            if (++c_st == p.stages) { c_st = 0; c_ph ^= 1u; }
            const int xoff = (wb0 + bi - cb0) * (kBoxK * 2);
#pragma unroll
            for (int s2 = 0; s2 < 2 * kKbx; s2++) {
                const uint32_t c = (uint32_t)(4 * (s2 & 1) + t);
                const int line0 = brow0 * kKbx + (s2 >> 1), line1 = brow1 * kKbx + (s2 >> 1);
                const uint4 wa = *reinterpret_cast<const uint4 *>(box + line0 * 128 + ((c ^ (uint32_t)(line0 & 7)) << 4));
                const uint4 wb = *reinterpret_cast<const uint4 *>(box + line1 * 128 + ((c ^ (uint32_t)(line1 & 7)) << 4));
                const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w};
                const uint32_t wwb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t ha[4], hb[4];
                    int4x8_to_half2x4(wwa[j], ha);
                    int4x8_to_half2x4(wwb[j], hb);
                    const uint32_t A0[4] = {ha[0], hb[0], ha[1], hb[1]};
                    const uint32_t A1[4] = {ha[2], hb[2], ha[3], hb[3]};
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        const uint4 xb = *reinterpret_cast<const uint4 *>(xrow[mt] + xoff + s2 * 256 + j * 64);
                        mma_16816(acc[0][mt], A0, xb.x, xb.y);
                        mma_16816(acc[1][mt], A1, xb.z, xb.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && i_left > 0) issue();
        }

        // ---- sparse stream, stage C: this tile's rows from the prefetched entries ---------------
        float osum[2] = {0.f, 0.f};
        if (p.any_ortho) {
            const OrthoView &ov_cur = p.L[l_cur].ov;
#pragma unroll
            for (int r = 0; r < 2; r++) {
                float a[MV];
#pragma unroll
                for (int m = 0; m < MV; m++) a[m] = 0.f;
                const int e0 = rp_cur[r][0], e1 = rp_cur[r][1];
                auto apply = [&](uint32_t pk) {
                    const int c = (int)(pk & 0xFFFFu);
                    if (c >= k_lo && c < k_hi) {
                        const float v = __half2float(__ushort_as_half((unsigned short)(pk >> 16)));
                        const int kk = c - k_lo;
                        const int q = kk >> 3, e = kk & 7;
                        const int sl = q >> 4, c16 = q & 15;
                        const unsigned char *px = xs + sl * 256 + (c16 & 3) * 64 + (c16 >> 2) * 16 + (((e & 3) << 1) | (e >> 2)) * 2;
#pragma unroll
                        for (int m = 0; m < MV; m++) {
                            const int mm = (MV == 1) ? 0 : min(m, M - 1);   // slots >= M are never stored
                            a[m] = fmaf(v, __half2float(*reinterpret_cast<const __half *>(px + (size_t)mm * p.pitch)), a[m]);
                        }
                    }
                };
                if (e0 + lane < e1) apply(ent[r][0]);
                if (e0 + 32 + lane < e1) apply(ent[r][1]);
                for (int e = e0 + 64 + lane; e < e1; e += 32) apply(load_entry(ov_cur, e));
                osum[r] = butterfly_reduce<MV>(a, lane);
            }
        }

        // ---- deferred exchange: finish the previous tile, then publish this one -----------------
        if (ti > 0) {
            if (!tile_wait(ti - 1) && !dead) { dead = true; if (lane == 0) atomicExch(p.status, 1); }
            finalize(ti - 1);
        }
        // single partial-sum buffer: every read of the previous tile's sums precedes the new writes
        if (rmask == 0) asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(kWarps * 32) : "memory");
        {
            float *mine = red + ((size_t)(ti & rmask) * kWarps + warp) * 16 * MV;
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int col = 8 * mt + 2 * t + q;
                    if (col < MV) {
                        mine[brow0 * MV + col] = acc[0][mt][q] + acc[1][mt][q];
                        mine[brow1 * MV + col] = acc[0][mt][2 + q] + acc[1][mt][2 + q];
                    }
                }
            }
            if (p.any_ortho && (lane & (LPG - 1)) == 0) {
                float *o = osm + (size_t)(ti & 1) * 16 * MV;
                o[warp * MV + lane / LPG] = osum[0];
                o[(warp + 8) * MV + lane / LPG] = osum[1];
            }
        }
        tile_arrive();
        sc_prev = sc_new;
        bias_prev = bias_new;

        if (p.any_ortho) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                rp_cur[r][0] = rp_nxt[r][0]; rp_cur[r][1] = rp_nxt[r][1];
                rp_nxt[r][0] = rp_fut[r][0]; rp_nxt[r][1] = rp_fut[r][1];
                ent[r][0] = ent_nxt[r][0]; ent[r][1] = ent_nxt[r][1];
            }
        }
    }
    if (nt_loop > 0) {
        if (!tile_wait(nt_loop - 1) && !dead) { if (lane == 0) atomicExch(p.status, 1); }
        finalize(nt_loop - 1);
    }
    // nobody may leave while a peer can still read its shared memory
    if (S > 1) { cluster_arrive(); cluster_wait(); }
    // multi-GPU: the last CTA raises this rank's flag on every peer and waits for theirs
    if constexpr (GATHER) {
        if (!gather_signal_and_wait(gp.gv, gridDim.x * gridDim.y)) atomicExch(p.status, 2);
    }
}

// ---- host ------------------------------------------------------------------------------------
int *kernel_status_word();   // api.cu

static size_t stream_smem_bytes(int MV, int kbx, int64_t M, int boxes_per_cta, int stages, int ng = 1, int red_bufs = 2)
{
    const size_t region = ((size_t)kWarps * stages * (16 * kbx * 128) + (((kWarps * stages + 1) * 8 + 127) & ~127) +
                           (size_t)red_bufs * kWarps * 16 * MV * 4 + (size_t)2 * 16 * MV * 4 + 1023) & ~(size_t)1023;
    return 1024 + (size_t)ng * region + (size_t)M * (boxes_per_cta * 512 * kbx + 64);
}

// layers[0..nl): layers that share x, M, K and the stream (nl == 1 for the ordinary forward)
template <int MV, int KBX, bool GATHER, int NG, int NL>
static int launch_stream_mv(const FwdArgs *layers, int nl, const StreamMaps &maps, int S, int stages, int red_bufs)
{
    constexpr int kBoxK = 256 * KBX;
    const FwdArgs &a = layers[0];
    StreamParams p;
    memset(&p, 0, sizeof(p));
    p.nl = nl;
    int tiles = 0;
    for (int l = 0; l < nl; l++) {
        const FwdArgs &f = layers[l];
        StreamLayer &Ly = p.L[l];
        Ly.scales = f.scales; Ly.y = f.y; Ly.bias = f.bias; Ly.ov = f.ortho; Ly.has_ortho = f.has_ortho; Ly.alpha = f.alpha;
        Ly.N = (int)f.N; Ly.ldy = (int)f.pitch_y(); Ly.tile0 = tiles;
        tiles += (int)ceil_div(f.N, 16);
        p.any_ortho |= f.has_ortho;
    }
    p.x = a.x;
    p.M = (int)a.M; p.K = (int)a.K;
    p.nboxes = (int)ceil_div(a.K, kBoxK);
    p.ntiles = tiles;
    const int boxes_per_cta = (int)ceil_div(p.nboxes, S);
    p.pitch = boxes_per_cta * kBoxK * 2 + 64;
    p.stages = stages;
    p.red_bufs = red_bufs;
    p.status = kernel_status_word();
    if (!p.status) return ORTHO_B200_ERR_CUDA;
    typename StreamGatherArg<GATHER>::type gp;
    if constexpr (GATHER) {
        gp.ldy = (int)a.pitch_y();
        if (a.gv) {
            gp.gv = *a.gv;
            if (a.gather_fused) *a.gather_fused = true;
        } else {               // pitched output without peers: a world of one whose buffer is y
            gp.gv = GatherView{};
            gp.gv.world = 1;
            gp.gv.y[0] = a.y;
        }
    }
    const size_t smem = stream_smem_bytes(MV, KBX, a.M, boxes_per_cta, stages, NG, red_bufs);
    if (smem > 227 * 1024) return ORTHO_B200_ERR_SHAPE;
    auto kern = decode_stream_kernel<MV, KBX, GATHER, NG, NL>;
    static bool attr_set[kMaxDevices] = {};       // the attribute is per device
    const int dev = current_device_index();
    if (dev < 0) return ORTHO_B200_ERR_CUDA;
    if (!attr_set[dev]) {
        OB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NG * kWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this grid may start (and prefetch weights) while the previous
    // kernel of the stream drains; the kernel waits for that kernel before touching activations
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    // persistent grid: as many clusters as can be co-resident, never more than there are tiles
    // (cached per device, cluster size and shared-memory footprint; a racing thread at worst asks twice)
    static struct { int dev, s; size_t smem; int n; } cache[16];
    static std::atomic<int> cache_n{0};
    int mc = 0;
    const int have = cache_n.load(std::memory_order_acquire);
    for (int i = 0; i < have && i < 16; i++)
        if (cache[i].dev == dev && cache[i].s == S && cache[i].smem == smem) mc = cache[i].n;
    if (mc == 0) {
        const int sms = device_sm_count(dev);
        cfg.gridDim = dim3((unsigned)S, (unsigned)sms, 1);
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = sms / S; }
        cfg.numAttrs = 2;
        mc = n;
        static std::mutex mu;
        std::lock_guard<std::mutex> lock(mu);
        const int slot = cache_n.load(std::memory_order_relaxed);
        if (slot < 16) { cache[slot] = {dev, S, smem, n}; cache_n.store(slot + 1, std::memory_order_release); }
    }
    const int units = (int)ceil_div(p.ntiles, NG);       // a CTA takes NG tiles per round
    int Gc = mc < units ? mc : units;
    cfg.gridDim = dim3((unsigned)S, (unsigned)Gc, 1);
    OB_CUDA(cudaLaunchKernelEx(&cfg, kern, maps, p, gp));
    count_launch();
    return ORTHO_B200_OK;
}

// One launch for nl layers that share x, M, K (M <= 16, K a multiple of 256, nl <= kMaxLayers).  More than one
// layer: plain outputs only (no peer gather).
int launch_decode_stream_multi(const FwdArgs *layers, int nl, int cfg_s, int cfg_stages)
{
    const FwdArgs &a = layers[0];
    if (a.M > 16 || nl < 1 || nl > kMaxLayers) return ORTHO_B200_ERR_SHAPE;
    const int MV = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : a.M <= 8 ? 8 : 16;
    const int kbx = (MV <= 8) ? 2 : 1;
    const int nboxes = (int)ceil_div(a.K, 256 * kbx);
    int S = cfg_s, stages = cfg_stages, ng = 1, red_bufs = 2;   // 0 = built-in choice
    if (S <= 0) {
        // one CTA per tile covers all of K when its activation slab fits; otherwise split K over the
        // smallest cluster that does
        S = 1;
        while (S < 8 && stream_smem_bytes(MV, kbx, a.M, (int)ceil_div(nboxes, S), 2) > 200 * 1024) S *= 2;
        // few row tiles (a narrow layer, or one GPU's shard of a layer): a warp group per tile would leave most of
        // the GPU idle for a whole K sweep, so K is split over a larger cluster while that still gives every warp a
        // box per tile and no more groups than can be resident (about two per SM)
        {
            int tiles = 0;
            for (int l = 0; l < nl; l++) tiles += (int)ceil_div(layers[l].N, 16);
            const int cap = 2 * device_sm_count(current_device_index());
            while (S < 8 && tiles * S * 2 <= cap && nboxes / (S * 2) >= kWarps) S *= 2;
        }
        // a large activation slab (8 or more tokens, or a long K) leaves room for one CTA per SM only;
        // two warp groups then share one slab when that needs no further split of K (a cluster costs a DSMEM
        // exchange per tile and makes every CTA walk the tile's sparse entries) and leaves each
        // warp at least one box per tile; without a cluster a single partial-sum buffer may make it fit
        const int bpc2 = (int)ceil_div(nboxes, S);
        if (nboxes / S >= kWarps && 2 * stream_smem_bytes(MV, kbx, a.M, bpc2, 2) > 227 * 1024) {   // one CTA per SM otherwise
            if (stream_smem_bytes(MV, kbx, a.M, bpc2, 2, 2, 2) <= 227 * 1024) ng = 2;
            else if (S == 1 && stream_smem_bytes(MV, kbx, a.M, bpc2, 2, 2, 1) <= 227 * 1024) { ng = 2; red_bufs = 1; }
        }
    }
    if (S > 8) S = 8;
    const int bpc = (int)ceil_div(nboxes, S);
    if (stages <= 0) {
        // one token: 2 CTAs of 128 registers per SM, and a third ring slot when two such CTAs still fit
        stages = (MV == 1 && stream_smem_bytes(MV, kbx, a.M, bpc, 3) <= 113 * 1024) ? 3 : 2;
    }
    while (stages > 2 && stream_smem_bytes(MV, kbx, a.M, bpc, stages, ng, red_bufs) > 227 * 1024) stages--;

    // per layer a [N][K/2 / 128][128 B] view of the packed base; blocks past the end of a row read as zero
    StreamMaps maps;
    memset(&maps, 0, sizeof(maps));
    for (int l = 0; l < nl; l++)
        if (!make_tensor_map_rows_of_128B(&maps.m[l], layers[l].w, (uint64_t)layers[l].N, (uint64_t)(a.K / 2), 16, (uint32_t)kbx))
            return ORTHO_B200_ERR_CUDA;
    // the GATHER instantiation serves the peer gather and, for one layer, any output whose pitch is not N
    const bool gather = nl == 1 && (a.gv || a.pitch_y() != a.N);
    if (nl > 1 && a.gv) return ORTHO_B200_ERR_SHAPE;
#define OB_STREAM(MV_, KBX_, NG_) \
    (nl > 1 ? launch_stream_mv<MV_, KBX_, false, NG_, kMaxLayers>(layers, nl, maps, S, stages, red_bufs) \
     : gather ? launch_stream_mv<MV_, KBX_, true, NG_, 1>(layers, nl, maps, S, stages, red_bufs) \
              : launch_stream_mv<MV_, KBX_, false, NG_, 1>(layers, nl, maps, S, stages, red_bufs))
    switch (MV) {
        case 1: return ng == 2 ? OB_STREAM(1, 2, 2) : OB_STREAM(1, 2, 1);
        case 2: return ng == 2 ? OB_STREAM(2, 2, 2) : OB_STREAM(2, 2, 1);
        case 4: return ng == 2 ? OB_STREAM(4, 2, 2) : OB_STREAM(4, 2, 1);
        case 8: return ng == 2 ? OB_STREAM(8, 2, 2) : OB_STREAM(8, 2, 1);
        default: return ng == 2 ? OB_STREAM(16, 1, 2) : OB_STREAM(16, 1, 1);
    }
#undef OB_STREAM
}

int launch_decode_stream(const FwdArgs &a, int cfg_s, int cfg_stages)
{
    return launch_decode_stream_multi(&a, 1, cfg_s, cfg_stages);
}

}  // namespace ob
