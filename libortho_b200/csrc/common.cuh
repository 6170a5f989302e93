// Shared device/host helpers of the sm_100a OrthoLinear forward.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ortho_b200.h"

namespace ob {

// ---- host-side status plumbing -----------------------------------------------------------------
void note_cuda_error(cudaError_t e);   // remembers e for ortho_b200_last_cuda_error()
void count_launch(int n = 1);          // feeds ortho_b200_launch_count()

#define OB_CUDA(call)                                                     \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) { ::ob::note_cuda_error(e__); return ORTHO_B200_ERR_CUDA; } \
    } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- per-device launch state ----------------------------------------------------------------------
// cudaFuncSetAttribute, the SM count and cluster occupancy belong to ONE device: caches of them are
// indexed by the current device (a process may run forwards on several GPUs) and only ever move from
// "unknown" to a value that every thread would compute identically, so they need no lock.
constexpr int kMaxDevices = 64;
static inline int current_device_index()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}
int device_sm_count(int dev);          // api.cu: multiprocessor count of device `dev`, cached

// ---- tuning hook state (ortho_b200_set_decode_config) ------------------------------------------------
// One record behind a mutex; every forward works on the snapshot it took when it started, so a
// concurrent change of the hook never shows half-applied inside one call.
struct Tuning {
    int wr = 0, wk = 0, u = 0, s = 0;   // generic decode kernel tiling (wr == 0: built-in choice)
    bool force_stream = false;          // streaming kernel with stream_s / stream_stages
    int stream_s = 0, stream_stages = 0;
    int prefill_above = 24;             // forwards with more tokens than this use the tensor-core kernels
    // forwards with mid_lo < tokens <= mid_hi use the tokens-as-M tensor-core kernel when they bring its workspace:
    // built in, above the streaming kernel's 16 tokens except on small layers up to 32 tokens; through the
    // hook, first (mid_first)
    int mid_lo = 16, mid_hi = 128;
    bool mid_first = false;
    bool gather_per_cta = false;        // peer exchange: every CTA signals the peers itself instead of the grid's last CTA
    bool patch_weights = true;          // tensor-core kernels fold the sparse entries into the weight tile (plan with ordered rows)
    int long_row_min = 64;              // = kLongRowMin: a plan's long-row threshold is max(this, 4 x the mean row)
};
constexpr int kPrefillAboveBuiltin = 24;
Tuning tuning_snapshot();              // decode.cu

// ---- the plan (definition shared by plan.cu / decode.cu / prefill.cu) -------------------------
// entries[i] = (f16 bits of value << 16) | column   for CSR entry i (row-major order kept)
struct Plan {
    uint32_t magic;
    int device;
    int64_t K, N, nnz;
    int64_t max_row_nnz;
    int32_t *row_ptr;     // [N+1] device copy
    uint32_t *entries;    // [nnz]
    float *row_max;       // [N] largest |value| of the row (infinite if the row holds a NaN)
    bool ordered;         // every row lists its columns in strictly ascending order, all inside [0, K)
    // Rows that stand out in length ("long": more than `heavy` entries = max(kLongRowMin, 4 x the mean row)) would
    // hold up the tensor-core kernel's in-flight sparse pass, so the plan lists them (hrow, ascending) and keeps
    // them once more as a zero-filled dense FP16 matrix hdense[n_pad][K] (n_pad = n_long rounded up to 128): a
    // pre-pass computes their sums as a small tensor-core GEMM (longrows.cu).  `heavy` is doubled until that
    // matrix fits kLongDenseMaxBytes; a CSR row that repeats a column cannot be held densely, and a plan that
    // meets one keeps no long rows.
    int heavy;
    int64_t n_long, n_pad;
    int32_t *hrow;
    __half *hdense;
};
constexpr int kLongRowMin = 64;
constexpr int64_t kLongDenseMaxBytes = 256ll << 20;
constexpr uint32_t kPlanMagic = 0x0B200A17u;

// view of the ortho component handed to kernels: either packed plan entries or raw CSR
struct OrthoView {
    const int32_t *row_ptr;
    const uint32_t *entries;   // non-null -> packed path
    const int32_t *col;        // raw CSR path
    const __half *val;
};
// one stored entry as (column, value); an entry outside [0, K) of a raw CSR view reads as an explicit zero
__device__ __forceinline__ void ortho_entry(const OrthoView &ov, int e, int K, int &c, float &v)
{
    if (ov.entries) {
        const uint32_t pk = ov.entries[e];
        c = (int)(pk & 0xFFFFu);
        v = __half2float(__ushort_as_half((unsigned short)(pk >> 16)));
    } else {
        c = ov.col[e];
        v = __half2float(ov.val[e]);
        if ((unsigned)c >= (unsigned)K) { c = 0; v = 0.f; }
    }
}

// Scale of a row's weight corrections: a sparse entry v of row n enters the weight tile as v * alpha / scale[n]
// (the epilogue multiplies the whole row by scale[n]).  Returns 0 when that cannot be represented safely in
// FP16 next to the integer weights (tiny or zero scale, huge values, NaN): such a row keeps the gather path.
// Converters and epilogue warps evaluate this independently and must agree, hence one function.
__device__ __forceinline__ float patch_rscale(float alpha, float scale, float row_max)
{
    const float r = __fdiv_rn(alpha, scale);
    const float top = __fmul_rn(row_max, fabsf(r));
    return (top <= 16384.f && fabsf(r) <= 3.0e38f && r != 0.f) ? r : 0.f;     // NaN and infinity fail the comparisons
}

// ---- INT4 -> FP16 in registers ------------------------------------------------------------------
// One 32-bit word holds 8 consecutive elements e0..e7 (e_i in bits [4i, 4i+4), low nibble = even
// element; src/ortho.c:315-320).  A nibble r is a 4-bit two's complement integer s (:321-323);
// r ^ 8 == s + 8.  OR-ing the exponent pattern 0x6400 (=1024.0) under the nibble yields the half
// 1024 + s + 8 for a nibble in bits 0-3, or 1024 + 16 (s + 8) for a nibble in bits 4-7.  Both are
// exact, so one subtract (or one fma by 1/16) gives s exactly.  Output pairs are
// (e0,e4) (e1,e5) (e2,e6) (e3,e7): the caller contracts them against activations stored in the
// same pair order, so no element ever has to be moved across a 16-bit boundary.
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) ^ c
    return d;
}

__device__ __forceinline__ void int4x8_to_half2x4(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t kLoMask = 0x000F000Fu, kHiMask = 0x00F000F0u;
    const uint32_t kLoMagic = 0x64086408u;   // 1024 | sign flip of a low nibble
    const uint32_t kHiMagic = 0x64806480u;   // 1024 | sign flip of a high nibble
    const __half2 kSubLo = __half2half2(__ushort_as_half((unsigned short)0x6408));   // 1032
    const __half2 kMulHi = __half2half2(__ushort_as_half((unsigned short)0x2C00));   // 1/16
    const __half2 kAddHi = __half2half2(__ushort_as_half((unsigned short)0xD480));   // -72
    uint32_t w8 = w >> 8;
    uint32_t a0 = lop3_and_xor(w, kLoMask, kLoMagic);
    uint32_t a1 = lop3_and_xor(w, kHiMask, kHiMagic);
    uint32_t a2 = lop3_and_xor(w8, kLoMask, kLoMagic);
    uint32_t a3 = lop3_and_xor(w8, kHiMask, kHiMagic);
    __half2 r0 = __hsub2(*reinterpret_cast<__half2 *>(&a0), kSubLo);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2 *>(&a1), kMulHi, kAddHi);
    __half2 r2 = __hsub2(*reinterpret_cast<__half2 *>(&a2), kSubLo);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2 *>(&a3), kMulHi, kAddHi);
    h[0] = *reinterpret_cast<uint32_t *>(&r0);
    h[1] = *reinterpret_cast<uint32_t *>(&r1);
    h[2] = *reinterpret_cast<uint32_t *>(&r2);
    h[3] = *reinterpret_cast<uint32_t *>(&r3);
}

// natural element order variant: pairs (e0,e1) (e2,e3) (e4,e5) (e6,e7).  A byte holds the pair
// (low nibble = even element).  prmt replicates byte i into both 16-bit halves under the 0x64
// exponent byte, the mask keeps bits 0-3 in the low half and bits 4-7 (now bits 20-23) in the high
// half, and one fma per pair applies {x - 1032, x/16 - 72} to the two halves.
__device__ __forceinline__ void int4x8_to_half2x4_natural(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t kExp = 0x64646464u;
    const uint32_t kMask = 0xFFF0FF0Fu;      // keep exponent bytes, low nibble (lo half), high nibble (hi half)
    const uint32_t kFlip = 0x00800008u;
    __half2 mul, add;
    {
        uint32_t m = 0x2C003C00u;            // hi = 1/16, lo = 1
        uint32_t a = 0xD480E408u;            // hi = -72,  lo = -1032
        mul = *reinterpret_cast<__half2 *>(&m);
        add = *reinterpret_cast<__half2 *>(&a);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t v;
        // bytes of result (high..low): 0x64, byte i of w, 0x64, byte i of w
        uint32_t sel = 0x4040u | (uint32_t)i | ((uint32_t)i << 8);
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(w), "r"(kExp), "r"(sel));
        v = lop3_and_xor(v, kMask, kFlip);
        __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&v), mul, add);
        h[i] = *reinterpret_cast<uint32_t *>(&r);
    }
}

// mma.sync m16n8k16, f16 x f16 -> f32 (legacy tensor path; used by the memory-bound decode kernel
// where the 16-row operand is the weight tile and the 8-column operand is the token block)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Reduce V per-lane values over the 32 lanes with a halving butterfly: V/2 + V/4 + ... + 1
// exchanges, then plain xor steps.  Returns the total of value index (lane >> (5 - log2 V)), valid
// in every lane of that index group.  The order of additions is fixed.
template <int V>
__device__ __forceinline__ float butterfly_reduce(float (&v)[V], int lane)
{
    int off = 16;
#pragma unroll
    for (int half = V / 2; half >= 1; half >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < half; j++) {
            const float send = up ? v[j] : v[j + half];
            const float keep = up ? v[j + half] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
    float r = v[0];
#pragma unroll
    for (int o2 = 16; o2 >= 1; o2 >>= 1)
        if (o2 <= off) r += __shfl_xor_sync(0xffffffffu, r, o2);
    return r;
}

// streaming 128-bit load of read-once weight bytes: bypass L1 allocation
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace ob

// launchers implemented in the kernel translation units
namespace ob {
struct FwdArgs {
    const uint8_t *w; const __half *scales; const __half *x; __half *y;
    const float *bias = nullptr;          // optional FP32 [N]: added in the FP32 epilogue, before the FP16 rounding
    OrthoView ortho; int has_ortho; float alpha;
    int64_t M, K, N, nnz;
    const Plan *plan;
    void *workspace; int64_t workspace_bytes;
    cudaStream_t stream;
    // output pitch in elements (0 = N) and, for the gathering entry point, the peer buffers: a
    // launcher whose kernel publishes to the peers itself sets *gather_fused
    int64_t ldy = 0;
    const struct GatherView *gv = nullptr;
    bool *gather_fused = nullptr;
    int64_t pitch_y() const { return ldy ? ldy : N; }
};
int launch_decode(const FwdArgs &a);
// the forward behind ortho_b200_forward(); ldy = output pitch in elements (0 = N), gv / gather_fused
// as in FwdArgs
int forward_impl(const void *q_weight, const void *q_scales_f16, const void *ortho_values_f16,
                 const int32_t *ortho_col_indices, const int32_t *ortho_row_ptr, int64_t nnz,
                 const void *x_f16, void *y_f16, int64_t M, int64_t K, int64_t N, float alpha,
                 const ortho_b200_plan *plan, void *workspace, int64_t workspace_bytes, void *stream,
                 int64_t ldy, const struct GatherView *gv, bool *gather_fused, const float *bias_f32 = nullptr);
int make_fwd_args(FwdArgs &a, const void *q_weight, const void *q_scales_f16, const void *ortho_values_f16,
                  const int32_t *ortho_col_indices, const int32_t *ortho_row_ptr, int64_t nnz,
                  const void *x_f16, void *y_f16, int64_t M, int64_t K, int64_t N, float alpha,
                  const ortho_b200_plan *plan, void *workspace, int64_t workspace_bytes, void *stream,
                  int64_t ldy, const float *bias_f32);
int launch_routed(const FwdArgs &a);                      // api.cu: picks the kernel family and launches
int launch_decode_multi(const FwdArgs *layers, int nl);   // decode.cu: one streaming launch for layers that share x
int launch_prefill(const FwdArgs &a);
int64_t long_rows_workspace_bytes(const Plan *pl, int64_t M);            // longrows.cu
int launch_long_rows(const FwdArgs &a, int Mp, void *ws, const float **part_out, int *nsplit_out);
int plan_build_long_rows(Plan *pl, cudaStream_t st, bool *dup_out);      // longrows.cu; returns a cudaError_t
int64_t prefill_workspace_bytes(int64_t M, int64_t K, int64_t N);
int64_t min_workspace_bytes(int64_t M, int64_t K, int64_t N);
int set_decode_config(int wr, int wk, int u, int s);
bool stream_kernel_selected(int64_t M, int64_t K);   // the forward of (M, K) will run decode_stream_kernel
// true = decode kernels: up to Tuning::prefill_above tokens, and narrow layers of up to 64 tokens
bool decode_regime(int64_t M, int64_t N, int64_t K);
// which kernel family a forward takes.  The tokens-as-M kernel needs its workspace whatever alpha is; a call
// inside its token range that brings none runs the kernels of the neighbouring regimes instead.
enum Route { kRouteDecode = 0, kRouteMid = 1, kRoutePrefill = 2 };
bool mid_token_range(int64_t M);
Route route_of(int64_t M, int64_t N, int64_t K, const void *workspace, int64_t workspace_bytes);
int launch_mid(const FwdArgs &a);                                  // mid.cu
int64_t mid_workspace_bytes(int64_t M, int64_t K, int64_t N);
}  // namespace ob
