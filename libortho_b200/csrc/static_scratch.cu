// Forward for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a region that is being
// captured into a CUDA graph, inside a real-time serving loop whose memory budget was fixed at
// start-up, or inside a plugin whose host application owns the allocator.  The ordinary forward
// asks such a caller for a workspace in the prefill regime (transposed activations + the FP32
// sparse term); this entry point instead keeps that scratch in a fixed array that is part of the
// library image, so the caller passes nothing but inputs and outputs.
//
// The array is one per process and device, it is shared by every call, and it keeps whatever the
// last call left in it.  Nothing in it has to start at zero: every byte the kernels read (the
// transposed activations including their zero padding, and the sparse-term rows of rows that own
// entries) is written earlier in the same call.  Two calls that overlap on the GPU (different
// streams, or two host threads) race on the array; serialise them.
#include <mutex>

#include "common.cuh"

namespace ob {

// 32 MiB: enough for e.g. K = N = 4096 at M = 512, or K = 8192, N = 1024 at M = 1024
__device__ __align__(256) unsigned char g_static_scratch[ORTHO_B200_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address, so the
// address is looked up once per device (with that device current) and cached.
static void *static_scratch_address(int *status)
{
    static std::mutex mu;
    static void *ptrs[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) { if (e != cudaSuccess) note_cuda_error(e); *status = ORTHO_B200_ERR_CUDA; return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
        if (e != cudaSuccess || !p) { note_cuda_error(e); *status = ORTHO_B200_ERR_CUDA; return nullptr; }
        ptrs[dev] = p;
    }
    *status = ORTHO_B200_OK;
    return ptrs[dev];
}

}  // namespace ob

using namespace ob;

extern "C" int ortho_b200_forward_static_scratch(const void *q_weight, const void *q_scales_f16,
                                                 const void *ortho_values_f16, const int32_t *ortho_col_indices,
                                                 const int32_t *ortho_row_ptr, int64_t nnz,
                                                 const void *x_f16, void *y_f16,
                                                 int64_t M, int64_t K, int64_t N, float alpha, void *stream)
{
    if (M == 0) return ORTHO_B200_OK;
    if (!q_weight || !q_scales_f16 || !x_f16 || !y_f16) return ORTHO_B200_ERR_NULL;
    if (M < 0 || N <= 0 || K <= 0 || (K % 32) != 0 || K > 65536 || nnz < 0 ||
        M > 0x7fffffffLL || N > 0x7fffff00LL || nnz > 0x7fffffffLL)
        return ORTHO_B200_ERR_SHAPE;
    if ((((uintptr_t)q_weight | (uintptr_t)x_f16 | (uintptr_t)y_f16) & 15u) != 0) return ORTHO_B200_ERR_ALIGN;
    if (((uintptr_t)q_scales_f16 & 1u) != 0) return ORTHO_B200_ERR_ALIGN;
    const bool has_ortho = (alpha > 0.0f) && (nnz > 0);
    if (has_ortho && (!ortho_values_f16 || !ortho_col_indices || !ortho_row_ptr)) return ORTHO_B200_ERR_NULL;

    // the same kernel choice as ortho_b200_forward makes for these sizes, so that both entries give the
    // same bits; only the tensor-core regime with an active sparse term needs scratch
    const bool decode = decode_regime(M, N, K);
    const int64_t need = (has_ortho && !decode) ? min_workspace_bytes(M, K, N) : 0;
    // (the tokens-as-M kernel is taken when its scratch fits the array, exactly as ortho_b200_forward takes it when
    // the caller's workspace is large enough; it is never required)
    if (need > (int64_t)ORTHO_B200_STATIC_SCRATCH_BYTES) return ORTHO_B200_ERR_SCRATCH_LIMIT;

    int major = 0, dev = 0;
    OB_CUDA(cudaGetDevice(&dev));
    OB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return ORTHO_B200_ERR_DEVICE;

    int st = ORTHO_B200_OK;
    void *scratch = static_scratch_address(&st);      // first call on a device: looks the address up
    if (st != ORTHO_B200_OK) return st;

    FwdArgs a;
    a.w = (const uint8_t *)q_weight;
    a.scales = (const __half *)q_scales_f16;
    a.x = (const __half *)x_f16;
    a.y = (__half *)y_f16;
    a.has_ortho = has_ortho ? 1 : 0;
    a.alpha = alpha;
    a.M = M; a.K = K; a.N = N; a.nnz = nnz;
    a.plan = nullptr;                                 // a plan would have to be allocated: raw CSR only
    a.ortho.row_ptr = has_ortho ? ortho_row_ptr : nullptr;
    a.ortho.entries = nullptr;
    a.ortho.col = has_ortho ? ortho_col_indices : nullptr;
    a.ortho.val = has_ortho ? (const __half *)ortho_values_f16 : nullptr;
    a.workspace = scratch;
    a.workspace_bytes = (int64_t)ORTHO_B200_STATIC_SCRATCH_BYTES;
    a.stream = (cudaStream_t)stream;
    return launch_routed(a);
}
