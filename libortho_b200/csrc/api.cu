// extern "C" surface: argument validation, status plumbing and the decode / prefill regime split.
//
// Takes the place of forward_cuda_wrapper (torch_bind/bindings.cpp:9-44) and of the host
// dispatcher orth_layer_forward_cuda (src/dual_gemm.cu:295-372) of the reference.  Unlike the
// reference dispatcher it never synchronises the device and it reports failures as status
// codes instead of dropping them.
#include <atomic>

#include "common.cuh"

namespace ob {

static thread_local int tl_last_cuda_error = 0;
static std::atomic<long long> g_launches{0};

void note_cuda_error(cudaError_t e) { tl_last_cuda_error = (int)e; (void)cudaGetLastError(); }
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// device word that kernels set when a bounded wait gives up; reset and read by
// ortho_b200_query_kernel_status()
__device__ int g_kernel_status_word;

int *kernel_status_word()
{
    static thread_local int cached_dev = -1;
    static thread_local int *cached = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev != cached_dev) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_kernel_status_word);
        if (e != cudaSuccess) { note_cuda_error(e); return nullptr; }
        cached = (int *)p;
        cached_dev = dev;
    }
    return cached;
}

int device_sm_count(int dev)
{
    static std::atomic<int> cached[kMaxDevices];
    if (dev < 0 || dev >= kMaxDevices) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n <= 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); return 148; }
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

static int check_device()
{
    static thread_local int checked_device = -1;
    int dev = 0;
    OB_CUDA(cudaGetDevice(&dev));
    if (dev == checked_device) return ORTHO_B200_OK;
    int major = 0;
    OB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return ORTHO_B200_ERR_DEVICE;
    checked_device = dev;
    return ORTHO_B200_OK;
}

}  // namespace ob

using namespace ob;

extern "C" const char *ortho_b200_strerror(int status)
{
    switch (status) {
        case ORTHO_B200_OK: return "ok";
        case ORTHO_B200_ERR_NULL: return "a required pointer is NULL";
        case ORTHO_B200_ERR_SHAPE: return "unsupported shape (need M,N >= 1, K a multiple of 32 and <= 65536)";
        case ORTHO_B200_ERR_ALIGN: return "q_weight, x and y must be 16-byte aligned";
        case ORTHO_B200_ERR_PLAN: return "plan is invalid or was built for another layer";
        case ORTHO_B200_ERR_WORKSPACE: return "workspace missing or smaller than ortho_b200_workspace_bytes()";
        case ORTHO_B200_ERR_CUDA: return "a CUDA call failed (see ortho_b200_last_cuda_error)";
        case ORTHO_B200_ERR_DEVICE: return "current device is not a compute capability 10.x GPU";
        case ORTHO_B200_ERR_KERNEL: return "a kernel gave up on a bounded wait";
        case ORTHO_B200_ERR_ALLOC: return "allocation failed";
        case ORTHO_B200_ERR_SCRATCH_LIMIT: return "this shape needs more scratch than the built-in ORTHO_B200_STATIC_SCRATCH_BYTES array holds";
        default: return "unknown status";
    }
}

extern "C" int ortho_b200_version(void) { return ORTHO_B200_VERSION; }
extern "C" int ortho_b200_last_cuda_error(void) { return tl_last_cuda_error; }
extern "C" int64_t ortho_b200_launch_count(void) { return (int64_t)g_launches.load(); }

extern "C" int ortho_b200_set_decode_config(int row_groups, int k_groups, int unroll, int k_split)
{
    return set_decode_config(row_groups, k_groups, unroll, k_split);
}

extern "C" int ortho_b200_query_kernel_status(void)
{
    int *w = kernel_status_word();
    if (!w) return ORTHO_B200_ERR_CUDA;
    int h = 0;
    OB_CUDA(cudaMemcpy(&h, w, sizeof(int), cudaMemcpyDeviceToHost));
    if (h != 0) {
        int zero = 0;
        OB_CUDA(cudaMemcpy(w, &zero, sizeof(int), cudaMemcpyHostToDevice));
        return ORTHO_B200_ERR_KERNEL;
    }
    return ORTHO_B200_OK;
}

namespace ob {
int64_t prefill_min_workspace_bytes(int64_t M, int64_t K, int64_t N);
// scratch a forward with an active ortho term cannot do without
int64_t min_workspace_bytes(int64_t M, int64_t K, int64_t N)
{
    if (decode_regime(M, N, K)) return 0;          // the decode kernels use no global scratch
    return prefill_min_workspace_bytes(M, K, N);
}
}  // namespace ob

extern "C" int64_t ortho_b200_workspace_bytes(int64_t M, int64_t K, int64_t N)
{
    const int64_t other = decode_regime(M, N, K) ? 0 : prefill_workspace_bytes(M, K, N);
    if (!mid_token_range(M)) return other;
    const int64_t mid = mid_workspace_bytes(M, K, N);
    return mid > other ? mid : other;
}

namespace ob {
int forward_impl(const void *q_weight, const void *q_scales_f16,
                 const void *ortho_values_f16, const int32_t *ortho_col_indices,
                 const int32_t *ortho_row_ptr, int64_t nnz,
                 const void *x_f16, void *y_f16,
                 int64_t M, int64_t K, int64_t N, float alpha,
                 const ortho_b200_plan *plan,
                 void *workspace, int64_t workspace_bytes, void *stream,
                 int64_t ldy, const GatherView *gv, bool *gather_fused, const float *bias_f32)
{
    FwdArgs a;
    const int st = make_fwd_args(a, q_weight, q_scales_f16, ortho_values_f16, ortho_col_indices, ortho_row_ptr, nnz,
                                 x_f16, y_f16, M, K, N, alpha, plan, workspace, workspace_bytes, stream, ldy, bias_f32);
    if (st != ORTHO_B200_OK || M == 0) return st;
    a.gv = gv; a.gather_fused = gather_fused;
    return launch_routed(a);
}

int launch_routed(const FwdArgs &a)
{
    switch (route_of(a.M, a.N, a.K, a.workspace, a.workspace_bytes)) {
        case kRouteMid: return launch_mid(a);
        case kRouteDecode: return launch_decode(a);
        default: return launch_prefill(a);
    }
}

// validates one layer's arguments and fills the launchers' argument record
int make_fwd_args(FwdArgs &a, const void *q_weight, const void *q_scales_f16,
                  const void *ortho_values_f16, const int32_t *ortho_col_indices,
                  const int32_t *ortho_row_ptr, int64_t nnz,
                  const void *x_f16, void *y_f16,
                  int64_t M, int64_t K, int64_t N, float alpha,
                  const ortho_b200_plan *plan,
                  void *workspace, int64_t workspace_bytes, void *stream,
                  int64_t ldy, const float *bias_f32)
{
    if (M == 0) return ORTHO_B200_OK;
    if (!q_weight || !q_scales_f16 || !x_f16 || !y_f16) return ORTHO_B200_ERR_NULL;
    if (M < 0 || N <= 0 || K <= 0 || (K % 32) != 0 || K > 65536 || nnz < 0 ||
        M > 0x7fffffffLL || N > 0x7fffff00LL || nnz > 0x7fffffffLL)
        return ORTHO_B200_ERR_SHAPE;
    if ((((uintptr_t)q_weight | (uintptr_t)x_f16 | (uintptr_t)y_f16) & 15u) != 0) return ORTHO_B200_ERR_ALIGN;
    if (((uintptr_t)q_scales_f16 & 1u) != 0 || ((uintptr_t)bias_f32 & 3u) != 0) return ORTHO_B200_ERR_ALIGN;

    const Plan *pl = reinterpret_cast<const Plan *>(plan);
    if (pl) {
        if (pl->magic != kPlanMagic || pl->K != K || pl->N != N) return ORTHO_B200_ERR_PLAN;
        if (ortho_values_f16 && pl->nnz != nnz) return ORTHO_B200_ERR_PLAN;
        nnz = pl->nnz;
    }
    // the ortho stream is gated exactly like the reference: alpha > 0 and a non-empty list
    // (src/ortho.c:343, src/dual_gemm.cu:212)
    const bool has_ortho = (alpha > 0.0f) && (nnz > 0);
    if (has_ortho && !pl && (!ortho_values_f16 || !ortho_col_indices || !ortho_row_ptr)) return ORTHO_B200_ERR_NULL;

    int st = check_device();
    if (st != ORTHO_B200_OK) return st;

    a.w = (const uint8_t *)q_weight;
    a.scales = (const __half *)q_scales_f16;
    a.x = (const __half *)x_f16;
    a.y = (__half *)y_f16;
    a.bias = bias_f32;
    a.has_ortho = has_ortho ? 1 : 0;
    a.alpha = alpha;
    a.M = M; a.K = K; a.N = N; a.nnz = nnz;
    a.plan = pl;
    if (has_ortho && pl) {
        a.ortho.row_ptr = pl->row_ptr; a.ortho.entries = pl->entries; a.ortho.col = nullptr; a.ortho.val = nullptr;
    } else if (has_ortho) {
        a.ortho.row_ptr = ortho_row_ptr; a.ortho.entries = nullptr;
        a.ortho.col = ortho_col_indices; a.ortho.val = (const __half *)ortho_values_f16;
    } else {
        a.ortho.row_ptr = nullptr; a.ortho.entries = nullptr; a.ortho.col = nullptr; a.ortho.val = nullptr;
    }
    a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    a.stream = (cudaStream_t)stream;
    if (ldy != 0 && ldy < N) return ORTHO_B200_ERR_SHAPE;
    a.ldy = ldy; a.gv = nullptr; a.gather_fused = nullptr;
    return ORTHO_B200_OK;
}
}  // namespace ob

extern "C" int ortho_b200_forward(const void *q_weight, const void *q_scales_f16,
                                  const void *ortho_values_f16, const int32_t *ortho_col_indices,
                                  const int32_t *ortho_row_ptr, int64_t nnz,
                                  const void *x_f16, void *y_f16,
                                  int64_t M, int64_t K, int64_t N, float alpha,
                                  const ortho_b200_plan *plan,
                                  void *workspace, int64_t workspace_bytes, void *stream)
{
    return ob::forward_impl(q_weight, q_scales_f16, ortho_values_f16, ortho_col_indices, ortho_row_ptr, nnz,
                            x_f16, y_f16, M, K, N, alpha, plan, workspace, workspace_bytes, stream,
                            0, nullptr, nullptr, nullptr);
}

// Several layers that read the same activations (separate Q / K / V or gate / up projections): in the
// decode regime their tiles are walked by ONE persistent launch, so that the fixed cost of a launch
// (a few microseconds on layers that stream for 5-20) is paid once per group instead of once per layer;
// elsewhere the layers run one after the other on the stream.  The reference reaches the operator with
// one blocking launch per layer (src/dual_gemm.cu:317-346,366; torch_bind/ortho_linear.py:139-151).
extern "C" int ortho_b200_forward_multi(const ortho_b200_layer_desc *layers, int n_layers,
                                        const void *x_f16, int64_t M, int64_t K,
                                        void *workspace, int64_t workspace_bytes, void *stream)
{
    if (n_layers < 0 || (n_layers > 0 && !layers)) return ORTHO_B200_ERR_NULL;
    if (n_layers == 0 || M == 0) return ORTHO_B200_OK;
    if (n_layers > ORTHO_B200_MULTI_MAX_LAYERS) return ORTHO_B200_ERR_SHAPE;
    FwdArgs a[ORTHO_B200_MULTI_MAX_LAYERS];
    bool all_stream = true;
    for (int l = 0; l < n_layers; l++) {
        const ortho_b200_layer_desc &d = layers[l];
        const int st = make_fwd_args(a[l], d.q_weight, d.q_scales_f16, d.ortho_values_f16, d.ortho_col_indices,
                                     d.ortho_row_ptr, d.nnz, x_f16, d.y_f16, M, K, d.N, d.alpha, d.plan,
                                     workspace, workspace_bytes, stream, d.ldy, d.bias_f32);
        if (st != ORTHO_B200_OK) return st;
        all_stream = all_stream && route_of(M, d.N, K, workspace, workspace_bytes) == kRouteDecode && stream_kernel_selected(M, K);
    }
    if (all_stream && n_layers > 1) return launch_decode_multi(a, n_layers);
    for (int l = 0; l < n_layers; l++) {
        const int st = launch_routed(a[l]);
        if (st != ORTHO_B200_OK) return st;
    }
    return ORTHO_B200_OK;
}

extern "C" int64_t ortho_b200_multi_workspace_bytes(const ortho_b200_layer_desc *layers, int n_layers, int64_t M, int64_t K)
{
    int64_t need = 0;
    for (int l = 0; l < n_layers; l++) {
        const ortho_b200_layer_desc &d = layers[l];
        const int64_t w = d.plan ? ortho_b200_plan_workspace_bytes(d.plan, M) : ortho_b200_workspace_bytes(M, K, d.N);
        if (w < 0) return -1;
        need = w > need ? w : need;
    }
    return need;
}
