// Peer-mapped output buffers for the N-sharded layer and the forward that gathers through them.
//
// Every rank (one process per GPU) allocates one device buffer, exports its inter-process handle,
// and opens the handles of the other ranks; the [M, N_total] output of a forward lives at the same
// byte offset of every rank's buffer.  ortho_b200_forward_gather() computes this rank's column slice
// and leaves the complete output in every rank's buffer when the stream reaches the end of the call:
//   * M <= 16 (streaming decode kernel): the kernel's finalize step stores straight into all
//     ranks' buffers and its last CTA exchanges the completion flags -- one launch;
//   * M > 24 (tcgen05 kernel): its epilogue stores every finished output tile into all ranks'
//     buffers while the MMAs of the next tiles run, and its last CTA exchanges the flags -- one launch;
//   * what is left (17..32 tokens on small layers or without a workspace, K not a multiple of 256): the compute kernel writes the local
//     buffer, gather_push_kernel copies the slice to the peers and exchanges the flags.
// Peer memory is only ever touched by plain loads / stores of these kernels.
// The reference has no multi-device path; the layer-level partition this serves is the row
// independence of src/ortho.c:354-366,389-396.
#include <cstdio>
#include <cstring>
#include <new>

#include "common.cuh"
#include "gather.cuh"

namespace ob {

constexpr uint32_t kCommMagic = 0x0B200C03u;

struct Comm {
    uint32_t magic;
    int rank, world, device;
    int64_t bytes;                 // usable bytes (control block lies behind them)
    int64_t ctrl_off;
    unsigned char *base[kMaxRanks];   // base[rank] is the local allocation
    bool opened[kMaxRanks];
    bool connected;
    bool deferred;
    bool per_cta;         // signalling form, fixed when the comm is created (the two forms count differently)
    long long timeout_ns;
};

int *kernel_status_word();   // api.cu

// copies the [M][nloc] slice at y[rank] to the same place of every other rank, then flags
__global__ void __launch_bounds__(256)
gather_push_kernel(const GatherView gv, int M, int nloc, long long ldy, int *status)
{
    const __half *src = gv.y[gv.rank];
    const bool vec = (nloc % 8) == 0 && (ldy % 8) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
    if (vec) {
        const int cpr = nloc / 8;
        const long long total = (long long)M * cpr;
        for (long long i = tid; i < total; i += nth) {
            const long long m = i / cpr, c = i - m * cpr;
            const size_t at = (size_t)m * (size_t)ldy + (size_t)c * 8;
            const uint4 v = *reinterpret_cast<const uint4 *>(src + at);
            for (int r = 0; r < gv.world; r++)
                if (r != gv.rank) *reinterpret_cast<uint4 *>(gv.y[r] + at) = v;
        }
    } else {
        const long long total = (long long)M * nloc;
        for (long long i = tid; i < total; i += nth) {
            const long long m = i / nloc, c = i - m * nloc;
            const size_t at = (size_t)m * (size_t)ldy + (size_t)c;
            const __half v = src[at];
            for (int r = 0; r < gv.world; r++)
                if (r != gv.rank) gv.y[r][at] = v;
        }
    }
    if (!gather_signal_and_wait(gv, gridDim.x)) atomicExch(status, 2);
}

// deferred mode: waits for the peers' flags of this rank's last exchange (one thread)
__global__ void gather_wait_kernel(const GatherView gv, int *status)
{
    if (!gather_wait_previous(gv)) atomicExch(status, 2);
}

}  // namespace ob

using namespace ob;

static Comm *as_comm(const ortho_b200_comm *c)
{
    Comm *cm = reinterpret_cast<Comm *>(const_cast<ortho_b200_comm *>(c));
    return (cm && cm->magic == kCommMagic) ? cm : nullptr;
}

extern "C" int ortho_b200_comm_create(int rank, int world, int64_t bytes, ortho_b200_comm **out)
{
    if (!out) return ORTHO_B200_ERR_NULL;
    *out = nullptr;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || bytes <= 0) return ORTHO_B200_ERR_SHAPE;
    Comm *cm = new (std::nothrow) Comm();
    if (!cm) return ORTHO_B200_ERR_ALLOC;
    memset(cm, 0, sizeof(Comm));
    cm->magic = kCommMagic;
    cm->rank = rank; cm->world = world;
    cm->bytes = bytes;
    cm->ctrl_off = (bytes + 255) & ~(int64_t)255;
    cm->timeout_ns = 2000000000LL;
    cm->per_cta = tuning_snapshot().gather_per_cta;
    cudaError_t e = cudaGetDevice(&cm->device);
    unsigned char *p = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&p, (size_t)cm->ctrl_off + 256);
    if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)cm->ctrl_off + 256);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        if (p) cudaFree(p);
        delete cm;
        return e == cudaErrorMemoryAllocation ? ORTHO_B200_ERR_ALLOC : ORTHO_B200_ERR_CUDA;
    }
    cm->base[rank] = p;
    cm->connected = (world == 1);
    *out = reinterpret_cast<ortho_b200_comm *>(cm);
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_comm_export(const ortho_b200_comm *comm, void *handle)
{
    Comm *cm = as_comm(comm);
    if (!cm || !handle) return ORTHO_B200_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) <= ORTHO_B200_COMM_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    OB_CUDA(cudaIpcGetMemHandle(&h, cm->base[cm->rank]));
    memset(handle, 0, ORTHO_B200_COMM_HANDLE_BYTES);
    memcpy(handle, &h, sizeof(h));
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_comm_connect(ortho_b200_comm *comm, const void *handles)
{
    Comm *cm = as_comm(comm);
    if (!cm || !handles) return ORTHO_B200_ERR_NULL;
    if (cm->connected) return ORTHO_B200_OK;
    const unsigned char *hs = static_cast<const unsigned char *>(handles);
    for (int r = 0; r < cm->world; r++) {
        if (r == cm->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, hs + (size_t)r * ORTHO_B200_COMM_HANDLE_BYTES, sizeof(h));
        void *p = nullptr;
        OB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        cm->base[r] = static_cast<unsigned char *>(p);
        cm->opened[r] = true;
    }
    cm->connected = true;
    return ORTHO_B200_OK;
}

extern "C" void *ortho_b200_comm_local(const ortho_b200_comm *comm)
{
    Comm *cm = as_comm(comm);
    return cm ? cm->base[cm->rank] : nullptr;
}

extern "C" int ortho_b200_comm_set_timeout_ms(ortho_b200_comm *comm, int64_t ms)
{
    Comm *cm = as_comm(comm);
    if (!cm) return ORTHO_B200_ERR_NULL;
    if (ms <= 0 || ms > 600000) return ORTHO_B200_ERR_SHAPE;
    cm->timeout_ns = ms * 1000000LL;
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_comm_set_deferred(ortho_b200_comm *comm, int on)
{
    Comm *cm = as_comm(comm);
    if (!cm) return ORTHO_B200_ERR_NULL;
    cm->deferred = on != 0;
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_comm_wait(ortho_b200_comm *comm, void *stream)
{
    Comm *cm = as_comm(comm);
    if (!cm) return ORTHO_B200_ERR_NULL;
    if (!cm->connected) return ORTHO_B200_ERR_PLAN;
    if (cm->world <= 1 || !cm->deferred) return ORTHO_B200_OK;
    GatherView gv;
    memset(&gv, 0, sizeof(gv));
    gv.world = cm->world; gv.rank = cm->rank; gv.timeout_ns = cm->timeout_ns; gv.deferred = 1;
    gv.per_cta = cm->per_cta ? 1 : 0;
    for (int r = 0; r < cm->world; r++) gv.ctrl[r] = reinterpret_cast<GatherCtrl *>(cm->base[r] + cm->ctrl_off);
    int *status = kernel_status_word();
    if (!status) return ORTHO_B200_ERR_CUDA;
    gather_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(gv, status);
    OB_CUDA(cudaGetLastError());
    count_launch();
    return ORTHO_B200_OK;
}

extern "C" int ortho_b200_comm_destroy(ortho_b200_comm *comm)
{
    Comm *cm = as_comm(comm);
    if (!cm) return ORTHO_B200_ERR_NULL;
    int st = ORTHO_B200_OK;
    for (int r = 0; r < cm->world; r++) {
        if (r == cm->rank || !cm->opened[r]) continue;
        cudaError_t e = cudaIpcCloseMemHandle(cm->base[r]);
        if (e != cudaSuccess) { note_cuda_error(e); st = ORTHO_B200_ERR_CUDA; }
    }
    cudaError_t e = cudaFree(cm->base[cm->rank]);
    if (e != cudaSuccess) { note_cuda_error(e); st = ORTHO_B200_ERR_CUDA; }
    cm->magic = 0;
    delete cm;
    return st;
}

extern "C" int ortho_b200_forward_gather(const void *q_weight, const void *q_scales_f16,
                                         const void *ortho_values_f16, const int32_t *ortho_col_indices,
                                         const int32_t *ortho_row_ptr, int64_t nnz,
                                         const void *x_f16,
                                         int64_t M, int64_t K, int64_t N_local, float alpha,
                                         const ortho_b200_plan *plan,
                                         void *workspace, int64_t workspace_bytes,
                                         ortho_b200_comm *comm, int64_t y_offset_bytes,
                                         int64_t N_total, int64_t n_offset, void *stream)
{
    Comm *cm = as_comm(comm);
    if (!cm) return ORTHO_B200_ERR_NULL;
    if (!cm->connected) return ORTHO_B200_ERR_PLAN;
    if (M < 0 || N_local < 0 || N_total <= 0 || n_offset < 0 || n_offset + N_local > N_total || y_offset_bytes < 0)
        return ORTHO_B200_ERR_SHAPE;
    if ((y_offset_bytes & 15) != 0) return ORTHO_B200_ERR_ALIGN;
    if (y_offset_bytes + M * N_total * 2 > cm->bytes) return ORTHO_B200_ERR_WORKSPACE;
    if (M == 0) return ORTHO_B200_OK;

    GatherView gv;
    memset(&gv, 0, sizeof(gv));
    gv.world = cm->world; gv.rank = cm->rank; gv.timeout_ns = cm->timeout_ns;
    gv.deferred = cm->deferred ? 1 : 0;
    gv.per_cta = cm->per_cta ? 1 : 0;
    for (int r = 0; r < cm->world; r++) {
        gv.y[r] = reinterpret_cast<__half *>(cm->base[r] + y_offset_bytes) + n_offset;
        gv.ctrl[r] = reinterpret_cast<GatherCtrl *>(cm->base[r] + cm->ctrl_off);
    }
    int *status = kernel_status_word();
    if (!status) return ORTHO_B200_ERR_CUDA;

    bool fused = false;
    // deferred mode: the streaming decode kernel waits for the previous exchange itself; any other
    // kernel is preceded by the one-thread wait kernel
    const bool self_waits = N_local > 0 && stream_kernel_selected(M, K) &&
                            route_of(M, N_local, K, workspace, workspace_bytes) == kRouteDecode;
    if (cm->deferred && cm->world > 1 && !self_waits) {
        gather_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(gv, status);
        OB_CUDA(cudaGetLastError());
        count_launch();
    }
    if (N_local > 0) {
        // the slice is computed by the ordinary forward with the output pitch of the full matrix
        int st = ob::forward_impl(q_weight, q_scales_f16, ortho_values_f16, ortho_col_indices, ortho_row_ptr, nnz,
                                  x_f16, gv.y[cm->rank], M, K, N_local, alpha, plan, workspace, workspace_bytes,
                                  stream, N_total, &gv, &fused);
        if (st != ORTHO_B200_OK) return st;
    }
    if (!fused && cm->world > 1) {
        const long long work = (long long)M * (N_local > 0 ? N_local : 1) / 8;
        int blocks = (int)((work + 255) / 256);
        if (blocks < 1) blocks = 1;
        if (blocks > 148) blocks = 148;    // all CTAs co-resident: the last one to finish exchanges the flags
        gather_push_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(gv, (int)M, (int)N_local, (long long)N_total, status);
        OB_CUDA(cudaGetLastError());
        count_launch();
    }
    return ORTHO_B200_OK;
}
