/*
 * ortho_b200 -- C ABI of the B200 (sm_100a) OrthoLinear forward
 *
 *     Y[M,N] = X[M,K] . dequant(W_base_int4[N,K])^T  +  alpha . X[M,K] . W_ortho[N,K]^T
 *
 * Plain pointers and sizes only; no C++ or torch types.  Every pointer is a DEVICE pointer
 * unless a comment says "host".  `stream` is a cudaStream_t passed as void* (NULL = the legacy
 * default stream).  All calls are asynchronous on `stream` and perform no host synchronisation
 * except where stated.  Every function returns ORTHO_B200_OK (0) or a positive status code;
 * nothing traps on the device.
 *
 * Weight layout (kept from the reference, include/ortho.h:22-28,41-53,63-71):
 *   q_weight   u8  [N, K/2] row-major; element idx = n*K + k lives in byte idx/2, low nibble for
 *              even idx, high nibble for odd; nibble = 4-bit two's complement in [-8, 7]
 *              (src/ortho.c:315-325)
 *   q_scales   f16 [N]   one scale per output row (module buffer, torch_bind/ortho_linear.py:60)
 *   CSR ortho  row_ptr i32 [N+1], col_indices i32 [nnz] (row-major sorted, unique),
 *              values f16 [nnz]            (torch_bind/ortho_linear.py:63-65, tools/sieve.py:119-152)
 *   alpha      float kill switch; the ortho term contributes only when alpha > 0 and nnz > 0
 *              (src/ortho.c:343)
 *   X f16 [M,K] row-major contiguous, Y f16 [M,N] row-major contiguous (ortho_linear.py:130-168)
 *
 * Constraints (violations return a status, there is no slow path): K a multiple of 32,
 * K <= 65536, q_weight / X / Y 16-byte aligned, M, N >= 1 (M == 0 is a no-op).
 */
#ifndef ORTHO_B200_H
#define ORTHO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORTHO_B200_VERSION 100

#if defined(__GNUC__)
#define ORTHO_B200_API __attribute__((visibility("default")))
#else
#define ORTHO_B200_API
#endif

enum {
    ORTHO_B200_OK = 0,
    ORTHO_B200_ERR_NULL = 1,        /* a required pointer is NULL                                  */
    ORTHO_B200_ERR_SHAPE = 2,       /* M/K/N/nnz outside the supported range (K%32, K<=65536, ...) */
    ORTHO_B200_ERR_ALIGN = 3,       /* a base pointer is not 16-byte aligned                       */
    ORTHO_B200_ERR_PLAN = 4,        /* plan does not belong to this layer (shape or nnz mismatch)  */
    ORTHO_B200_ERR_WORKSPACE = 5,   /* workspace missing or smaller than ortho_b200_workspace_bytes */
    ORTHO_B200_ERR_CUDA = 6,        /* a CUDA call failed; see ortho_b200_last_cuda_error()        */
    ORTHO_B200_ERR_DEVICE = 7,      /* the current device is not compute capability 10.x           */
    ORTHO_B200_ERR_KERNEL = 8,      /* a kernel reported a bounded wait that ran out               */
    ORTHO_B200_ERR_ALLOC = 9,       /* host or device allocation failed                            */
    ORTHO_B200_ERR_SCRATCH_LIMIT = 10 /* needs more scratch than ORTHO_B200_STATIC_SCRATCH_BYTES   */
};

/* Replaces: the 0 / -1 convention of the reference C API (include/ortho.h:76-79,132-135). */
ORTHO_B200_API const char *ortho_b200_strerror(int status);
ORTHO_B200_API int ortho_b200_version(void);
/* cudaError_t value recorded by the last call on this host thread that returned ERR_CUDA. */
ORTHO_B200_API int ortho_b200_last_cuda_error(void);

/* ---------------------------------------------------------------------------------------------
 * Plan: the GPU-side re-layout of one layer's sparse ortho component, built once per layer.
 * Has no counterpart in the reference (its kernels read CSR directly,
 * src/dual_gemm.cu:106-130); it takes the place of the per-call orth_layer_t the binding builds
 * on its stack (torch_bind/bindings.cpp:19-36).  The plan owns only its own device copies
 * (packed {col16|f16 value} entries in row order, row pointers, the list of long rows and their dense FP16 copy);
 * it never retains the caller's pointers.  Creation allocates device memory, launches the
 * re-layout kernels on `stream` and synchronises that stream once.  A plan is immutable after
 * creation and may be shared by concurrent forwards.  nnz == 0 yields a valid empty plan.
 * ------------------------------------------------------------------------------------------- */
typedef struct ortho_b200_plan ortho_b200_plan;

ORTHO_B200_API int ortho_b200_plan_create(ortho_b200_plan **plan_out,
                           const int32_t *row_ptr, const int32_t *col_indices,
                           const void *values_f16, int64_t nnz,
                           int64_t in_features, int64_t out_features, void *stream);
ORTHO_B200_API int ortho_b200_plan_destroy(ortho_b200_plan *plan);
ORTHO_B200_API int64_t ortho_b200_plan_nnz(const ortho_b200_plan *plan);
/* largest number of stored entries in one output row (host value cached at creation) */
ORTHO_B200_API int64_t ortho_b200_plan_max_row_nnz(const ortho_b200_plan *plan);
/* 1 when every row lists its columns in strictly ascending order inside [0, in_features) (what
 * tools/sieve.py:131-136 produces), 0 otherwise, -1 for an invalid handle.  Only such plans let the tensor-core
 * kernels fold the sparse entries into their weight tiles; any other plan takes the gather path. */
ORTHO_B200_API int ortho_b200_plan_rows_ordered(const ortho_b200_plan *plan);

/* Decodes the re-laid-out entries back to (row, col, f16 value) triplets, entry i of the plan
 * to slot i of the outputs (each sized nnz).  Exists so that a test can prove the sparse index
 * decode bit-exact against the CSR arrays (row-major order, tools/sieve.py:131-136). */
ORTHO_B200_API int ortho_b200_plan_decode_dump(const ortho_b200_plan *plan, int32_t *rows_out, int32_t *cols_out,
                                void *values_f16_out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Bit-exactness probe for the base: writes, for every element, the raw integer produced by the
 * same in-register INT4 unpack the forward kernels use, and (float)w_int * (float)scale[n].
 * Follows src/ortho.c:315-325 (unpack) and :363 (scale application).  Either output may be NULL.
 * ------------------------------------------------------------------------------------------- */
ORTHO_B200_API int ortho_b200_dequant_dump(const void *q_weight, const void *q_scales_f16,
                            int64_t out_features, int64_t in_features,
                            int8_t *w_int_out, float *w_deq_out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Forward.  Replaces orth_layer_forward_cuda (include/ortho.h:141-144, src/dual_gemm.cu:295-372)
 * as reached from the binding's forward(q_weight, q_scales, ortho_values, ortho_col_indices,
 * ortho_row_ptr, input, output, alpha) (torch_bind/bindings.cpp:9-18, call site
 * torch_bind/ortho_linear.py:142-151); same argument order and meaning, plus explicit sizes,
 * the optional plan, a caller-owned workspace and the stream.
 *
 *   M <= 16   : memory-bound streaming kernels; also M <= 32 on layers of at most 4096 x 4096 weights, and, for
 *               calls without a workspace, M <= 24, M <= 32 with N <= 4096 and M <= 64 with N <= 1024 while
 *               N * K <= 4096 * 8192 (ORTHO_B200_DECODE_MAX_M is the most these kernels accept).  No global scratch.
 *   17 .. 128 : tcgen05 kernel with the token block as the MMA's M operand (256 weight rows per instruction),
 *               taken when the call brings ortho_b200_workspace_bytes(M, K, N) bytes of workspace, whatever alpha
 *               is; without it the call runs the kernel of the neighbouring regime.  With a plan whose rows are in
 *               column order and that lists no long rows, the sparse entries are folded into its weight tile.
 *   larger M  : tcgen05 / TMEM prefill kernel (weight tile as the M operand).  With an active ortho term
 *               (alpha > 0 and nnz > 0) and a plan whose rows are in column order the entries are folded into the
 *               weight tile, and the workspace is needed only when the plan lists long rows (their tensor-core
 *               pre-pass sums; same size and layout as below); without such a plan the kernel gathers the term and
 *               needs the workspace for the transposed activations.  Missing workspace that is needed:
 *               ERR_WORKSPACE.  Otherwise the workspace is optional (split-K of the last wave).
 * Size the workspace with ortho_b200_workspace_bytes / ortho_b200_plan_workspace_bytes and pass it, 256-byte
 * aligned, whenever that is not 0.  The first forward of a kernel variant on a device sets function attributes:
 * issue it outside any stream capture.
 * plan may be NULL: the kernels then read the CSR arrays directly.  With a plan the CSR
 * pointers may be NULL.  alpha <= 0 or nnz == 0 skips the sparse stream entirely, so the output
 * is bit-identical to the base-only result (src/ortho.c:343 and the reference null test,
 * tests/benchmark_null_test.c:127-131).  Borrowed pointers are only used until the launched
 * kernels finish.
 * ------------------------------------------------------------------------------------------- */
#define ORTHO_B200_DECODE_MAX_M 64

ORTHO_B200_API int64_t ortho_b200_workspace_bytes(int64_t M, int64_t K, int64_t N);
/* Workspace for forwards that pass this plan (the prefill regime keeps the pre-pass sums of the plan's long rows
 * there, so it may need more than the plan-less bound); 0 for the streaming kernels or for an empty plan. */
ORTHO_B200_API int64_t ortho_b200_plan_workspace_bytes(const ortho_b200_plan *plan, int64_t M);

ORTHO_B200_API int ortho_b200_forward(const void *q_weight, const void *q_scales_f16,
                       const void *ortho_values_f16, const int32_t *ortho_col_indices,
                       const int32_t *ortho_row_ptr, int64_t nnz,
                       const void *x_f16, void *y_f16,
                       int64_t M, int64_t K, int64_t N, float alpha,
                       const ortho_b200_plan *plan,
                       void *workspace, int64_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Forward of several layers that share the activations, with an optional bias per layer.
 *
 * Takes the place of (a) one operator call per projection where a model keeps Q / K / V or gate / up as
 * separate layers -- the reference launches and synchronises once per layer
 * (src/dual_gemm.cu:317-346,366; call site torch_bind/ortho_linear.py:139-151) -- and (b) the separate
 * element-wise `output += bias` after the kernel (torch_bind/ortho_linear.py:71-74,164-166): bias_f32
 * (FP32 [N], may be NULL) is added in the kernels' FP32 epilogue before the single FP16 rounding.
 * Every layer has its own alpha (the reference's kill switch, per layer).  All layers read x [M, K];
 * layer l writes y_f16 [M, N] with row pitch ldy (0 = N).  For M <= 16 and K a multiple of 256 the tiles
 * of all layers are walked by one persistent kernel launch; otherwise the layers run one after the other on
 * the stream, sharing the workspace (ortho_b200_multi_workspace_bytes = the largest any of them needs).
 * n_layers <= ORTHO_B200_MULTI_MAX_LAYERS.  n_layers == 1 is the ordinary forward plus the bias.
 * ------------------------------------------------------------------------------------------- */
#define ORTHO_B200_MULTI_MAX_LAYERS 4
typedef struct ortho_b200_layer_desc {
    const void *q_weight;               /* u8  [N, K/2] */
    const void *q_scales_f16;           /* f16 [N] */
    const void *ortho_values_f16;       /* f16 [nnz]   (may be NULL with a plan or when nnz == 0) */
    const int32_t *ortho_col_indices;   /* i32 [nnz] */
    const int32_t *ortho_row_ptr;       /* i32 [N+1] */
    int64_t nnz;
    const ortho_b200_plan *plan;        /* optional */
    const float *bias_f32;              /* optional FP32 [N] */
    void *y_f16;                        /* f16 [M, N], row pitch ldy */
    int64_t N;
    int64_t ldy;                        /* elements between token rows of y; 0 = N */
    float alpha;
    int32_t reserved;                   /* set to 0 */
} ortho_b200_layer_desc;

ORTHO_B200_API int64_t ortho_b200_multi_workspace_bytes(const ortho_b200_layer_desc *layers, int n_layers, int64_t M, int64_t K);
ORTHO_B200_API int ortho_b200_forward_multi(const ortho_b200_layer_desc *layers, int n_layers,
                       const void *x_f16, int64_t M, int64_t K,
                       void *workspace, int64_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Forward for callers that cannot allocate device memory.  It has no counterpart in the reference.
 *
 * Who needs it: code that runs where cudaMalloc must not be called -- a host application that owns
 * the allocator and hands a plugin only tensors, a serving loop whose memory was fixed at start-up,
 * or a section that is about to be recorded into a CUDA graph.  ortho_b200_forward asks such a
 * caller for a workspace in the tensor-core regimes, and a plan has to be allocated too.  This entry
 * point takes neither: it reads the CSR arrays directly and keeps the scratch in a fixed array of
 * ORTHO_B200_STATIC_SCRATCH_BYTES that is part of the library image.  Every GPU that loads the
 * library holds that array until the process exits.  It picks the kernel exactly as ortho_b200_forward
 * does when given a workspace of that size, so both entries produce the same bits.
 *
 * Limits and rules:
 *  - the one case it refuses (ORTHO_B200_ERR_SCRATCH_LIMIT, nothing launched) is a prefill-regime call
 *    with an active ortho term whose transposed activations, K * roundup(M, 256) * 2 bytes, exceed
 *    ORTHO_B200_STATIC_SCRATCH_BYTES; alpha <= 0, nnz == 0 and the streaming regime need no scratch;
 *  - the first call on a device looks up the array's device address (cudaGetSymbolAddress, no
 *    allocation); make that first call before any stream capture begins;
 *  - all calls share the one array and it keeps the previous call's contents.  Nothing in it needs
 *    clearing by the caller (each call writes what it later reads; the flag words of split tiles are
 *    cleared on the stream by the call itself), but calls that overlap on the GPU -- other streams,
 *    other host threads -- race on it: issue them one after another on one stream;
 *  - no cudaMalloc / cudaFree or any other allocating call is made.
 * Arguments as for ortho_b200_forward, without plan and workspace.
 * ------------------------------------------------------------------------------------------- */
#define ORTHO_B200_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

ORTHO_B200_API int ortho_b200_forward_static_scratch(const void *q_weight, const void *q_scales_f16,
                       const void *ortho_values_f16, const int32_t *ortho_col_indices,
                       const int32_t *ortho_row_ptr, int64_t nnz,
                       const void *x_f16, void *y_f16,
                       int64_t M, int64_t K, int64_t N, float alpha, void *stream);

/* ---------------------------------------------------------------------------------------------
 * N-sharded layer: output all-gather through peer-mapped buffers (one process per GPU).
 * The reference has no multi-device path; this is the exchange step a tensor-parallel caller needs
 * after sharding the layer over output rows (rows are independent: src/ortho.c:354-366,389-396).
 *
 * comm_create   allocates `bytes` of device memory on the current device for rank `rank` of `world`
 *               (world <= 8) plus a small control block.
 * comm_export   writes this rank's inter-process handle (ORTHO_B200_COMM_HANDLE_BYTES bytes); the
 *               caller exchanges the handles of all ranks by any means (e.g. an all-gather on the host).
 * comm_connect  opens the other ranks' buffers; `handles` = world handles in rank order.
 * comm_local    device pointer of the local buffer: the gathered outputs appear there.
 * forward_gather computes this rank's N_local output columns (arguments as ortho_b200_forward, the
 *               weights being the rank's row shard) and stores them at columns
 *               [n_offset, n_offset + N_local) of the [M, N_total] FP16 matrix that starts
 *               y_offset_bytes into EVERY rank's buffer.  When the stream reaches the end of the call
 *               all ranks' slices of this forward are present in the local buffer.  Every rank must
 *               issue the same sequence of forward_gather calls on a comm; a buffer region may be
 *               reused by the second next call at the earliest (alternate two regions).  For M <= 16
 *               and for M > 24 the peer stores and the flag exchange are part of the compute kernel
 *               itself; the shapes in between add one copy kernel.  A rank whose peers do not arrive within the timeout
 *               (default 2 s) records a kernel status (ortho_b200_query_kernel_status) and returns.
 *               n_offset must be a multiple of 8; y_offset_bytes a multiple of 16.
 * ------------------------------------------------------------------------------------------- */
typedef struct ortho_b200_comm ortho_b200_comm;
#define ORTHO_B200_COMM_HANDLE_BYTES 64
#define ORTHO_B200_COMM_MAX_RANKS 8

ORTHO_B200_API int ortho_b200_comm_create(int rank, int world, int64_t bytes, ortho_b200_comm **out);
ORTHO_B200_API int ortho_b200_comm_export(const ortho_b200_comm *comm, void *handle);
ORTHO_B200_API int ortho_b200_comm_connect(ortho_b200_comm *comm, const void *handles);
ORTHO_B200_API void *ortho_b200_comm_local(const ortho_b200_comm *comm);
ORTHO_B200_API int ortho_b200_comm_set_timeout_ms(ortho_b200_comm *comm, int64_t ms);
/* Deferred mode (off by default): a forward_gather only signals its own exchange; the NEXT
 * forward_gather on the same comm waits for it after its own weight prefetch and before it reads
 * its input, which hides the flag latency of a chain of layers.  Any other consumer of a gathered
 * output must be preceded by ortho_b200_comm_wait(comm, stream).  Set identically on every rank. */
ORTHO_B200_API int ortho_b200_comm_set_deferred(ortho_b200_comm *comm, int on);
ORTHO_B200_API int ortho_b200_comm_wait(ortho_b200_comm *comm, void *stream);
ORTHO_B200_API int ortho_b200_comm_destroy(ortho_b200_comm *comm);
ORTHO_B200_API int ortho_b200_forward_gather(const void *q_weight, const void *q_scales_f16,
                       const void *ortho_values_f16, const int32_t *ortho_col_indices,
                       const int32_t *ortho_row_ptr, int64_t nnz,
                       const void *x_f16,
                       int64_t M, int64_t K, int64_t N_local, float alpha,
                       const ortho_b200_plan *plan,
                       void *workspace, int64_t workspace_bytes,
                       ortho_b200_comm *comm, int64_t y_offset_bytes,
                       int64_t N_total, int64_t n_offset, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Device-side packer: produces the buffers the forward consumes from FP32 weights that are already
 * on the GPU.  Replaces the torch chain of OrthoLinear.load_from_weights
 * (torch_bind/ortho_linear.py:79-128) and pack_ortho_sparse(..., "csr") (tools/sieve.py:119-152),
 * with bit-identical results:
 *   pack_base : scales = max(rowmax|W| / 7, 1e-6) unless scales_in (FP32, [N]) is given;
 *               w_int = clamp(round_half_even(W / scale), -8, 7); two per byte, even index low.
 *               Writes q_weight_out [N, K/2] and q_scales_f16_out [N].  K a multiple of 8.
 *   csr_count : row_ptr_out [N+1] of the positions with W_ortho != 0 (row_ptr_out[N] = nnz;
 *               read it back to size the next call's outputs).
 *   csr_fill  : col_out / val_f16_out [nnz] in row-major order, values rounded to FP16.
 * W and W_ortho are [N, K] FP32, row-major, 16-byte aligned.
 * ------------------------------------------------------------------------------------------- */
ORTHO_B200_API int ortho_b200_pack_base(const float *w, int64_t N, int64_t K, const float *scales_in,
                       void *q_weight_out, void *q_scales_f16_out, void *stream);
ORTHO_B200_API int ortho_b200_csr_count(const float *w_ortho, int64_t N, int64_t K, int32_t *row_ptr_out, void *stream);
ORTHO_B200_API int ortho_b200_csr_fill(const float *w_ortho, int64_t N, int64_t K, const int32_t *row_ptr,
                       int32_t *col_out, void *val_f16_out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Device-side Hessian sieve: splits FP32 weights W [N, K] that are already on the GPU into the
 * INT4-representable base and the sparse residual, bit-identical to hessian_sieve / quantize_int4 of
 * the reference (tools/sieve.py:13-23, 25-76):
 *   base  = clamp(round_half_even(W / s), -8, 7) * s with s = max(rowmax|W|, 1e-8) / 7
 *   ortho = (W - base) where (W - base)^2 / (h_inv_diag[k] + 1e-6) > threshold, else (signed) zero
 * keep_top_k < 0: threshold = curvature_thresh.  keep_top_k >= 0: threshold = the keep_top_k-th largest
 * score (the caller passes int(sparsity_target * N * K); 0 keeps nothing), found on the device by a
 * byte-wise radix select without storing the scores.  h_inv_diag is the FP32 [K] diagonal.  scratch:
 * ortho_b200_sieve_scratch_bytes(N) bytes, 256-byte aligned.  K a multiple of 4, pointers 16-byte aligned.
 * The outputs feed ortho_b200_pack_base / ortho_b200_csr_count / ortho_b200_csr_fill.
 * ------------------------------------------------------------------------------------------- */
ORTHO_B200_API int64_t ortho_b200_sieve_scratch_bytes(int64_t N);
ORTHO_B200_API int ortho_b200_sieve(const float *w, const float *h_inv_diag, int64_t N, int64_t K,
                       float curvature_thresh, int64_t keep_top_k,
                       float *w_base_out, float *w_ortho_out,
                       void *scratch, int64_t scratch_bytes, void *stream);

/* Synchronises the device and reports whether any kernel of this library gave up on a bounded
 * wait since the last query (ERR_KERNEL, and the flag is cleared) or not (OK).  Replaces the
 * cudaDeviceSynchronize + error check at the end of the reference dispatcher
 * (src/dual_gemm.cu:361-371), as an explicit call instead of a cost on every forward. */
ORTHO_B200_API int ortho_b200_query_kernel_status(void);

/* Benchmark/tuning hook: overrides the decode kernels' tiling for forwards that START after the call
 * returns, from any thread of this process (the state sits behind a lock; a forward uses the
 * snapshot it took on entry).
 *   row_groups > 0 : generic kernel with (row groups per CTA, k groups per CTA, loads in flight,
 *                    k split over the cluster);
 *   row_groups == -1: streaming TMA kernel (M <= 16) with k_split CTAs per cluster and `unroll`
 *                    ring slots per warp (either may be 0 for the built-in choice);
 *   row_groups == -3: forwards with more than k_split tokens (0..ORTHO_B200_DECODE_MAX_M) use the
 *                    tensor-core kernels (built-in: 24);
 *   row_groups == -4: forwards with unroll < tokens <= k_split (<= 128) use the tokens-as-M tensor-core kernel
 *                    before any other rule (unroll == k_split: never); 0, 0 restores the built-in rule;
 *   row_groups == -5: plans created after the call treat rows of more than max(k_split, 4 x the mean row)
 *                    entries as long rows (8..65536; 0 restores the built-in 64);
 *   row_groups == -6: k_split = 0 makes the tensor-core kernels compute the sparse term as gathers from the
 *                    transposed activations even when the plan's rows are in column order; 1 restores the
 *                    built-in behaviour (entries folded into the weight tile);
 *   row_groups == -7: k_split = 1 makes comms created after the call use per-CTA signalling in the peer exchange
 *                    (every CTA adds itself to a counter on every peer once its stores are out) instead of one
 *                    flag raised by the grid's last CTA; all ranks of a group must use the same setting;
 *   row_groups == 0 : restore the built-in choice of kernel and tiling (not the -3 ... -7 settings).
 * Returns ERR_SHAPE for an unsupported tuple. */
ORTHO_B200_API int ortho_b200_set_decode_config(int row_groups, int k_groups, int unroll, int k_split);

/* Number of kernel launches issued by this library from this process (all threads). */
ORTHO_B200_API int64_t ortho_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ORTHO_B200_H */
