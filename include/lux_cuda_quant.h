/*
 * lux_cuda_quant.h -- C ABI of libluxgpu_backend_cuda.so beyond the base vtable.
 *
 * The plugin is a drop-in backend for the Lux GPU core: it exports
 * `lux_gpu_backend_init` (include/lux/gpu/backend_plugin.h:423-445) and fills
 * the unchanged 64-slot `lux_gpu_backend_vtbl` (backend_plugin.h:82-382),
 * ABI version 2 (backend_plugin.h:24).  The base vtable has no slot for a
 * quantized matmul, so the entry points of that path are published, without
 * touching the header, in three additive ways:
 *
 *   (i)   `vtbl->_reserved[0]` (backend_plugin.h:379-380, "reserved for future
 *         expansion") holds a `const lux_gpu_quant_vtbl*`; other backends leave
 *         it NULL, and cores that do not know it never read it;
 *   (ii)  the exported getter `lux_gpu_cuda_quant_vtbl()` returns the same table
 *         (for `dlsym`);
 *   (iii) `kernel_load(ctx, NULL, "lux.qmm.affine")` + `kernel_dispatch` with
 *         the buffer list {x, wq, scales, biases, y, params} reaches the same
 *         code through the existing custom-kernel slots
 *         (backend_plugin.h:103-114); `params` is a `lux_qmm_params` buffer.
 *
 * Every function mirrors the argument shape of the nearest base op,
 * `op_matmul_f32(ctx, a, b, out, M, K, N)` (backend_plugin.h:129; CPU
 * implementation src/cpu_backend.cpp:243-266): context first, input buffers,
 * output buffer, then dimensions.  All work is enqueued on the context's
 * stream; `sync` / `buffer_copy_to_host` of the base vtable order after it.
 * Errors are `LuxBackendError` values (backend_plugin.h:49-56); nothing throws
 * or aborts across this boundary and there is no CPU fallback: on a machine
 * without a usable GPU `lux_gpu_backend_init` returns false.
 *
 * Packed format (w^ = scale*q + bias per group along K):
 *   wq      uint32[N][K*bits/32], LSB-first along K
 *             4-bit: q[n][k] = (wq[n][k>>3] >> (4*(k&7))) & 0xF
 *             8-bit: q[n][k] = (wq[n][k>>2] >> (8*(k&3))) & 0xFF
 *   scales, biases  [N][K/group]  (fp32 or bf16), group in {32, 64, 128}
 *   y[m][n] = sum_k x[m][k] * w^[n][k]
 * Supported dtype combinations (x, scales/biases) -> w^ precision:
 *   (F32, F32|BF16): w^ = fl32(fl32(s*q)+b), fp32 math, fp32 accumulate
 *   (BF16, BF16)   : w^ = RNE_bf16(exact s*q+b) (one bf16 FMA), fp32 accumulate
 *   y may be F32 or BF16 (RNE of the fp32 sum).  (BF16, F32) is NOT_SUPPORTED.
 */
#ifndef LUX_CUDA_QUANT_H
#define LUX_CUDA_QUANT_H

#include "lux/gpu/backend_plugin.h"
#include "lux/gpu/kernel_loader.h"

#ifdef __cplusplus
extern "C" {
#endif

#define LUX_CUDA_QUANT_MAGIC 0x4C515854u /* "LQXT" */
#define LUX_CUDA_PRO_RMS_NORM 1
#define LUX_CUDA_PRO_SUM3 2
#define LUX_CUDA_QUANT_VERSION 7u /* 2: symm_* and qmatmul_sharded_push appended; 3: sum3, mul_rms_norm; 4: qmatmul_pro; 5: qmatmul_batch; 6: qmatmul_sharded_push_batch; 7: qmatmul_sharded_push_pro */
#define LUX_CUDA_QMM_KERNEL_NAME "lux.qmm.affine"
#define LUX_CUDA_NCCL_UID_BYTES 128

/* parameter block of the kernel_dispatch route (iii); 32 bytes */
typedef struct lux_qmm_params {
    int32_t M, K, N, bits, group, x_dtype, sb_dtype, y_dtype;
} lux_qmm_params;

/* One rank of a column-sharded layer (see shard_* below). */
typedef struct LuxCudaShardComm LuxCudaShardComm;
/* One rank's copy of a buffer that its peers can store into (see symm_*). */
typedef struct LuxCudaSymmBuffer LuxCudaSymmBuffer;
#define LUX_CUDA_SYMM_HANDLE_BYTES 96
/* A recorded sequence of calls on one context (see graph_*). */
typedef struct LuxCudaGraph LuxCudaGraph;

typedef struct lux_gpu_quant_vtbl {
    uint32_t magic;   /* LUX_CUDA_QUANT_MAGIC */
    uint32_t version; /* LUX_CUDA_QUANT_VERSION */
    uint32_t size;    /* sizeof(lux_gpu_quant_vtbl) of the library that filled it */
    uint32_t _pad;

    /* y[M,N] = x[M,K] . dequant(wq[N,K])^T.  M <= 16 runs the decode GEMV
     * kernels, larger M the tcgen05 GEMM.  Replaces (for quantized weights)
     * op_matmul_f32, backend_plugin.h:129 / src/cpu_backend.cpp:243-266. */
    LuxBackendError (*qmatmul)(LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* wq,
                               LuxBackendBuffer* scales, LuxBackendBuffer* biases, LuxBackendBuffer* y,
                               int M, int K, int N, int bits, int group,
                               LuxBackendDtype x_dtype, LuxBackendDtype sb_dtype, LuxBackendDtype y_dtype);

    /* out[N,K] = dequant(wq): F32 (two-rounding rule) or BF16 (single-rounding
     * rule).  Exists so the dequantised weights can be checked bit for bit.
     * No counterpart in the reference (it has no quantized format). */
    LuxBackendError (*dequantize)(LuxBackendContext* ctx, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                                  LuxBackendBuffer* biases, LuxBackendBuffer* out, int N, int K, int bits,
                                  int group, LuxBackendDtype sb_dtype, LuxBackendDtype out_dtype);

    /* q[N,K] (one byte per element) = unpack(wq).  Bit-exact check of the packing. */
    LuxBackendError (*unpack)(LuxBackendContext* ctx, LuxBackendBuffer* wq, LuxBackendBuffer* q_out,
                              int N, int K, int bits);

    /* Affine min/max quantiser, the producer of the format: w fp32 [N,K] ->
     * (wq, scales, biases).  No counterpart in the reference. */
    LuxBackendError (*quantize)(LuxBackendContext* ctx, LuxBackendBuffer* w, LuxBackendBuffer* wq,
                                LuxBackendBuffer* scales, LuxBackendBuffer* biases, int N, int K, int bits,
                                int group, LuxBackendDtype sb_dtype);

    /* Row-wise rms-norm with unit or given weight, fp32 math, in/out dtype
     * F32 or BF16.  Formula of op_rms_norm_f32 (backend_plugin.h:178;
     * kernels/cpu/tensor_ops.c:546-566). weight may be NULL. */
    LuxBackendError (*rms_norm)(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out,
                                LuxBackendBuffer* weight, size_t rows, size_t dim, float eps,
                                LuxBackendDtype in_dtype, LuxBackendDtype out_dtype);

    /* --- buffer interop ---------------------------------------------------- */
    /* Device address of a buffer (valid until buffer_free). */
    void* (*buffer_device_ptr)(LuxBackendContext* ctx, LuxBackendBuffer* buf);
    /* Size in bytes the buffer was allocated with. */
    size_t (*buffer_size)(LuxBackendContext* ctx, LuxBackendBuffer* buf);
    /* Non-owning buffer around device memory that someone else allocated on the
     * context's device (buffer_free releases only the handle). */
    LuxBackendBuffer* (*buffer_wrap)(LuxBackendContext* ctx, void* device_ptr, size_t bytes);
    /* Stream-ordered host->device copy that does NOT wait: `src` must be pinned
     * and stay untouched until the next sync.  buffer_copy_from_host of the
     * base vtable keeps the reference's blocking semantics
     * (src/cpu_backend.cpp:155-160). */
    LuxBackendError (*buffer_copy_from_host_async)(LuxBackendContext* ctx, LuxBackendBuffer* buf,
                                                   const void* src, size_t bytes);
    /* Pinned host memory for the two copies above. */
    void* (*host_alloc_pinned)(size_t bytes);
    void (*host_free_pinned)(void* p);
    /* The context's CUDA stream (a cudaStream_t), for callers that enqueue their own work. */
    void* (*context_stream)(LuxBackendContext* ctx);
    /* Allocator statistics of the context's device: bytes held from the
     * driver, bytes handed out, number of driver allocations so far. */
    LuxBackendError (*allocator_stats)(LuxBackendContext* ctx, uint64_t* reserved, uint64_t* in_use,
                                       uint64_t* driver_allocs);
    /* Return cached, unused device memory to the driver. */
    LuxBackendError (*allocator_trim)(LuxBackendContext* ctx);

    /* --- device-side timing (CUDA events on the context's stream) ----------- */
    /* slot 0..15; elapsed_ms synchronises on the stop event. */
    LuxBackendError (*timer_record)(LuxBackendContext* ctx, int slot);
    LuxBackendError (*timer_elapsed_ms)(LuxBackendContext* ctx, int start_slot, int stop_slot, float* ms);
    /* Write `bytes` (> L2) of the context's flush buffer so the next kernel
     * starts with a cold L2. */
    LuxBackendError (*flush_l2)(LuxBackendContext* ctx);
    /* Name of the kernel the last qmatmul on this context launched, number of
     * kernels launched by the plugin on this context so far. */
    const char* (*last_kernel)(LuxBackendContext* ctx);
    uint64_t (*launch_count)(LuxBackendContext* ctx);

    /* --- CUDA graphs over the context's stream ------------------------------ */
    /* Calls made on the context between graph_begin and graph_end are recorded
     * instead of run (no sync / copy_to_host in between; run each shape once
     * eagerly first so workspaces exist).  graph_launch replays them
     * stream-ordered.  The reference has no counterpart (its stream API is a
     * stub, src/gpu_core.cpp:791-828). */
    LuxBackendError (*graph_begin)(LuxBackendContext* ctx);
    LuxBackendError (*graph_end)(LuxBackendContext* ctx, LuxCudaGraph** out);
    LuxBackendError (*graph_launch)(LuxBackendContext* ctx, LuxCudaGraph* graph);
    void (*graph_destroy)(LuxCudaGraph* graph);

    /* --- column-sharded layers: rank r owns columns [r*Nl, (r+1)*Nl) -------- */
    /* rank 0 obtains an id and hands it to the others (any host channel). */
    LuxBackendError (*shard_unique_id)(void* out_uid /* LUX_CUDA_NCCL_UID_BYTES */);
    /* one process per GPU */
    LuxBackendError (*shard_comm_create)(LuxBackendContext* ctx, int rank, int world, const void* uid,
                                         LuxCudaShardComm** out);
    /* one process driving `world` contexts */
    LuxBackendError (*shard_comm_create_all)(LuxBackendContext** ctxs, int world, LuxCudaShardComm** out);
    void (*shard_comm_destroy)(LuxCudaShardComm* comm);
    /* y_full[M, world*Nl] on every rank: local slice = x . dequant(wq_local)^T,
     * then all-gather of the slices (NCCL over NVLink) and the column
     * interleave.  `staging` holds world*M*Nl elements of y_dtype.
     * In the single-process form call it once per rank between
     * shard_group_begin / shard_group_end. */
    LuxBackendError (*qmatmul_sharded)(LuxCudaShardComm* comm, LuxBackendBuffer* x, LuxBackendBuffer* wq_local,
                                       LuxBackendBuffer* scales_local, LuxBackendBuffer* biases_local,
                                       LuxBackendBuffer* y_full, LuxBackendBuffer* staging,
                                       int M, int K, int N_local, int bits, int group,
                                       LuxBackendDtype x_dtype, LuxBackendDtype sb_dtype, LuxBackendDtype y_dtype);
    LuxBackendError (*shard_group_begin)(void);
    LuxBackendError (*shard_group_end)(void);

    /* --- column-sharded decode with the all-gather inside the matmul kernel (version >= 2) ---
     * Every rank holds the whole y[M, world*Nl] in a "symmetric" buffer that its peers can store into
     * over NVLink.  Set-up, once: symm_alloc on every rank; symm_export gives LUX_CUDA_SYMM_HANDLE_BYTES
     * to pass to the other ranks by any host channel; symm_attach takes all ranks' handles in rank order
     * (own entry ignored; other processes are reached by CUDA IPC, the same process directly).
     * symm_buffer is the local copy as an ordinary buffer (borrowed: valid until symm_free).  Before
     * symm_free every rank must be past its last call that stores into the buffer. */
    LuxBackendError (*symm_alloc)(LuxBackendContext* ctx, int rank, int world, size_t bytes, LuxCudaSymmBuffer** out);
    LuxBackendError (*symm_export)(LuxCudaSymmBuffer* buf, void* handle_out /* LUX_CUDA_SYMM_HANDLE_BYTES */);
    LuxBackendError (*symm_attach)(LuxCudaSymmBuffer* buf, const void* handles /* world x LUX_CUDA_SYMM_HANDLE_BYTES */);
    LuxBackendBuffer* (*symm_buffer)(LuxCudaSymmBuffer* buf);
    void (*symm_free)(LuxCudaSymmBuffer* buf);
    /* y_full[:, rank*Nl : (rank+1)*Nl] = x . dequant(wq_local)^T, delivered into every rank's copy of y_full by
     * the matmul kernel itself; when the call's work on the stream ends the peers' columns of the same call
     * have arrived, so whatever is enqueued after it sees the whole y_full.  M <= 16: ONE decode launch (may be
     * recorded with graph_begin/graph_end).  M > 16: the prefill GEMM stores its tiles into all copies from
     * its epilogue, between two device-side barriers over the ranks.  All ranks must make the same calls on
     * the same buffer in the same order (a rank waits up to 2 s for its peers, then the next sync returns
     * INTERNAL).  bf16 x / scales / biases, Nl a multiple of 16, world <= 8, K as the kernels need it;
     * anything else is NOT_SUPPORTED (use qmatmul_sharded). */
    LuxBackendError (*qmatmul_sharded_push)(LuxCudaSymmBuffer* y_full, LuxBackendBuffer* x, LuxBackendBuffer* wq_local,
                                            LuxBackendBuffer* scales_local, LuxBackendBuffer* biases_local,
                                            int M, int K, int N_local, int bits, int group, LuxBackendDtype y_dtype);

    /* --- the elementwise steps between the projections of a decode layer, bf16 (version >= 3) ---
     * The inputs are column blocks of one row-major bf16 buffer with row stride `ld` elements, i.e. the
     * output of a fused q|k|v or gate|up projection; fp32 math, one rounding to bf16 per result.
     * sum3: out[r][c] = in[r][c] + in[r][cols+c] + in[r][2*cols+c]   (the add of op_add_f32,
     * backend_plugin.h:120, applied twice).  mul_rms_norm: m = in[r][c] * in[r][cols+c] rounded to bf16
     * (op_mul_f32, backend_plugin.h:122), then out = m * rsqrt(mean(m^2) + eps) per row (op_rms_norm_f32
     * with unit weight, backend_plugin.h:178; kernels/cpu/tensor_ops.c:546-566). */
    LuxBackendError (*sum3)(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t rows, size_t cols,
                            size_t ld);
    LuxBackendError (*mul_rms_norm)(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t rows,
                                    size_t cols, size_t ld, float eps);

    /* --- decode matmul with one of those steps applied to x as the kernel loads it (version >= 4) ---
     * y = prologue(x) . dequant(Wq)^T for M <= 8, bf16 x / scales / biases, in ONE launch:
     *   LUX_CUDA_PRO_RMS_NORM: x' = rms_norm(x) per row (unit weight, eps; rounded to bf16 as op_rms_norm_f32's
     *                          output would be); x is [M][x_ld], its first K columns are used;
     *   LUX_CUDA_PRO_SUM3:     x' = bf16(x[r][k] + x[r][K+k] + x[r][2K+k]), x is [M][x_ld], x_ld >= 3K.
     * The same results as the step followed by qmatmul (bit for bit for SUM3; for RMS_NORM the row's sum of
     * squares is accumulated in another order, which can move a normalised value by one bf16 step), without
     * the launch and the round trip of x'.  NOT_SUPPORTED when the shape is not taken (M > 8, a K the decode
     * kernel does not take, or for RMS_NORM a K longer than 16 k-blocks of 128 packed bytes): call the step and
     * qmatmul instead. */
    LuxBackendError (*qmatmul_pro)(LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                                   LuxBackendBuffer* biases, LuxBackendBuffer* y, int M, int K, int N, int bits, int group,
                                   LuxBackendDtype y_dtype, int prologue, size_t x_ld, float eps);

    /* --- several independent decode matmuls of one shape in one call (version >= 5) ---
     * (The reference's matmul slot, op_matmul_f32, backend_plugin.h:129, takes one matmul per call and its public
     * API forwards them one by one, src/gpu_core.cpp:450-474: this entry has no counterpart there.)
     * y[i] = x[i] . dequant(wq[i], scales[i], biases[i])^T for i < n: n layers (or n requests on one layer) of the
     * same K, N, bits, group, bf16, each with its own M[i] <= 16.  The same bits as n calls of qmatmul.  The matmuls
     * run in as few launches as their shapes allow (those with M <= 8 together, those with M > 8 together, up to 48
     * per launch), each launch a persistent kernel that goes from one matmul to the next without draining: what a
     * single decode launch spends on starting and on finishing is paid once per launch.  Nothing orders the
     * matmuls of a call among themselves: no y[i] may be an x[j] of the same call.  Shapes the decode kernel
     * does not take whole (K split over CTAs, fp32, M > 16) run as n calls of qmatmul. */
    LuxBackendError (*qmatmul_batch)(LuxBackendContext* ctx, int n, LuxBackendBuffer* const* x, LuxBackendBuffer* const* wq,
                                     LuxBackendBuffer* const* scales, LuxBackendBuffer* const* biases,
                                     LuxBackendBuffer* const* y, const int* M, int K, int N, int bits, int group,
                                     LuxBackendDtype y_dtype);

    /* --- several independent column-sharded decode matmuls of one shape in one call (version >= 6) ---
     * (No counterpart in the reference, whose multi-device support ends at create_context(device_index),
     * backend_plugin.h:84.)
     * qmatmul_batch for a layer whose columns are sharded over ranks: item i's full output y_i[M[i], world*Nl]
     * lies at byte offset y_offset[i] (a multiple of 16; the outputs do not overlap) of the symmetric buffer, on
     * every rank; this rank computes columns [rank*Nl, (rank+1)*Nl) of every item and the kernel stores them
     * into all ranks' copies as it goes from one matmul to the next.  The ranks meet once per launch, not once per
     * matmul (up to 48 matmuls per launch; items with M <= 8 and with M > 8 in separate launches): when the
     * call's work on the stream ends, every y_i is whole on this rank.  The same rules as qmatmul_sharded_push
     * (same calls in the same order on all ranks, bf16, Nl a multiple of 16, M[i] <= 16); results are the bits
     * of qmatmul_sharded_push item by item.  Shapes the batched kernel does not take (K split over CTAs) run as n
     * single pushes inside the call. */
    LuxBackendError (*qmatmul_sharded_push_batch)(LuxCudaSymmBuffer* y_all, int n, LuxBackendBuffer* const* x,
                                                  LuxBackendBuffer* const* wq_local, LuxBackendBuffer* const* scales_local,
                                                  LuxBackendBuffer* const* biases_local, const size_t* y_offset, const int* M,
                                                  int K, int N_local, int bits, int group, LuxBackendDtype y_dtype);

    /* --- qmatmul_pro for a column-sharded layer (version >= 7) ---
     * qmatmul_sharded_push with one of qmatmul_pro's prologues applied to x as the kernel loads it: x is the whole
     * (gathered) activation buffer [M][x_ld] on this rank, e.g. the symmetric buffer of the previous projection;
     * M <= 8.  Same results as the step on every rank followed by qmatmul_sharded_push, in one launch per rank.
     * NOT_SUPPORTED as for qmatmul_pro (M > 8, a K the decode kernel does not take or splits over CTAs on this
     * rank's share of the columns, for RMS_NORM a K longer than 16 k-blocks): call the step and
     * qmatmul_sharded_push instead -- the same decision on every rank, since it depends on the shape only. */
    LuxBackendError (*qmatmul_sharded_push_pro)(LuxCudaSymmBuffer* y_full, LuxBackendBuffer* x, LuxBackendBuffer* wq_local,
                                                LuxBackendBuffer* scales_local, LuxBackendBuffer* biases_local,
                                                int M, int K, int N_local, int bits, int group, LuxBackendDtype y_dtype,
                                                int prologue, size_t x_ld, float eps);
} lux_gpu_quant_vtbl;

/* Entry points exported with default visibility. */
LUX_GPU_BACKEND_EXPORT bool lux_gpu_backend_init(lux_gpu_backend_desc* out); /* backend_plugin.h:423 */
LUX_GPU_BACKEND_EXPORT const lux_gpu_quant_vtbl* lux_gpu_cuda_quant_vtbl(void);
/* Layout facts of the ABI the library was compiled against, for bindings that
 * mirror the struct by hand: sizeof(vtbl), offsetof(op_matmul_f32),
 * offsetof(op_ntt_forward), offsetof(_reserved), sizeof(desc). */
LUX_GPU_BACKEND_EXPORT void lux_gpu_cuda_abi_layout(uint32_t out[5]);
/* Decode-regime quantized matmul (bf16 x, bf16 scales/biases, 1 <= M <= 16) that allocates nothing.
 * No counterpart in the reference.
 *
 * For hosts that must not allocate device memory once they are running: a serving process that
 * has handed every free byte of HBM to its own arena (so a driver allocation would fail or stall
 * the device while it trims), or code running under a no-allocation policy after start-up.  The
 * ordinary qmatmul grows a per-context workspace through the plugin's allocator the first time a
 * shape needs it; this variant instead uses a 4 MiB scratch array compiled into the library
 * image.  Every GPU that loads the library carries those 4 MiB until the process exits.
 *
 * Same arguments and results as qmatmul (bit-identical output); the caller still owns x, wq,
 * scales, biases and y.  Shapes whose scratch need exceeds 4 MiB (only layers with very few
 * rows and a very long K) are refused with INVALID_ARGUMENT and a message in
 * lux_gpu_cuda_last_error(); shapes the decode kernel does not take return NOT_SUPPORTED.
 * The first call on a device looks up the scratch array's device address (once per device);
 * make that first call before starting any stream capture.  All calls on a device share the one
 * array: it keeps whatever the last call left, the kernel itself restores the part that must be
 * zero, and two calls that overlap on the GPU (different contexts of one device) would corrupt
 * each other -- run them one after the other. */
LUX_GPU_BACKEND_EXPORT LuxBackendError lux_gpu_cuda_qmatmul_decode_noalloc(
    LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
    LuxBackendBuffer* biases, LuxBackendBuffer* y, int M, int K, int N, int bits, int group,
    LuxBackendDtype y_dtype);
/* The reference's hook for a backend's table of built-in kernels: the core declares it as a weak function that
 * returns NULL (src/kernel_loader.cpp:191-210) and looks kernels up in whatever a backend linked into the same
 * image returns (lux_kernel_registry_get / _find, include/lux/gpu/kernel_loader.h:84-97).  The plugin's table
 * lists the kernel variants behind "lux.qmm.affine" (entry_point = the variant: bits, rows of x it takes) and the
 * helper kernels; they are compiled into the library (source and binary are NULL: nothing to compile at run
 * time), so the table is a directory of names, in the reference's own format. */
LUX_GPU_BACKEND_EXPORT const LuxKernelRegistry* lux_kernel_registry_cuda_get(void);
/* Last error text of the calling thread ("" if none). */
LUX_GPU_BACKEND_EXPORT const char* lux_gpu_cuda_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* LUX_CUDA_QUANT_H */
