// Host side of the quantized-matmul entry points (lux_gpu_quant_vtbl):
// argument validation, kernel choice, the decode workspace, buffer interop,
// device timers.  Mirrors the shape of op_matmul_f32(ctx, a, b, out, M, K, N)
// (include/lux/gpu/backend_plugin.h:129) and returns INVALID_ARGUMENT on NULL
// or undersized buffers the way the CPU backend does
// (src/cpu_backend.cpp:243-247).
#include <cstring>
#include <new>

#include "internal.h"

namespace luxcuda {

namespace {

size_t dtype_size(int dt) {
    switch (dt) {
        case LUX_DTYPE_FLOAT32: return 4;
        case LUX_DTYPE_BFLOAT16: return 2;
        default: return 0;
    }
}

LuxBackendError check_format(int K, int bits, int group) {
    if (bits != 4 && bits != 8) {
        set_last_error("qmatmul: bits must be 4 or 8 (got %d)", bits);
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (group != 32 && group != 64 && group != 128) {
        set_last_error("qmatmul: group must be 32, 64 or 128 (got %d)", group);
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (K <= 0 || K % group) {
        set_last_error("qmatmul: K=%d must be a positive multiple of group=%d", K, group);
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    return LUX_BACKEND_OK;
}

}  // namespace

static bool ranges_overlap(const char* a_lo, size_t a_bytes, const char* b_lo, const char* b_hi) {
    return a_lo < b_hi && b_lo < a_lo + a_bytes;
}
bool chain_is_open(const Context* c) {
    static const bool disabled = getenv("LUXCUDA_NO_PDL") != nullptr;
    if (disabled || c->stream_exposed) return false;
    return c->chain_launches == c->launches.load() && c->chain_copies == c->copies.load();
}
void note_chain_launch(Context* c, const void* out, size_t out_bytes) {
    c->chain_launches = c->launches.load();
    c->chain_copies = c->copies.load();
    c->chain_out_lo = (const char*)out;
    c->chain_out_hi = (const char*)out + out_bytes;
}
bool decode_may_overlap(const Context* c, const QmmArgs& a) {
    if (!chain_is_open(c)) return false;
    const size_t sb = (size_t)a.N * (a.K / a.group) * 2;
    return !ranges_overlap((const char*)a.wq, (size_t)a.N * a.K * a.bits / 8, c->chain_out_lo, c->chain_out_hi) &&
           !ranges_overlap((const char*)a.scales, sb, c->chain_out_lo, c->chain_out_hi) &&
           !ranges_overlap((const char*)a.biases, sb, c->chain_out_lo, c->chain_out_hi);
}
bool decode_x_stable(const Context* c, const QmmArgs& a) {
    return !ranges_overlap((const char*)a.x, (size_t)a.M * a.K * 2, c->chain_out_lo, c->chain_out_hi);
}
void note_decode_launch(Context* c, const QmmArgs& a) {
    c->chain_launches = c->launches.load();
    c->chain_copies = c->copies.load();
    c->chain_out_lo = (const char*)a.y;
    c->chain_out_hi = (const char*)a.y + (size_t)a.M * a.N * (a.y_dtype == LUX_DTYPE_BFLOAT16 ? 2 : 4);
}

LuxBackendError ensure_qmv_workspace(Context* c, size_t bytes) {
    if (bytes <= c->qmv_ws_bytes) return LUX_BACKEND_OK;
    // Growing means an allocation and a memset: neither belongs into a stream capture.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(c->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) {
        set_last_error("qmatmul: this shape needs a larger decode workspace (%zu bytes); run it once outside the graph capture first", bytes);
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    cudaError_t e = cudaSuccess;
    Block* nb = c->dev->acquire(bytes, c->stream, &e);
    if (!nb) return map_cuda_error(e, "qmv workspace");
    // arrival counters start at zero; every launch leaves them at zero
    e = cudaMemsetAsync(nb->ptr, 0, bytes, c->stream);
    c->copies++;
    if (e != cudaSuccess) {
        c->dev->release(nb, c->stream);
        return map_cuda_error(e, "qmv workspace memset");
    }
    if (c->qmv_ws) c->qmv_ws_retired.push_back(c->qmv_ws);  // graphs recorded earlier still point at it
    c->qmv_ws = nb;
    c->qmv_ws_bytes = bytes;
    return LUX_BACKEND_OK;
}

LuxBackendError ensure_qmm_workspace(Context* c) {
    if (c->qmm_ws) return LUX_BACKEND_OK;
    const size_t bytes = qmm_tc_workspace_bytes(c->dev->sm_count);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(c->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) {
        set_last_error("qmatmul: the prefill kernel's workspace does not exist yet; run one M > 16 call outside the graph capture first");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    cudaError_t e = cudaSuccess;
    Block* nb = c->dev->acquire(bytes, c->stream, &e);
    if (!nb) return map_cuda_error(e, "qmm workspace");
    e = cudaMemsetAsync(nb->ptr, 0, bytes, c->stream);  // the flags start at zero; every launch leaves them at zero
    c->copies++;
    if (e != cudaSuccess) {
        c->dev->release(nb, c->stream);
        return map_cuda_error(e, "qmm workspace memset");
    }
    c->qmm_ws = nb;
    return LUX_BACKEND_OK;
}

LuxBackendError qmatmul_on_stream(Context* c, const QmmArgs& a) {
    if (a.M == 0 || a.N == 0) return LUX_BACKEND_OK;
    const char* name = "";
    cudaError_t e = cudaSuccess;
    int launches = 1;
    if (a.x_dtype == LUX_DTYPE_BFLOAT16) {
        if (a.M > 16 && qmm_tc_supported(a, c->dev->sm_count)) {
            LuxBackendError le = ensure_qmm_workspace(c);
            if (le != LUX_BACKEND_OK) return le;
            e = launch_qmm_tc(a, c->qmm_ws->ptr, c->dev->sm_count, c->stream, &name);
        } else {
            // decode kernel, 16 rows of x per launch
            QmmArgs chunk = a;
            chunk.M = a.M < 16 ? a.M : 16;
            if (qmv_mma_supported(chunk, c->dev->sm_count)) {
                const size_t ws = qmv_mma_workspace_bytes(chunk, c->dev->sm_count);
                LuxBackendError le = ensure_qmv_workspace(c, ws);
                if (le != LUX_BACKEND_OK) return le;
                const size_t ysz = dtype_size(a.y_dtype);
                launches = 0;
                for (int m0 = 0; m0 < a.M && e == cudaSuccess; m0 += 16) {
                    chunk.M = a.M - m0 < 16 ? a.M - m0 : 16;
                    chunk.x = (const char*)a.x + (size_t)m0 * a.K * 2;
                    chunk.y = (char*)a.y + (size_t)m0 * a.N * ysz;
                    e = launch_qmv_mma(chunk, c->qmv_ws->ptr, c->dev->sm_count, c->stream, &name, decode_may_overlap(c, chunk),
                                       nullptr, decode_x_stable(c, chunk));
                    if (e == cudaSuccess) {
                        c->launches++;
                        note_decode_launch(c, chunk);
                    }
                }
            } else {
                e = launch_qmv_simt(a, c->stream, &name);
            }
        }
    } else {
        e = launch_qmv_simt(a, c->stream, &name);
    }
    if (e != cudaSuccess) return map_cuda_error(e, name);
    c->last_kernel = name;
    c->launches += launches;
    if (getenv("LUXCUDA_TRACE")) fprintf(stderr, "luxcuda: qmatmul M=%d K=%d N=%d bits=%d group=%d -> %s\n", a.M, a.K, a.N, a.bits, a.group, name);
    return LUX_BACKEND_OK;
}

namespace {

LuxBackendError qmatmul(LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                        LuxBackendBuffer* biases, LuxBackendBuffer* y, int M, int K, int N, int bits, int group,
                        LuxBackendDtype x_dtype, LuxBackendDtype sb_dtype, LuxBackendDtype y_dtype) {
    Context* c = as_ctx(ctx);
    Buffer *bx = as_buf(x), *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases), *by = as_buf(y);
    if (!c || !bx || !bw || !bs || !bb || !by || M < 0 || N < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError fe = check_format(K, bits, group);
    if (fe != LUX_BACKEND_OK) return fe;
    const size_t xs = dtype_size(x_dtype), ss = dtype_size(sb_dtype), ys = dtype_size(y_dtype);
    if (!xs || !ss || !ys) {
        set_last_error("qmatmul: dtypes must be FLOAT32 or BFLOAT16");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (x_dtype == LUX_DTYPE_BFLOAT16 && sb_dtype != LUX_DTYPE_BFLOAT16) {
        set_last_error("qmatmul: bf16 activations need bf16 scales/biases");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    if ((size_t)M * K * xs > bx->bytes || (size_t)N * K * bits / 8 > bw->bytes ||
        (size_t)N * (K / group) * ss > bs->bytes || (size_t)N * (K / group) * ss > bb->bytes ||
        (size_t)M * N * ys > by->bytes) {
        set_last_error("qmatmul: a buffer is smaller than its shape needs");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (((uintptr_t)bx->ptr | (uintptr_t)bw->ptr | (uintptr_t)bs->ptr | (uintptr_t)bb->ptr | (uintptr_t)by->ptr) & 15) {
        set_last_error("qmatmul: buffers must be 16-byte aligned");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    QmmArgs a{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, by->ptr, M, K, N, bits, group,
              (int)x_dtype, (int)sb_dtype, (int)y_dtype};
    a.error = c->err_dev;
    LuxBackendError r = qmatmul_on_stream(c, a);
    bx->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = by->last_stream = c->stream;
    return r;
}

LuxBackendError dequantize(LuxBackendContext* ctx, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                           LuxBackendBuffer* biases, LuxBackendBuffer* out, int N, int K, int bits, int group,
                           LuxBackendDtype sb_dtype, LuxBackendDtype out_dtype) {
    Context* c = as_ctx(ctx);
    Buffer *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases), *bo = as_buf(out);
    if (!c || !bw || !bs || !bb || !bo || N < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError fe = check_format(K, bits, group);
    if (fe != LUX_BACKEND_OK) return fe;
    const size_t ss = dtype_size(sb_dtype), os = dtype_size(out_dtype);
    if (!ss || !os) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (out_dtype == LUX_DTYPE_BFLOAT16 && sb_dtype != LUX_DTYPE_BFLOAT16) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if ((size_t)N * K * bits / 8 > bw->bytes || (size_t)N * (K / group) * ss > bs->bytes ||
        (size_t)N * (K / group) * ss > bb->bytes || (size_t)N * K * os > bo->bytes)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_dequantize((const uint32_t*)bw->ptr, bs->ptr, bb->ptr, bo->ptr, N, K, bits, group,
                                   (int)sb_dtype, (int)out_dtype, c->stream));
    c->launches++;
    bw->last_stream = bs->last_stream = bb->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError unpack(LuxBackendContext* ctx, LuxBackendBuffer* wq, LuxBackendBuffer* q_out, int N, int K, int bits) {
    Context* c = as_ctx(ctx);
    Buffer *bw = as_buf(wq), *bo = as_buf(q_out);
    if (!c || !bw || !bo || N < 0 || K <= 0 || (bits != 4 && bits != 8) || (K * bits) % 32)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((size_t)N * K * bits / 8 > bw->bytes || (size_t)N * K > bo->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_unpack((const uint32_t*)bw->ptr, (uint8_t*)bo->ptr, N, K, bits, c->stream));
    c->launches++;
    bw->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError quantize(LuxBackendContext* ctx, LuxBackendBuffer* w, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                         LuxBackendBuffer* biases, int N, int K, int bits, int group, LuxBackendDtype sb_dtype) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(w), *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases);
    if (!c || !bi || !bw || !bs || !bb || N < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError fe = check_format(K, bits, group);
    if (fe != LUX_BACKEND_OK) return fe;
    const size_t ss = dtype_size(sb_dtype);
    if (!ss) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((size_t)N * K * 4 > bi->bytes || (size_t)N * K * bits / 8 > bw->bytes ||
        (size_t)N * (K / group) * ss > bs->bytes || (size_t)N * (K / group) * ss > bb->bytes)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_quantize((const float*)bi->ptr, (uint32_t*)bw->ptr, bs->ptr, bb->ptr, N, K, bits, group,
                                 (int)sb_dtype, c->stream));
    c->launches++;
    bi->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError rms_norm(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, LuxBackendBuffer* weight,
                         size_t rows, size_t dim, float eps, LuxBackendDtype in_dtype, LuxBackendDtype out_dtype) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out), *bw = weight ? as_buf(weight) : nullptr;
    if (!c || !bi || !bo || (weight && !bw)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t is = dtype_size(in_dtype), os = dtype_size(out_dtype);
    if (!is || !os) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (rows * dim * is > bi->bytes || rows * dim * os > bo->bytes || (bw && dim * 4 > bw->bytes))
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    // behind a chain kernel the whole kernel waits for it on the device (it reads nothing before that wait)
    LUX_CUDA_TRY(launch_rms_norm(bi->ptr, bo->ptr, bw ? (const float*)bw->ptr : nullptr, rows, dim, eps, (int)in_dtype,
                                 (int)out_dtype, c->stream, chain_is_open(c)));
    c->launches++;
    note_chain_launch(c, bo->ptr, rows * dim * os);
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError sum3(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t rows, size_t cols, size_t ld) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!c || !bi || !bo || ld < 3 * cols) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (rows && ((rows - 1) * ld + 3 * cols) * 2 > bi->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (rows * cols * 2 > bo->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_sum3(bi->ptr, bo->ptr, rows, cols, ld, c->stream, chain_is_open(c)));
    c->launches++;
    note_chain_launch(c, bo->ptr, rows * cols * 2);
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError mul_rms_norm(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t rows, size_t cols,
                             size_t ld, float eps) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!c || !bi || !bo || ld < 2 * cols) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (rows && ((rows - 1) * ld + 2 * cols) * 2 > bi->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (rows * cols * 2 > bo->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_mul_rms_norm(bi->ptr, bo->ptr, rows, cols, ld, eps, c->stream, chain_is_open(c)));
    c->launches++;
    note_chain_launch(c, bo->ptr, rows * cols * 2);
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError qmatmul_pro(LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                            LuxBackendBuffer* biases, LuxBackendBuffer* y, int M, int K, int N, int bits, int group,
                            LuxBackendDtype y_dtype, int prologue, size_t x_ld, float eps) {
    Context* c = as_ctx(ctx);
    Buffer *bx = as_buf(x), *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases), *by = as_buf(y);
    if (!c || !bx || !bw || !bs || !bb || !by || M < 0 || N < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError fe = check_format(K, bits, group);
    if (fe != LUX_BACKEND_OK) return fe;
    const size_t ys = dtype_size(y_dtype);
    const size_t span = prologue == LUX_CUDA_PRO_SUM3 ? (size_t)3 * K : (size_t)K;
    if (!ys || (prologue != LUX_CUDA_PRO_RMS_NORM && prologue != LUX_CUDA_PRO_SUM3) || x_ld < span || (x_ld & 7) ||
        x_ld > (size_t)INT32_MAX) {
        set_last_error("qmatmul_pro: prologue must be RMS_NORM or SUM3, x_ld a multiple of 8 that holds the columns read");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (M == 0 || N == 0) return LUX_BACKEND_OK;
    if (((size_t)(M - 1) * x_ld + span) * 2 > bx->bytes || (size_t)N * K * bits / 8 > bw->bytes ||
        (size_t)N * (K / group) * 2 > bs->bytes || (size_t)N * (K / group) * 2 > bb->bytes || (size_t)M * N * ys > by->bytes) {
        set_last_error("qmatmul_pro: a buffer is smaller than its shape needs");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (((uintptr_t)bx->ptr | (uintptr_t)bw->ptr | (uintptr_t)bs->ptr | (uintptr_t)bb->ptr | (uintptr_t)by->ptr) & 15) {
        set_last_error("qmatmul_pro: buffers must be 16-byte aligned");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    QmmArgs a{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, by->ptr, M, K, N, bits, group,
              (int)LUX_DTYPE_BFLOAT16, (int)LUX_DTYPE_BFLOAT16, (int)y_dtype};
    a.pro = prologue;
    a.error = c->err_dev;
    a.x_ld = (int)x_ld;
    a.eps = eps;
    if (M > 8 || !qmv_mma_supported(a, c->dev->sm_count)) {
        set_last_error("qmatmul_pro: shape not taken by the decode kernel with a prologue (M <= 8, K as qmatmul's decode path)");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    LuxBackendError le = ensure_qmv_workspace(c, qmv_mma_workspace_bytes(a, c->dev->sm_count));
    if (le != LUX_BACKEND_OK) return le;
    const char* name = "";
    // (x is the output of the launch before: never read ahead of the wait for it)
    cudaError_t e = launch_qmv_mma(a, c->qmv_ws->ptr, c->dev->sm_count, c->stream, &name, decode_may_overlap(c, a), nullptr, false);
    if (e == cudaErrorNotSupported) {
        cudaGetLastError();
        set_last_error("qmatmul_pro: the rms-norm prologue needs K within 16 k-blocks of 128 packed bytes and no K split");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    if (e != cudaSuccess) return map_cuda_error(e, name);
    c->launches++;
    note_decode_launch(c, a);
    c->last_kernel = name;
    bx->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = by->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

LuxBackendError qmatmul_batch(LuxBackendContext* ctx, int n, LuxBackendBuffer* const* x, LuxBackendBuffer* const* wq,
                              LuxBackendBuffer* const* scales, LuxBackendBuffer* const* biases, LuxBackendBuffer* const* y,
                              const int* M, int K, int N, int bits, int group, LuxBackendDtype y_dtype) {
    Context* c = as_ctx(ctx);
    if (!c || n < 0 || (n && (!x || !wq || !scales || !biases || !y || !M)) || N < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError fe = check_format(K, bits, group);
    if (fe != LUX_BACKEND_OK) return fe;
    const size_t ys = dtype_size(y_dtype);
    if (!ys) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0 || N == 0) return LUX_BACKEND_OK;
    std::vector<QmmArgs> items((size_t)n);
    bool decode = true;
    for (int i = 0; i < n; i++) {
        Buffer *bx = as_buf(x[i]), *bw = as_buf(wq[i]), *bs = as_buf(scales[i]), *bb = as_buf(biases[i]), *by = as_buf(y[i]);
        if (!bx || !bw || !bs || !bb || !by || M[i] < 1) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        if ((size_t)M[i] * K * 2 > bx->bytes || (size_t)N * K * bits / 8 > bw->bytes || (size_t)N * (K / group) * 2 > bs->bytes ||
            (size_t)N * (K / group) * 2 > bb->bytes || (size_t)M[i] * N * ys > by->bytes) {
            set_last_error("qmatmul_batch: a buffer of item %d is smaller than its shape needs", i);
            return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        }
        if (((uintptr_t)bx->ptr | (uintptr_t)bw->ptr | (uintptr_t)bs->ptr | (uintptr_t)bb->ptr | (uintptr_t)by->ptr) & 15) {
            set_last_error("qmatmul_batch: buffers must be 16-byte aligned");
            return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        }
        items[i] = QmmArgs{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, by->ptr, M[i], K, N, bits, group,
                           (int)LUX_DTYPE_BFLOAT16, (int)LUX_DTYPE_BFLOAT16, (int)y_dtype};
        items[i].error = c->err_dev;
        decode = decode && M[i] <= 16;
    }
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    const char* name = "";
    bool batched = false;
    if (decode) {
        // the items with M <= 8 and those with M > 8, each kind in launches of at most qmv_batch_max()
        batched = true;
        std::vector<QmmArgs> kind;
        for (int hi = 0; hi < 2 && batched; hi++) {
            kind.clear();
            for (const QmmArgs& a : items)
                if ((a.M > 8) == (hi == 1)) kind.push_back(a);
            for (size_t i0 = 0; i0 < kind.size() && batched; i0 += (size_t)qmv_batch_max()) {
                const int cnt = (int)std::min(kind.size() - i0, (size_t)qmv_batch_max());
                cudaError_t e = launch_qmv_batch(kind.data() + i0, cnt, c->dev->sm_count, c->stream, &name);
                if (e == cudaErrorNotSupported && hi == 0 && i0 == 0) {
                    cudaGetLastError();
                    batched = false;  // nothing launched yet: one by one below
                } else if (e != cudaSuccess) {
                    return map_cuda_error(e, name);
                } else {
                    c->launches++;
                }
            }
        }
    }
    if (!batched) {
        for (const QmmArgs& a : items) {
            LuxBackendError r = qmatmul_on_stream(c, a);
            if (r != LUX_BACKEND_OK) return r;
        }
    } else {
        c->last_kernel = name;
    }
    for (int i = 0; i < n; i++)
        as_buf(x[i])->last_stream = as_buf(wq[i])->last_stream = as_buf(scales[i])->last_stream = as_buf(biases[i])->last_stream =
            as_buf(y[i])->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

// --- buffer interop ---------------------------------------------------------
void* buffer_device_ptr(LuxBackendContext*, LuxBackendBuffer* buf) {
    Buffer* b = as_buf(buf);
    if (b) b->exposed = true;
    return b ? b->ptr : nullptr;
}
size_t buffer_size(LuxBackendContext*, LuxBackendBuffer* buf) {
    Buffer* b = as_buf(buf);
    return b ? b->bytes : 0;
}
LuxBackendBuffer* buffer_wrap(LuxBackendContext* ctx, void* device_ptr, size_t bytes) {
    Context* c = as_ctx(ctx);
    if (!c || !device_ptr) return nullptr;
    auto* b = new (std::nothrow) Buffer();
    if (!b) return nullptr;
    b->dev = c->dev;
    b->ptr = device_ptr;
    b->bytes = bytes;
    b->last_stream = c->stream;
    return reinterpret_cast<LuxBackendBuffer*>(b);
}
LuxBackendError buffer_copy_from_host_async(LuxBackendContext* ctx, LuxBackendBuffer* buf, const void* src, size_t bytes) {
    Context* c = as_ctx(ctx);
    Buffer* b = as_buf(buf);
    if (!c || !b || !src) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t n = bytes < b->bytes ? bytes : b->bytes;
    if (!n) return LUX_BACKEND_OK;
    DeviceGuard g(c->dev->device());
    c->copies++;
    LUX_CUDA_TRY(cudaMemcpyAsync(b->ptr, src, n, cudaMemcpyHostToDevice, c->stream));
    b->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
void* host_alloc_pinned(size_t bytes) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
void host_free_pinned(void* p) {
    if (p) cudaFreeHost(p);
}
void* context_stream(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    if (!c) return nullptr;
    c->stream_exposed = true;  // from now on the host may enqueue work of its own on it
    return (void*)c->stream;
}
LuxBackendError allocator_stats(LuxBackendContext* ctx, uint64_t* reserved, uint64_t* in_use, uint64_t* driver_allocs) {
    Context* c = as_ctx(ctx);
    if (!c) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    c->dev->stats(reserved, in_use, driver_allocs);
    return LUX_BACKEND_OK;
}
LuxBackendError allocator_trim(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    if (!c) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    c->dev->trim();
    return LUX_BACKEND_OK;
}

// --- timers -----------------------------------------------------------------
LuxBackendError timer_record(LuxBackendContext* ctx, int slot) {
    Context* c = as_ctx(ctx);
    if (!c || slot < 0 || slot >= kTimerSlots) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    if (!c->timers[slot]) LUX_CUDA_TRY(cudaEventCreate(&c->timers[slot]));
    LUX_CUDA_TRY(cudaEventRecord(c->timers[slot], c->stream));
    return LUX_BACKEND_OK;
}
LuxBackendError timer_elapsed_ms(LuxBackendContext* ctx, int a, int b, float* ms) {
    Context* c = as_ctx(ctx);
    if (!c || !ms || a < 0 || b < 0 || a >= kTimerSlots || b >= kTimerSlots || !c->timers[a] || !c->timers[b])
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(cudaEventSynchronize(c->timers[b]));
    LUX_CUDA_TRY(cudaEventElapsedTime(ms, c->timers[a], c->timers[b]));
    return LUX_BACKEND_OK;
}
LuxBackendError flush_l2(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    if (!c) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    size_t bytes = 0;
    cudaError_t e = cudaSuccess;
    void* p = c->dev->flush_buffer(&bytes, &e);
    if (!p) return map_cuda_error(e, "flush buffer");
    LUX_CUDA_TRY(launch_flush(p, bytes, c->stream));
    return LUX_BACKEND_OK;
}
const char* last_kernel(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    return c ? c->last_kernel : "";
}
uint64_t launch_count(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    return c ? c->launches.load() : 0;
}

// --- CUDA graphs --------------------------------------------------------------
}  // namespace
}  // namespace luxcuda
struct LuxCudaGraph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int device = 0;
    uint64_t launches = 0;  // plugin kernels recorded in the graph
};
namespace luxcuda {
namespace {
thread_local uint64_t t_capture_base = 0;

LuxBackendError graph_begin(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    if (!c) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    t_capture_base = c->launches.load();
    return LUX_BACKEND_OK;
}
LuxBackendError graph_end(LuxBackendContext* ctx, LuxCudaGraph** out) {
    Context* c = as_ctx(ctx);
    if (!c || !out) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    cudaGraph_t graph = nullptr;
    LUX_CUDA_TRY(cudaStreamEndCapture(c->stream, &graph));
    auto* gr = new (std::nothrow) LuxCudaGraph();
    if (!gr) {
        cudaGraphDestroy(graph);
        return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    }
    gr->graph = graph;
    gr->device = c->dev->device();
    gr->launches = c->launches.load() - t_capture_base;
    c->launches -= gr->launches;  // recorded, not run
    cudaError_t e = cudaGraphInstantiate(&gr->exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        delete gr;
        return map_cuda_error(e, "cudaGraphInstantiate");
    }
    *out = gr;
    return LUX_BACKEND_OK;
}
LuxBackendError graph_launch(LuxBackendContext* ctx, LuxCudaGraph* gr) {
    Context* c = as_ctx(ctx);
    if (!c || !gr || !gr->exec || gr->device != c->dev->device()) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(cudaGraphLaunch(gr->exec, c->stream));
    c->launches += gr->launches;
    return LUX_BACKEND_OK;
}
void graph_destroy(LuxCudaGraph* gr) {
    if (!gr) return;
    DeviceGuard g(gr->device);
    if (gr->exec) cudaGraphExecDestroy(gr->exec);
    if (gr->graph) cudaGraphDestroy(gr->graph);
    delete gr;
}

lux_gpu_quant_vtbl g_quant;
std::once_flag g_quant_once;

void fill_quant() {
    std::memset(&g_quant, 0, sizeof(g_quant));
    g_quant.magic = LUX_CUDA_QUANT_MAGIC;
    g_quant.version = LUX_CUDA_QUANT_VERSION;
    g_quant.size = (uint32_t)sizeof(g_quant);
    g_quant.qmatmul = qmatmul;
    g_quant.dequantize = dequantize;
    g_quant.unpack = unpack;
    g_quant.quantize = quantize;
    g_quant.rms_norm = rms_norm;
    g_quant.buffer_device_ptr = buffer_device_ptr;
    g_quant.buffer_size = buffer_size;
    g_quant.buffer_wrap = buffer_wrap;
    g_quant.buffer_copy_from_host_async = buffer_copy_from_host_async;
    g_quant.host_alloc_pinned = host_alloc_pinned;
    g_quant.host_free_pinned = host_free_pinned;
    g_quant.context_stream = context_stream;
    g_quant.allocator_stats = allocator_stats;
    g_quant.allocator_trim = allocator_trim;
    g_quant.timer_record = timer_record;
    g_quant.timer_elapsed_ms = timer_elapsed_ms;
    g_quant.flush_l2 = flush_l2;
    g_quant.last_kernel = last_kernel;
    g_quant.launch_count = launch_count;
    g_quant.graph_begin = graph_begin;
    g_quant.graph_end = graph_end;
    g_quant.graph_launch = graph_launch;
    g_quant.graph_destroy = graph_destroy;
    fill_shard_entries(&g_quant);
    fill_symm_entries(&g_quant);
    g_quant.sum3 = sum3;
    g_quant.mul_rms_norm = mul_rms_norm;
    g_quant.qmatmul_pro = qmatmul_pro;
    g_quant.qmatmul_batch = qmatmul_batch;
}

}  // namespace

const lux_gpu_quant_vtbl* quant_vtbl() {
    std::call_once(g_quant_once, fill_quant);
    return &g_quant;
}

}  // namespace luxcuda
