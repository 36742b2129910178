// libluxgpu_backend_cuda.so: the base vtable of the Lux GPU plugin ABI
// (include/lux/gpu/backend_plugin.h:82-382), filled for NVIDIA B200.
//
// Semantics follow the built-in CPU backend (src/cpu_backend.cpp) wherever the
// core or its test harness depends on them:
//   * buffer_alloc returns zeroed memory (cpu_backend.cpp:121-131);
//   * copies clamp to min(bytes, buffer size) (cpu_backend.cpp:148-160);
//   * buffer_copy_to_host blocks and is ordered after all earlier work of the
//     context, because callers read results without calling sync first
//     (test/test_core.cpp:66-70);
//   * buffer_free works after the owning context was destroyed and ignores its
//     ctx argument (src/gpu_core.cpp:216-233 frees tensors of a dead context);
//   * op_matmul_f32 is A[M,K].B[K,N] row-major with a sequential fp32 k-sum,
//     multiply then add (cpu_backend.cpp:253-264) -- bit-identical results;
//   * op_ntt_forward/inverse take HOST pointers and transform in place
//     (cpu_backend.cpp:269-323).
// Slots the CPU backend leaves NULL and this plugin does not implement stay
// NULL ("unsupported", src/gpu_core.cpp:446,499,833).
#include <cstddef>
#include <cstring>
#include <new>

#include "internal.h"

using namespace luxcuda;

static_assert(sizeof(lux_gpu_backend_vtbl) == 64 * sizeof(void*), "plugin ABI v2 has 64 slots");
static_assert(offsetof(lux_gpu_backend_vtbl, _reserved) == 60 * sizeof(void*), "reserved slots are the last four");
static_assert(LUX_GPU_BACKEND_ABI_VERSION == 2, "written against ABI version 2");

namespace {

// ---------------------------------------------------------------------------
// lifecycle
// ---------------------------------------------------------------------------
LuxBackendContext* create_context(int device_index) {
    cudaError_t e = cudaSuccess;
    auto dev = device_state(device_index, &e);
    if (!dev) {
        map_cuda_error(e, "create_context");
        return nullptr;
    }
    auto* c = new (std::nothrow) Context();
    if (!c) return nullptr;
    c->dev = dev;
    c->stream = dev->acquire_stream();
    if (!c->stream) {
        set_last_error("create_context: no stream");
        delete c;
        return nullptr;
    }
    {
        // the context's error word (see Context::err_host); without it the kernels fall back to the process's word
        DeviceGuard g(dev->device());
        void* hp = nullptr;
        void* dp = nullptr;
        if (cudaHostAlloc(&hp, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess &&
            cudaHostGetDevicePointer(&dp, hp, 0) == cudaSuccess) {
            c->err_host = static_cast<int*>(hp);
            *c->err_host = 0;
            c->err_dev = static_cast<int*>(dp);
        } else {
            if (hp) cudaFreeHost(hp);
            cudaGetLastError();
        }
    }
    return reinterpret_cast<LuxBackendContext*>(c);
}

void destroy_context(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    if (!c) return;
    {
        DeviceGuard g(c->dev->device());
        cudaStreamSynchronize(c->stream);
        for (auto& ev : c->timers)
            if (ev) cudaEventDestroy(ev);
    }
    if (c->qmv_ws) c->dev->release(c->qmv_ws, c->stream);
    for (Block* b : c->qmv_ws_retired) c->dev->release(b, c->stream);
    if (c->qmm_ws) c->dev->release(c->qmm_ws, c->stream);
    if (c->err_host) cudaFreeHost(c->err_host);
    c->dev->release_stream(c->stream);
    c->magic = 0;
    delete c;
}

LuxBackendError get_device_count(int* count) {
    if (!count) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    *count = n;
    return LUX_BACKEND_OK;
}

LuxBackendError get_device_info(LuxBackendContext* ctx, LuxBackendDeviceInfo* info) {
    Context* c = as_ctx(ctx);
    if (!c || !info) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    size_t free_b = 0, total_b = 0;
    LUX_CUDA_TRY(cudaMemGetInfo(&free_b, &total_b));
    info->name = c->dev->prop.name;  // lives as long as the device state; the core copies nothing
    info->vendor = "NVIDIA";
    info->memory_total = total_b;
    info->memory_available = free_b;
    info->compute_units = c->dev->sm_count;
    info->max_workgroup_size = c->dev->prop.maxThreadsPerBlock;
    info->is_discrete = true;
    info->is_unified_memory = false;
    return LUX_BACKEND_OK;
}

LuxBackendError sync(LuxBackendContext* ctx) {
    Context* c = as_ctx(ctx);
    if (!c) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(cudaStreamSynchronize(c->stream));
    if (take_context_error(c) | take_device_error()) {
        set_last_error("a kernel timed out on an internal wait and returned early; results are invalid");
        return LUX_BACKEND_ERROR_INTERNAL;
    }
    return LUX_BACKEND_OK;
}

// ---------------------------------------------------------------------------
// buffers
// ---------------------------------------------------------------------------
Buffer* new_buffer(Context* c, size_t bytes) {
    cudaError_t e = cudaSuccess;
    Block* blk = c->dev->acquire(bytes, c->stream, &e);
    if (!blk) {
        map_cuda_error(e, "buffer_alloc");
        return nullptr;
    }
    auto* b = new (std::nothrow) Buffer();
    if (!b) {
        c->dev->release(blk, c->stream);
        return nullptr;
    }
    b->dev = c->dev;
    b->block = blk;
    b->ptr = blk->ptr;
    b->bytes = bytes;
    b->last_stream = c->stream;
    return b;
}

LuxBackendBuffer* buffer_alloc(LuxBackendContext* ctx, size_t bytes) {
    Context* c = as_ctx(ctx);
    if (!c) return nullptr;
    Buffer* b = new_buffer(c, bytes);
    if (!b) return nullptr;
    if (bytes) {
        DeviceGuard g(c->dev->device());
        c->copies++;
        if (cudaMemsetAsync(b->ptr, 0, bytes, c->stream) != cudaSuccess) {
            cudaGetLastError();
            c->dev->release(b->block, c->stream);
            delete b;
            return nullptr;
        }
    }
    return reinterpret_cast<LuxBackendBuffer*>(b);
}

LuxBackendBuffer* buffer_alloc_with_data(LuxBackendContext* ctx, const void* data, size_t bytes) {
    Context* c = as_ctx(ctx);
    if (!c || (!data && bytes)) return nullptr;
    Buffer* b = new_buffer(c, bytes);
    if (!b) return nullptr;
    if (bytes) {
        DeviceGuard g(c->dev->device());
        // The caller keeps `data` and may change it right after this returns.
        c->copies++;
        cudaError_t e = cudaMemcpyAsync(b->ptr, data, bytes, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) {
            map_cuda_error(e, "buffer_alloc_with_data");
            c->dev->release(b->block, c->stream);
            delete b;
            return nullptr;
        }
    }
    return reinterpret_cast<LuxBackendBuffer*>(b);
}

void buffer_free(LuxBackendContext* /*ctx may dangle*/, LuxBackendBuffer* buf) {
    Buffer* b = as_buf(buf);
    if (!b) return;
    if (b->block) b->dev->release(b->block, b->last_stream);
    b->magic = 0;
    delete b;
}

LuxBackendError buffer_copy_to_host(LuxBackendContext* ctx, LuxBackendBuffer* buf, void* dst, size_t bytes) {
    Context* c = as_ctx(ctx);
    Buffer* b = as_buf(buf);
    if (!c || !b || !dst) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    size_t n = bytes < b->bytes ? bytes : b->bytes;
    if (!n) return LUX_BACKEND_OK;
    DeviceGuard g(c->dev->device());
    c->copies++;
    LUX_CUDA_TRY(cudaMemcpyAsync(dst, b->ptr, n, cudaMemcpyDeviceToHost, c->stream));
    LUX_CUDA_TRY(cudaStreamSynchronize(c->stream));
    if (take_context_error(c) | take_device_error()) {
        set_last_error("a kernel timed out on an internal wait and returned early; results are invalid");
        return LUX_BACKEND_ERROR_INTERNAL;
    }
    return LUX_BACKEND_OK;
}

LuxBackendError buffer_copy_from_host(LuxBackendContext* ctx, LuxBackendBuffer* buf, const void* src, size_t bytes) {
    Context* c = as_ctx(ctx);
    Buffer* b = as_buf(buf);
    if (!c || !b || !src) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    size_t n = bytes < b->bytes ? bytes : b->bytes;
    if (!n) return LUX_BACKEND_OK;
    DeviceGuard g(c->dev->device());
    c->copies++;
    LUX_CUDA_TRY(cudaMemcpyAsync(b->ptr, src, n, cudaMemcpyHostToDevice, c->stream));
    LUX_CUDA_TRY(cudaStreamSynchronize(c->stream));  // the caller may reuse src at once
    b->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

void* buffer_get_host_ptr(LuxBackendContext*, LuxBackendBuffer*) { return nullptr; }  // discrete GPU

// ---------------------------------------------------------------------------
// custom kernels: source/binary loading is not offered; the one built-in name
// gives the quantized matmul through the unchanged dispatch slot.
// ---------------------------------------------------------------------------
LuxBackendKernel* kernel_load(LuxBackendContext* ctx, const char* /*source*/, const char* entry_point) {
    if (!as_ctx(ctx) || !entry_point) return nullptr;
    if (std::strcmp(entry_point, LUX_CUDA_QMM_KERNEL_NAME) != 0) {
        set_last_error("kernel_load: only the built-in kernel \"%s\" is available", LUX_CUDA_QMM_KERNEL_NAME);
        return nullptr;
    }
    auto* k = new (std::nothrow) Kernel();
    if (k) k->builtin_id = 1;
    return reinterpret_cast<LuxBackendKernel*>(k);
}

LuxBackendKernel* kernel_load_binary(LuxBackendContext*, const void*, size_t, const char*) { return nullptr; }

void kernel_destroy(LuxBackendContext*, LuxBackendKernel* kernel) {
    auto* k = reinterpret_cast<Kernel*>(kernel);
    if (k && k->magic == kKernMagic) {
        k->magic = 0;
        delete k;
    }
}

LuxBackendError kernel_dispatch(LuxBackendContext* ctx, LuxBackendKernel* kernel, uint32_t, uint32_t, uint32_t,
                                uint32_t, uint32_t, uint32_t, LuxBackendBuffer** buffers, int num_buffers) {
    Context* c = as_ctx(ctx);
    auto* k = reinterpret_cast<Kernel*>(kernel);
    if (!c || !k || k->magic != kKernMagic || !buffers) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (k->builtin_id != 1) return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    if (num_buffers != 6) {
        set_last_error("lux.qmm.affine expects 6 buffers {x, wq, scales, biases, y, params}");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    Buffer* pb = as_buf(buffers[5]);
    if (!pb || pb->bytes < sizeof(lux_qmm_params)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    // The dispatch ABI carries no scalars, so the shape travels in a device buffer and has to be read back:
    // once per content -- while nothing has touched the buffer since (LastStream), the copy kept with it is used
    // and the dispatch enqueues without waiting for the stream.
    static_assert(sizeof(lux_qmm_params) <= sizeof(pb->params_copy), "parameter block larger than its host copy");
    lux_qmm_params p;
    if (pb->params_uses != pb->last_stream.uses || pb->exposed || !pb->block) {  // (wrapped memory is the host's)
        DeviceGuard g(c->dev->device());
        c->copies++;
        LUX_CUDA_TRY(cudaMemcpyAsync(pb->params_copy, pb->ptr, sizeof(p), cudaMemcpyDeviceToHost, c->stream));
        LUX_CUDA_TRY(cudaStreamSynchronize(c->stream));
        pb->params_uses = pb->last_stream.uses;
    }
    memcpy(&p, pb->params_copy, sizeof(p));
    return quant_vtbl()->qmatmul(ctx, buffers[0], buffers[1], buffers[2], buffers[3], buffers[4], p.M, p.K, p.N,
                                 p.bits, p.group, (LuxBackendDtype)p.x_dtype, (LuxBackendDtype)p.sb_dtype,
                                 (LuxBackendDtype)p.y_dtype);
}

// ---------------------------------------------------------------------------
// fp32 ops the harness needs
// ---------------------------------------------------------------------------
LuxBackendError binary(LuxBackendContext* ctx, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out,
                       size_t n, BinOp op) {
    Context* c = as_ctx(ctx);
    Buffer *ba = as_buf(a), *bb = as_buf(b), *bo = as_buf(out);
    if (!c || !ba || !bb || !bo) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n * sizeof(float) > ba->bytes || n * sizeof(float) > bb->bytes || n * sizeof(float) > bo->bytes)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!n) return LUX_BACKEND_OK;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_binary_f32(op, (const float*)ba->ptr, (const float*)bb->ptr, (float*)bo->ptr, n, c->stream));
    c->launches++;
    ba->last_stream = bb->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
LuxBackendError op_add(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary(c, a, b, o, n, BinOp::Add); }
LuxBackendError op_sub(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary(c, a, b, o, n, BinOp::Sub); }
LuxBackendError op_mul(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary(c, a, b, o, n, BinOp::Mul); }
LuxBackendError op_div(LuxBackendContext* c, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* o, size_t n) { return binary(c, a, b, o, n, BinOp::Div); }

LuxBackendError op_matmul(LuxBackendContext* ctx, LuxBackendBuffer* a, LuxBackendBuffer* b, LuxBackendBuffer* out,
                          int M, int K, int N) {
    Context* c = as_ctx(ctx);
    Buffer *ba = as_buf(a), *bb = as_buf(b), *bo = as_buf(out);
    if (!c || !ba || !bb || !bo || M < 0 || K < 0 || N < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if ((size_t)M * K * 4 > ba->bytes || (size_t)K * N * 4 > bb->bytes || (size_t)M * N * 4 > bo->bytes)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!M || !N) return LUX_BACKEND_OK;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_matmul_f32((const float*)ba->ptr, (const float*)bb->ptr, (float*)bo->ptr, M, K, N, c->stream));
    c->launches++;
    ba->last_stream = bb->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

// ---------------------------------------------------------------------------
// the remaining fp32 tensor ops (backend_plugin.h:130-178; forwarded by src/gpu_core.cpp:430-789)
// ---------------------------------------------------------------------------
// in -> out over n elements each (unary maps, copy)
LuxBackendError unary(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t n, int op) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!c || !bi || !bo || n * sizeof(float) > bi->bytes || n * sizeof(float) > bo->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!n) return LUX_BACKEND_OK;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_unary_f32(op, (const float*)bi->ptr, (float*)bo->ptr, n, c->stream));
    c->launches++;
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
#define LUXCUDA_UNARY(name, code) \
    LuxBackendError name(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return unary(c, i, o, n, code); }
LUXCUDA_UNARY(op_exp, 0)
LUXCUDA_UNARY(op_log, 1)
LUXCUDA_UNARY(op_sqrt, 2)
LUXCUDA_UNARY(op_neg, 3)
LUXCUDA_UNARY(op_abs, 4)
LUXCUDA_UNARY(op_tanh, 5)
LUXCUDA_UNARY(op_sigmoid, 6)
LUXCUDA_UNARY(op_relu, 7)
LUXCUDA_UNARY(op_gelu, 8)
LUXCUDA_UNARY(op_copy, 9)
#undef LUXCUDA_UNARY

LuxBackendError op_transpose(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, int rows, int cols) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!c || !bi || !bo || rows < 0 || cols < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t bytes = (size_t)rows * cols * sizeof(float);
    if (bytes > bi->bytes || bytes > bo->bytes) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_transpose_f32((const float*)bi->ptr, (float*)bo->ptr, rows, cols, c->stream));
    c->launches++;
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}

// outer rows of inner elements -> outer results
LuxBackendError reduce_rows(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t outer, size_t inner, int op) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!c || !bi || !bo || outer * inner * sizeof(float) > bi->bytes || outer * sizeof(float) > bo->bytes)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_reduce_rows_f32(op, (const float*)bi->ptr, (float*)bo->ptr, outer, inner, c->stream));
    c->launches++;
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
LuxBackendError op_reduce_sum(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return reduce_rows(c, i, o, 1, n, 0); }
LuxBackendError op_reduce_max(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return reduce_rows(c, i, o, 1, n, 1); }
LuxBackendError op_reduce_min(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return reduce_rows(c, i, o, 1, n, 2); }
LuxBackendError op_reduce_mean(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t n) { return reduce_rows(c, i, o, 1, n, 3); }
LuxBackendError op_reduce_sum_axis(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t outer, size_t inner) {
    return reduce_rows(c, i, o, outer, inner, 0);
}
LuxBackendError op_reduce_max_axis(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t outer, size_t inner) {
    return reduce_rows(c, i, o, outer, inner, 1);
}

LuxBackendError softmax(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, size_t batch, size_t dim, bool log) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out);
    if (!c || !bi || !bo || batch * dim * sizeof(float) > bi->bytes || batch * dim * sizeof(float) > bo->bytes)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_softmax_f32((const float*)bi->ptr, (float*)bo->ptr, batch, dim, log, c->stream));
    c->launches++;
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
LuxBackendError op_softmax(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t b, size_t d) { return softmax(c, i, o, b, d, false); }
LuxBackendError op_log_softmax(LuxBackendContext* c, LuxBackendBuffer* i, LuxBackendBuffer* o, size_t b, size_t d) { return softmax(c, i, o, b, d, true); }

LuxBackendError op_layer_norm(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, LuxBackendBuffer* gamma,
                              LuxBackendBuffer* beta, size_t batch, size_t dim, float eps) {
    Context* c = as_ctx(ctx);
    Buffer *bi = as_buf(in), *bo = as_buf(out), *bg = gamma ? as_buf(gamma) : nullptr, *bb = beta ? as_buf(beta) : nullptr;
    if (!c || !bi || !bo || (gamma && !bg) || (beta && !bb)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (batch * dim * sizeof(float) > bi->bytes || batch * dim * sizeof(float) > bo->bytes || (bg && dim * sizeof(float) > bg->bytes) ||
        (bb && dim * sizeof(float) > bb->bytes))
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    LUX_CUDA_TRY(launch_layer_norm_f32((const float*)bi->ptr, (float*)bo->ptr, bg ? (const float*)bg->ptr : nullptr,
                                       bb ? (const float*)bb->ptr : nullptr, batch, dim, eps, c->stream));
    c->launches++;
    bi->last_stream = bo->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
// op_rms_norm_f32 (backend_plugin.h:178): the row kernel of the quantized path with fp32 in and out
LuxBackendError op_rms_norm(LuxBackendContext* ctx, LuxBackendBuffer* in, LuxBackendBuffer* out, LuxBackendBuffer* weight,
                            size_t batch, size_t dim, float eps) {
    return quant_vtbl()->rms_norm(ctx, in, out, weight, batch, dim, eps, LUX_DTYPE_FLOAT32, LUX_DTYPE_FLOAT32);
}

LuxBackendError op_ntt(LuxBackendContext* ctx, uint64_t* data, size_t n, uint64_t modulus, bool inverse) {
    Context* c = as_ctx(ctx);
    if (!c || !data || n == 0 || (n & (n - 1)) != 0 || modulus < 2) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    DeviceGuard g(c->dev->device());
    c->copies++;
    LUX_CUDA_TRY(ntt_device(data, n, modulus, inverse, c->stream));
    c->launches++;
    return LUX_BACKEND_OK;
}
LuxBackendError op_ntt_forward(LuxBackendContext* c, uint64_t* d, size_t n, uint64_t m) { return op_ntt(c, d, n, m, false); }
LuxBackendError op_ntt_inverse(LuxBackendContext* c, uint64_t* d, size_t n, uint64_t m) { return op_ntt(c, d, n, m, true); }

lux_gpu_backend_vtbl g_vtbl;  // zero-initialised: every unlisted slot is NULL
std::once_flag g_vtbl_once;

void fill_vtbl() {
    std::memset(&g_vtbl, 0, sizeof(g_vtbl));
    g_vtbl.create_context = create_context;
    g_vtbl.destroy_context = destroy_context;
    g_vtbl.get_device_count = get_device_count;
    g_vtbl.get_device_info = get_device_info;
    g_vtbl.sync = sync;
    g_vtbl.buffer_alloc = buffer_alloc;
    g_vtbl.buffer_alloc_with_data = buffer_alloc_with_data;
    g_vtbl.buffer_free = buffer_free;
    g_vtbl.buffer_copy_to_host = buffer_copy_to_host;
    g_vtbl.buffer_copy_from_host = buffer_copy_from_host;
    g_vtbl.buffer_get_host_ptr = buffer_get_host_ptr;
    g_vtbl.kernel_load = kernel_load;
    g_vtbl.kernel_load_binary = kernel_load_binary;
    g_vtbl.kernel_destroy = kernel_destroy;
    g_vtbl.kernel_dispatch = kernel_dispatch;
    g_vtbl.op_add_f32 = op_add;
    g_vtbl.op_sub_f32 = op_sub;
    g_vtbl.op_mul_f32 = op_mul;
    g_vtbl.op_div_f32 = op_div;
    g_vtbl.op_matmul_f32 = op_matmul;
    g_vtbl.op_transpose_f32 = op_transpose;
    g_vtbl.op_reduce_sum_f32 = op_reduce_sum;
    g_vtbl.op_reduce_max_f32 = op_reduce_max;
    g_vtbl.op_reduce_min_f32 = op_reduce_min;
    g_vtbl.op_reduce_mean_f32 = op_reduce_mean;
    g_vtbl.op_reduce_sum_axis_f32 = op_reduce_sum_axis;
    g_vtbl.op_reduce_max_axis_f32 = op_reduce_max_axis;
    g_vtbl.op_softmax_f32 = op_softmax;
    g_vtbl.op_log_softmax_f32 = op_log_softmax;
    g_vtbl.op_exp_f32 = op_exp;
    g_vtbl.op_log_f32 = op_log;
    g_vtbl.op_sqrt_f32 = op_sqrt;
    g_vtbl.op_neg_f32 = op_neg;
    g_vtbl.op_abs_f32 = op_abs;
    g_vtbl.op_tanh_f32 = op_tanh;
    g_vtbl.op_sigmoid_f32 = op_sigmoid;
    g_vtbl.op_relu_f32 = op_relu;
    g_vtbl.op_gelu_f32 = op_gelu;
    g_vtbl.op_copy_f32 = op_copy;
    g_vtbl.op_layer_norm_f32 = op_layer_norm;
    g_vtbl.op_rms_norm_f32 = op_rms_norm;
    g_vtbl.op_ntt_forward = op_ntt_forward;
    g_vtbl.op_ntt_inverse = op_ntt_inverse;
    g_vtbl._reserved[0] = const_cast<lux_gpu_quant_vtbl*>(quant_vtbl());
}

// Directory of the kernels compiled into the library, in the format of the reference's kernel registry
// (include/lux/gpu/kernel_loader.h:70-90).  name = kernel family, entry_point = variant.
const LuxEmbeddedKernel g_kernels[] = {
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<4,m8>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},   // decode GEMV, 4-bit, M <= 8
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<4,m16>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},  // decode GEMV, 4-bit, M <= 16
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<4,m8,rms>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},   // x = rms-norm of the buffer, applied as it is loaded
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<4,m8,sum3>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},  // x = sum of three column blocks
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<8,m8>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<8,m8,rms>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<8,m8,sum3>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_mma<8,m16>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<4,m8>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},  // several decode matmuls of one shape per launch
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<4,m16>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<8,m8>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<8,m16>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<4,m8,push>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},  // the same, column-sharded: tiles stored into every rank's y
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<4,m16,push>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<8,m8,push>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_batch<8,m16,push>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmm_tc<4>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},       // prefill GEMM (tcgen05), M > 16
    {LUX_CUDA_QMM_KERNEL_NAME, "qmm_tc<8>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmm_tc<4,stream-k>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},  // the same, k-stages split evenly over the SMs
    {LUX_CUDA_QMM_KERNEL_NAME, "qmm_tc<8,stream-k>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmm_tc<4,pairs>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},     // the same on pairs of CTAs (cta_group::2)
    {LUX_CUDA_QMM_KERNEL_NAME, "qmm_tc<8,pairs>", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {LUX_CUDA_QMM_KERNEL_NAME, "qmv_simt", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},        // fp32 activations, odd K
    {"lux.qmm.dequantize", "dequantize", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {"lux.qmm.unpack", "unpack", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {"lux.qmm.quantize", "quantize", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {"lux.rms_norm", "rms_norm", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {"lux.sum3", "sum3", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
    {"lux.mul_rms_norm", "mul_rms_norm", LUX_KERNEL_LANG_CUDA, nullptr, 0, nullptr, 0},
};
const LuxKernelRegistry g_registry = {"cuda", g_kernels, sizeof(g_kernels) / sizeof(g_kernels[0])};

}  // namespace

extern "C" {

LUX_GPU_BACKEND_EXPORT const LuxKernelRegistry* lux_kernel_registry_cuda_get(void) { return &g_registry; }

LUX_GPU_BACKEND_EXPORT bool lux_gpu_backend_init(lux_gpu_backend_desc* out) {
    if (!out) return false;
    std::call_once(g_vtbl_once, fill_vtbl);
    out->abi_version = LUX_GPU_BACKEND_ABI_VERSION;
    out->backend_name = "cuda";
    out->backend_version = "0.1.0-b200";
    out->capabilities = LUX_CAP_TENSOR_OPS | LUX_CAP_MATMUL | LUX_CAP_NTT | LUX_CAP_CUSTOM_KERNELS;
    out->vtbl = &g_vtbl;
    // "false" = backend unavailable on this system: no driver, no device, or
    // not a Blackwell (sm_100) part -- the kernels are built for sm_100a only.
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return false;
    }
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, 0) != cudaSuccess || p.major != 10) {
        cudaGetLastError();
        return false;
    }
    return true;
}

LUX_GPU_BACKEND_EXPORT const lux_gpu_quant_vtbl* lux_gpu_cuda_quant_vtbl(void) { return quant_vtbl(); }

LUX_GPU_BACKEND_EXPORT void lux_gpu_cuda_abi_layout(uint32_t out[5]) {
    out[0] = (uint32_t)sizeof(lux_gpu_backend_vtbl);
    out[1] = (uint32_t)offsetof(lux_gpu_backend_vtbl, op_matmul_f32);
    out[2] = (uint32_t)offsetof(lux_gpu_backend_vtbl, op_ntt_forward);
    out[3] = (uint32_t)offsetof(lux_gpu_backend_vtbl, _reserved);
    out[4] = (uint32_t)sizeof(lux_gpu_backend_desc);
}

LUX_GPU_BACKEND_EXPORT const char* lux_gpu_cuda_last_error(void) { return luxcuda::last_error(); }

}  // extern "C"
