// Column-sharded layers: rank r of `world` owns output columns
// [r*Nl, (r+1)*Nl) of a layer (its rows of Wq / scales / biases stay resident
// on its GPU), computes its slice with the single-GPU kernels and the slices
// are all-gathered over NVLink with NCCL, then interleaved into the row-major
// y[M, world*Nl].  The reference has no multi-device path beyond
// create_context(device_index) (include/lux/gpu/backend_plugin.h:84).
//
// NCCL is resolved lazily with dlopen so the plugin loads (RTLD_NOW,
// src/plugin_loader.hpp:274) on machines without it; the sharded entry points
// then return NOT_SUPPORTED.
#include <dlfcn.h>
#include <nccl.h>

#include <new>
#include <vector>

#include "internal.h"

struct LuxCudaShardComm {
    luxcuda::Context* ctx;
    ncclComm_t comm;
    int rank, world;
};

namespace luxcuda {

namespace {

struct NcclApi {
    void* handle = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommInitAll) CommInitAll = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    bool ok = false;
};

NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* env = getenv("LUXCUDA_NCCL_LIB");
        const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
#define LUX_SYM(name) api.name = reinterpret_cast<decltype(api.name)>(dlsym(api.handle, "nccl" #name))
        LUX_SYM(GetUniqueId);
        LUX_SYM(CommInitRank);
        LUX_SYM(CommInitAll);
        LUX_SYM(CommDestroy);
        LUX_SYM(AllGather);
        LUX_SYM(GroupStart);
        LUX_SYM(GroupEnd);
        LUX_SYM(GetErrorString);
#undef LUX_SYM
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommInitAll && api.CommDestroy && api.AllGather &&
                 api.GroupStart && api.GroupEnd && api.GetErrorString;
    });
    return api;
}

LuxBackendError nccl_error(ncclResult_t r, const char* what) {
    set_last_error("%s: NCCL %s", what, nccl().GetErrorString ? nccl().GetErrorString(r) : "error");
    return r == ncclInvalidArgument || r == ncclInvalidUsage ? LUX_BACKEND_ERROR_INVALID_ARGUMENT
                                                             : LUX_BACKEND_ERROR_INTERNAL;
}
#define LUX_NCCL_TRY(expr)                                      \
    do {                                                        \
        ncclResult_t _r = (expr);                               \
        if (_r != ncclSuccess) return nccl_error(_r, #expr);    \
    } while (0)

LuxBackendError need_nccl() {
    if (nccl().ok) return LUX_BACKEND_OK;
    set_last_error("NCCL (libnccl.so.2) not found: sharded entry points unavailable");
    return LUX_BACKEND_ERROR_NOT_SUPPORTED;
}

static_assert(sizeof(ncclUniqueId) == LUX_CUDA_NCCL_UID_BYTES, "unique id size");

LuxBackendError shard_unique_id(void* out_uid) {
    if (!out_uid) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError e = need_nccl();
    if (e != LUX_BACKEND_OK) return e;
    LUX_NCCL_TRY(nccl().GetUniqueId(reinterpret_cast<ncclUniqueId*>(out_uid)));
    return LUX_BACKEND_OK;
}

LuxBackendError shard_comm_create(LuxBackendContext* ctx, int rank, int world, const void* uid, LuxCudaShardComm** out) {
    Context* c = as_ctx(ctx);
    if (!c || !out || world < 1 || rank < 0 || rank >= world || (world > 1 && !uid)) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    auto* sc = new (std::nothrow) LuxCudaShardComm{c, nullptr, rank, world};
    if (!sc) return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    if (world > 1) {
        LuxBackendError e = need_nccl();
        if (e != LUX_BACKEND_OK) {
            delete sc;
            return e;
        }
        DeviceGuard g(c->dev->device());
        ncclUniqueId id;
        memcpy(&id, uid, sizeof(id));
        ncclResult_t r = nccl().CommInitRank(&sc->comm, world, id, rank);
        if (r != ncclSuccess) {
            delete sc;
            return nccl_error(r, "ncclCommInitRank");
        }
    }
    *out = sc;
    return LUX_BACKEND_OK;
}

LuxBackendError shard_comm_create_all(LuxBackendContext** ctxs, int world, LuxCudaShardComm** out) {
    if (!ctxs || !out || world < 1) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    std::vector<int> devs(world);
    for (int r = 0; r < world; r++) {
        Context* c = as_ctx(ctxs[r]);
        if (!c) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        devs[r] = c->dev->device();
    }
    std::vector<ncclComm_t> comms(world, nullptr);
    if (world > 1) {
        LuxBackendError e = need_nccl();
        if (e != LUX_BACKEND_OK) return e;
        LUX_NCCL_TRY(nccl().CommInitAll(comms.data(), world, devs.data()));
    }
    for (int r = 0; r < world; r++) {
        out[r] = new (std::nothrow) LuxCudaShardComm{as_ctx(ctxs[r]), comms[r], r, world};
        if (!out[r]) return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    }
    return LUX_BACKEND_OK;
}

void shard_comm_destroy(LuxCudaShardComm* sc) {
    if (!sc) return;
    if (sc->comm && nccl().ok) {
        DeviceGuard g(sc->ctx->dev->device());
        cudaStreamSynchronize(sc->ctx->stream);
        nccl().CommDestroy(sc->comm);
    }
    delete sc;
}

// Inside shard_group_begin/end NCCL defers its calls to the end of the group,
// so the column interleave that must follow each all-gather is deferred too.
struct Deferred {
    Context* ctx;
    const void* staging;
    void* y;
    int world, M, nl, elem;
};
thread_local bool t_in_group = false;
thread_local std::vector<Deferred> t_deferred;

LuxBackendError run_interleave(const Deferred& d) {
    DeviceGuard g(d.ctx->dev->device());
    LUX_CUDA_TRY(launch_gather_columns(d.staging, d.y, d.world, d.M, d.nl, d.elem, d.ctx->stream));
    d.ctx->launches++;
    return LUX_BACKEND_OK;
}

LuxBackendError shard_group_begin() {
    if (t_in_group) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    LuxBackendError e = need_nccl();
    if (e != LUX_BACKEND_OK) return e;
    LUX_NCCL_TRY(nccl().GroupStart());
    t_in_group = true;
    t_deferred.clear();
    return LUX_BACKEND_OK;
}

LuxBackendError shard_group_end() {
    if (!t_in_group) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    t_in_group = false;
    ncclResult_t r = nccl().GroupEnd();
    std::vector<Deferred> todo;
    todo.swap(t_deferred);
    if (r != ncclSuccess) return nccl_error(r, "ncclGroupEnd");
    for (const auto& d : todo) {
        LuxBackendError e = run_interleave(d);
        if (e != LUX_BACKEND_OK) return e;
    }
    return LUX_BACKEND_OK;
}

LuxBackendError qmatmul_sharded(LuxCudaShardComm* sc, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                                LuxBackendBuffer* biases, LuxBackendBuffer* y_full, LuxBackendBuffer* staging, int M,
                                int K, int Nl, int bits, int group, LuxBackendDtype x_dtype, LuxBackendDtype sb_dtype,
                                LuxBackendDtype y_dtype) {
    if (!sc || !sc->ctx) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Context* c = sc->ctx;
    const lux_gpu_quant_vtbl* q = quant_vtbl();
    auto* cctx = reinterpret_cast<LuxBackendContext*>(c);
    if (sc->world == 1) return q->qmatmul(cctx, x, wq, scales, biases, y_full, M, K, Nl, bits, group, x_dtype, sb_dtype, y_dtype);
    // The library's all-gather is not recorded into CUDA graphs here: a capture of it together with the
    // plugin's kernels once hung a two-GPU run on this class of machine (cause not established), and every
    // rank would have to capture and replay the same collective sequence anyway.  Refuse instead.
    {
        DeviceGuard g(c->dev->device());
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(c->stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            set_last_error("qmatmul_sharded: not available while the context's stream is being captured into a graph; "
                           "use qmatmul_sharded_push (peer stores) inside graphs");
            return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        }
    }
    Buffer *by = as_buf(y_full), *bst = as_buf(staging);
    const size_t ys = y_dtype == LUX_DTYPE_BFLOAT16 ? 2 : (y_dtype == LUX_DTYPE_FLOAT32 ? 4 : 0);
    if (!by || !bst || !ys || M < 0 || Nl < 0) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    const size_t slice = (size_t)M * Nl * ys;
    if (slice * sc->world > by->bytes || slice * sc->world > bst->bytes) {
        set_last_error("qmatmul_sharded: y_full/staging smaller than world*M*N_local elements");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (slice == 0) return LUX_BACKEND_OK;
    // local slice straight into its place in the staging buffer (in-place all-gather)
    Buffer view = *bst;
    view.block = nullptr;
    view.ptr = (char*)bst->ptr + slice * sc->rank;
    view.bytes = slice;
    LuxBackendError e = q->qmatmul(cctx, x, wq, scales, biases, reinterpret_cast<LuxBackendBuffer*>(&view), M, K, Nl, bits,
                                   group, x_dtype, sb_dtype, y_dtype);
    if (e != LUX_BACKEND_OK) return e;
    {
        DeviceGuard g(c->dev->device());
        c->copies++;  // a library kernel the context does not count as its own: ends a chain of decode launches
        LUX_NCCL_TRY(nccl().AllGather(view.ptr, bst->ptr, slice, ncclUint8, sc->comm, c->stream));
    }
    Deferred d{c, bst->ptr, by->ptr, sc->world, M, Nl, (int)ys};
    by->last_stream = bst->last_stream = c->stream;
    if (t_in_group) {
        t_deferred.push_back(d);
        return LUX_BACKEND_OK;
    }
    return run_interleave(d);
}

}  // namespace

void fill_shard_entries(lux_gpu_quant_vtbl* t) {
    t->shard_unique_id = shard_unique_id;
    t->shard_comm_create = shard_comm_create;
    t->shard_comm_create_all = shard_comm_create_all;
    t->shard_comm_destroy = shard_comm_destroy;
    t->qmatmul_sharded = qmatmul_sharded;
    t->shard_group_begin = shard_group_begin;
    t->shard_group_end = shard_group_end;
}

}  // namespace luxcuda
