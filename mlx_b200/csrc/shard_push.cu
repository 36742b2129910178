// Column-sharded decode matmul whose all-gather is done by the matmul kernel itself: every rank keeps a
// full copy of y in a buffer its peers can store into ("symmetric buffer"), the decode kernel writes its
// columns into all copies over NVLink (peer pointers, plain stores) and ends when the peers' columns have
// arrived (flag words at the head of each buffer; qmv_mma.cu has the protocol).  One launch per call, no
// collective library on the data path, no interleave pass, and the launch can be recorded in a CUDA graph.
//
// Peers in other processes are reached through CUDA IPC handles, peers in the same process directly.
// The reference has no multi-device path beyond create_context(device_index)
// (include/lux/gpu/backend_plugin.h:84).
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <new>
#include <utility>
#include <vector>

#include "internal.h"

struct LuxCudaSymmBuffer {
    luxcuda::Context* ctx = nullptr;
    int rank = 0, world = 1;
    void* base = nullptr;   // cudaMalloc: [flag words, kHeader bytes][data][inbox: 2 x data]
    size_t bytes = 0;       // of the data part
    luxcuda::Buffer view;   // the data part as an ordinary (non-owning) buffer
    void* peer_base[luxcuda::kMaxShardWorld] = {};
    bool ipc_opened[luxcuda::kMaxShardWorld] = {};
    bool attached = false;
};

namespace luxcuda {

namespace {

constexpr size_t kHeader = 256;

struct Handle {  // what travels between ranks; LUX_CUDA_SYMM_HANDLE_BYTES
    uint64_t pid;
    int32_t device;
    int32_t rank;
    uint64_t ptr;
    cudaIpcMemHandle_t ipc;
    uint8_t pad[LUX_CUDA_SYMM_HANDLE_BYTES - 24 - sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(Handle) == LUX_CUDA_SYMM_HANDLE_BYTES, "handle size");

// Barrier over the ranks of a symmetric buffer, on the device: every rank bumps its count of barriers, writes
// it into its slot on every peer and waits until every peer's slot here has reached it.  One warp; the waits
// are bounded (on a time-out the host-visible error word is raised and the kernel returns).
// Flag words used: [kBarEpoch] this rank's count, [kBarSlot + q] the count announced by rank q.
constexpr int kBarEpoch = 2, kBarSlot = 32;
struct BarrierArgs {
    uint32_t* flags[kMaxShardWorld];
    int world, me;
    int* error;
    long long limit_ns;  // of a wait for a peer's count
};
__global__ void symm_barrier_kernel(const __grid_constant__ BarrierArgs a) {
    const int q = threadIdx.x;
    uint32_t* mine = a.flags[a.me];
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(mine + kBarEpoch) + 1;
    __syncwarp();
    bool ok = true;
    if (q < a.world && q != a.me) {
        __threadfence_system();  // whatever this rank stored into the peers before is out before the count
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.flags[q] + kBarSlot + a.me), "r"(e) : "memory");
        long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            uint32_t v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + kBarSlot + q) : "memory");
            if ((int32_t)(v - e) >= 0) break;
            long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > a.limit_ns) {
                ok = false;
                break;
            }
            __nanosleep(200);
        }
        __threadfence_system();
    }
    ok = __all_sync(0xffffffffu, ok);
    if (q == 0) {
        *reinterpret_cast<volatile uint32_t*>(mine + kBarEpoch) = e;
        if (!ok && a.error) *a.error = 3;
    }
}

LuxBackendError symm_alloc(LuxBackendContext* ctx, int rank, int world, size_t bytes, LuxCudaSymmBuffer** out) {
    Context* c = as_ctx(ctx);
    if (!c || !out || world < 1 || world > kMaxShardWorld || rank < 0 || rank >= world || bytes == 0)
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    auto* sb = new (std::nothrow) LuxCudaSymmBuffer();
    if (!sb) return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
    DeviceGuard g(c->dev->device());
    // a whole driver allocation of its own: that is what an IPC handle names
    const size_t data = (bytes + 255) & ~size_t(255);  // the inbox (8 bytes per 4 bytes of a peer's columns) follows
    cudaError_t e = cudaMalloc(&sb->base, kHeader + 3 * data);
    if (e == cudaSuccess) e = cudaMemset(sb->base, 0, kHeader + 3 * data);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (sb->base) cudaFree(sb->base);
        delete sb;
        return map_cuda_error(e, "symm_alloc");
    }
    sb->ctx = c;
    sb->rank = rank;
    sb->world = world;
    sb->bytes = bytes;
    sb->view.dev = c->dev;
    sb->view.block = nullptr;
    sb->view.ptr = static_cast<char*>(sb->base) + kHeader;
    sb->view.bytes = bytes;
    sb->view.last_stream = c->stream;
    sb->peer_base[rank] = sb->base;
    sb->attached = world == 1;
    *out = sb;
    return LUX_BACKEND_OK;
}

LuxBackendError symm_export(LuxCudaSymmBuffer* sb, void* handle_out) {
    if (!sb || !handle_out) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Handle h;
    memset(&h, 0, sizeof(h));
    h.pid = (uint64_t)getpid();
    h.device = sb->ctx->dev->device();
    h.rank = sb->rank;
    h.ptr = (uint64_t)(uintptr_t)sb->base;
    DeviceGuard g(sb->ctx->dev->device());
    LUX_CUDA_TRY(cudaIpcGetMemHandle(&h.ipc, sb->base));
    memcpy(handle_out, &h, sizeof(h));
    return LUX_BACKEND_OK;
}

LuxBackendError symm_attach(LuxCudaSymmBuffer* sb, const void* handles) {
    if (!sb || !handles) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (sb->attached) return LUX_BACKEND_OK;
    const int dev = sb->ctx->dev->device();
    DeviceGuard g(dev);
    for (int r = 0; r < sb->world; r++) {
        if (r == sb->rank) continue;
        Handle h;
        memcpy(&h, static_cast<const char*>(handles) + (size_t)r * sizeof(Handle), sizeof(h));
        if (h.rank != r) {
            set_last_error("symm_attach: handle %d belongs to rank %d (handles must be in rank order)", r, h.rank);
            return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        }
        if (h.pid == (uint64_t)getpid()) {  // same process: the pointer itself, once the GPUs may reach each other
            if (h.device != dev) {
                cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (e != cudaSuccess) return map_cuda_error(e, "cudaDeviceEnablePeerAccess");
            }
            sb->peer_base[r] = (void*)(uintptr_t)h.ptr;
        } else {
            LUX_CUDA_TRY(cudaIpcOpenMemHandle(&sb->peer_base[r], h.ipc, cudaIpcMemLazyEnablePeerAccess));
            sb->ipc_opened[r] = true;
        }
    }
    sb->attached = true;
    // A rank that once gave up on a peer stops waiting for peers for good; a fresh attachment is a fresh start.
    LUX_CUDA_TRY(reset_peer_lost());
    return LUX_BACKEND_OK;
}

LuxBackendBuffer* symm_buffer(LuxCudaSymmBuffer* sb) {
    return sb ? reinterpret_cast<LuxBackendBuffer*>(&sb->view) : nullptr;
}

// The caller makes sure no peer still stores into the buffer (all ranks past their last call).
void symm_free(LuxCudaSymmBuffer* sb) {
    if (!sb) return;
    DeviceGuard g(sb->ctx->dev->device());
    cudaStreamSynchronize(sb->ctx->stream);
    for (int r = 0; r < sb->world; r++)
        if (sb->ipc_opened[r]) cudaIpcCloseMemHandle(sb->peer_base[r]);
    cudaFree(sb->base);
    delete sb;
}

// One decode launch that delivers this rank's columns of the y at byte offset `yoff` of the symmetric buffer into
// every rank's copy (the caller holds the context's lock and has checked the buffers).  The inbox of a y lies at
// twice its offset in the inbox area, so outputs that do not overlap have inboxes that do not overlap.
LuxBackendError push_decode_at(LuxCudaSymmBuffer* sb, const QmmArgs& a, size_t yoff) {
    Context* c = sb->ctx;
    if (!qmv_mma_supported(a, c->dev->sm_count)) {
        set_last_error("qmatmul_sharded_push: shape not taken by the decode kernel (K must be a multiple of %d)", 1024 / a.bits);
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    LuxBackendError le = ensure_qmv_workspace(c, qmv_mma_workspace_bytes(a, c->dev->sm_count));
    if (le != LUX_BACKEND_OK) return le;
    ShardPush sp;
    sp.world = sb->world;
    sp.me = sb->rank;
    sp.ld = a.N * sb->world;
    sp.col0 = sb->rank * a.N;
    sp.inbox_off = ((sb->bytes + 255) & ~size_t(255)) + yoff;  // from the y at yoff: (inbox area - yoff) + 2 * yoff
    for (int r = 0; r < sb->world; r++) {
        sp.flags[r] = static_cast<uint32_t*>(sb->peer_base[r]);
        sp.y[r] = static_cast<char*>(sb->peer_base[r]) + kHeader + yoff;
    }
    QmmArgs local = a;
    local.y = static_cast<char*>(sb->view.ptr) + yoff;
    QmmArgs whole = local;  // what the launch writes, for the chain bookkeeping: every column of the local copy
    whole.N = sp.ld;
    const char* name = "";
    cudaError_t e = launch_qmv_mma(local, c->qmv_ws->ptr, c->dev->sm_count, c->stream, &name, decode_may_overlap(c, local), &sp);
    if (e == cudaErrorNotSupported && a.pro) {
        cudaGetLastError();
        set_last_error("qmatmul_sharded_push_pro: the prologue needs M <= 8, no K split, and for the rms-norm K within 16 k-blocks of 128 packed bytes");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    if (e != cudaSuccess) return map_cuda_error(e, name);
    c->last_kernel = name;
    c->launches++;
    note_decode_launch(c, whole);
    return LUX_BACKEND_OK;
}

LuxBackendError qmatmul_sharded_push(LuxCudaSymmBuffer* sb, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                                     LuxBackendBuffer* biases, int M, int K, int Nl, int bits, int group,
                                     LuxBackendDtype y_dtype) {
    if (!sb) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Context* c = sb->ctx;
    Buffer *bx = as_buf(x), *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases);
    if (!bx || !bw || !bs || !bb) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (y_dtype != LUX_DTYPE_BFLOAT16 && y_dtype != LUX_DTYPE_FLOAT32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!sb->attached) {
        set_last_error("qmatmul_sharded_push: symm_attach has not been called");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (M < 1 || Nl < 1 || (Nl & 15) || K < 1 || (bits != 4 && bits != 8) ||
        (group != 32 && group != 64 && group != 128) || K % group) {
        set_last_error("qmatmul_sharded_push: needs M >= 1, N_local a multiple of 16, bits 4|8, group 32|64|128");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    const size_t ys = y_dtype == LUX_DTYPE_BFLOAT16 ? 2 : 4;
    const size_t ld = (size_t)Nl * sb->world;
    if ((size_t)M * K * 2 > bx->bytes || (size_t)Nl * K * bits / 8 > bw->bytes || (size_t)Nl * (K / group) * 2 > bs->bytes ||
        (size_t)Nl * (K / group) * 2 > bb->bytes || (size_t)M * ld * ys > sb->bytes) {
        set_last_error("qmatmul_sharded_push: a buffer is smaller than its shape needs");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    QmmArgs a{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, sb->view.ptr, M, K, Nl, bits, group,
              LUX_DTYPE_BFLOAT16, LUX_DTYPE_BFLOAT16, (int)y_dtype};
    a.error = c->err_dev;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    if (M > 16) {
        // Prefill: the tcgen05 GEMM stores every tile into all ranks' copies of y from its epilogue, so the
        // transfer runs under the remaining tiles.  A device-side barrier over the ranks before it (every rank
        // is done reading its y of the previous call) and one after it (every rank's tiles have landed).
        if (!qmm_tc_supported(a, c->dev->sm_count)) {
            set_last_error("qmatmul_sharded_push: shape not taken by the prefill kernel (K must be a multiple of 64)");
            return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        }
        ShardPush sp;
        sp.world = sb->world;
        sp.me = sb->rank;
        sp.ld = (int)ld;
        sp.col0 = sb->rank * Nl;
        BarrierArgs ba;
        ba.world = sb->world;
        ba.me = sb->rank;
        ba.error = c->err_dev ? c->err_dev : device_error_word();
        ba.limit_ns = peer_wait_limit_ns();
        for (int r = 0; r < kMaxShardWorld; r++) ba.flags[r] = nullptr;
        for (int r = 0; r < sb->world; r++) {
            sp.y[r] = static_cast<char*>(sb->peer_base[r]) + kHeader;
            ba.flags[r] = static_cast<uint32_t*>(sb->peer_base[r]);
        }
        const char* name = "";
        if (sb->world > 1) {
            symm_barrier_kernel<<<1, 32, 0, c->stream>>>(ba);
            LUX_CUDA_TRY(cudaGetLastError());
        }
        LuxBackendError le = ensure_qmm_workspace(c);
        if (le != LUX_BACKEND_OK) return le;
        cudaError_t e = launch_qmm_tc(a, c->qmm_ws->ptr, c->dev->sm_count, c->stream, &name, &sp);
        if (e != cudaSuccess) return map_cuda_error(e, name);
        if (sb->world > 1) {
            symm_barrier_kernel<<<1, 32, 0, c->stream>>>(ba);
            LUX_CUDA_TRY(cudaGetLastError());
        }
        c->last_kernel = name;
        c->launches += sb->world > 1 ? 3 : 1;
        bx->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = sb->view.last_stream = c->stream;
        return LUX_BACKEND_OK;
    }
    LuxBackendError le = push_decode_at(sb, a, 0);
    if (le == LUX_BACKEND_OK) bx->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = sb->view.last_stream = c->stream;
    return le;
}

LuxBackendError qmatmul_sharded_push_pro(LuxCudaSymmBuffer* sb, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales,
                                         LuxBackendBuffer* biases, int M, int K, int Nl, int bits, int group, LuxBackendDtype y_dtype,
                                         int prologue, size_t x_ld, float eps) {
    if (!sb) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    Context* c = sb->ctx;
    Buffer *bx = as_buf(x), *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases);
    if (!bx || !bw || !bs || !bb) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (y_dtype != LUX_DTYPE_BFLOAT16 && y_dtype != LUX_DTYPE_FLOAT32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (prologue != LUX_CUDA_PRO_RMS_NORM && prologue != LUX_CUDA_PRO_SUM3) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!sb->attached) {
        set_last_error("qmatmul_sharded_push_pro: symm_attach has not been called");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (M < 1 || M > 8 || Nl < 1 || (Nl & 15) || K < 1 || (bits != 4 && bits != 8) ||
        (group != 32 && group != 64 && group != 128) || K % group) {
        set_last_error("qmatmul_sharded_push_pro: needs 1 <= M <= 8, N_local a multiple of 16, bits 4|8, group 32|64|128");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    const size_t ys = y_dtype == LUX_DTYPE_BFLOAT16 ? 2 : 4;
    const size_t ld = (size_t)Nl * sb->world;
    const size_t need_ld = prologue == LUX_CUDA_PRO_SUM3 ? (size_t)3 * K : (size_t)K;
    if (x_ld < need_ld || (x_ld & 7) || ((size_t)(M - 1) * x_ld + need_ld) * 2 > bx->bytes || (size_t)Nl * K * bits / 8 > bw->bytes ||
        (size_t)Nl * (K / group) * 2 > bs->bytes || (size_t)Nl * (K / group) * 2 > bb->bytes || (size_t)M * ld * ys > sb->bytes) {
        set_last_error("qmatmul_sharded_push_pro: a buffer is smaller than its shape needs (x is [M][x_ld], x_ld a multiple of 8)");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    QmmArgs a{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, sb->view.ptr, M, K, Nl, bits, group,
              LUX_DTYPE_BFLOAT16, LUX_DTYPE_BFLOAT16, (int)y_dtype};
    a.pro = prologue;
    a.x_ld = (int)x_ld;
    a.eps = eps;
    a.error = c->err_dev;
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    LuxBackendError le = push_decode_at(sb, a, 0);
    if (le == LUX_BACKEND_OK) bx->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = sb->view.last_stream = c->stream;
    return le;
}

// n independent decode matmuls of one column-sharded shape, their outputs at given offsets of the symmetric buffer
LuxBackendError qmatmul_sharded_push_batch(LuxCudaSymmBuffer* sb, int n, LuxBackendBuffer* const* x, LuxBackendBuffer* const* wq,
                                           LuxBackendBuffer* const* scales, LuxBackendBuffer* const* biases, const size_t* y_offset,
                                           const int* M, int K, int Nl, int bits, int group, LuxBackendDtype y_dtype) {
    if (!sb || n < 0 || (n > 0 && (!x || !wq || !scales || !biases || !y_offset || !M))) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (n == 0) return LUX_BACKEND_OK;
    Context* c = sb->ctx;
    if (y_dtype != LUX_DTYPE_BFLOAT16 && y_dtype != LUX_DTYPE_FLOAT32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (!sb->attached) {
        set_last_error("qmatmul_sharded_push_batch: symm_attach has not been called");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    if (Nl < 1 || (Nl & 15) || K < 1 || (bits != 4 && bits != 8) || (group != 32 && group != 64 && group != 128) || K % group) {
        set_last_error("qmatmul_sharded_push_batch: needs N_local a multiple of 16, bits 4|8, group 32|64|128");
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    const size_t ys = y_dtype == LUX_DTYPE_BFLOAT16 ? 2 : 4;
    const size_t ld = (size_t)Nl * sb->world;
    std::vector<QmmArgs> items((size_t)n);
    std::vector<std::pair<size_t, size_t>> spans((size_t)n);  // [offset, end) of every output
    for (int i = 0; i < n; i++) {
        Buffer *bx = as_buf(x[i]), *bw = as_buf(wq[i]), *bs = as_buf(scales[i]), *bb = as_buf(biases[i]);
        if (!bx || !bw || !bs || !bb) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        if (M[i] < 1 || M[i] > 16) {
            set_last_error("qmatmul_sharded_push_batch: item %d has M = %d (1..16 rows of x per item)", i, M[i]);
            return LUX_BACKEND_ERROR_NOT_SUPPORTED;
        }
        const size_t ybytes = (size_t)M[i] * ld * ys;
        if ((size_t)M[i] * K * 2 > bx->bytes || (size_t)Nl * K * bits / 8 > bw->bytes || (size_t)Nl * (K / group) * 2 > bs->bytes ||
            (size_t)Nl * (K / group) * 2 > bb->bytes || (y_offset[i] & 15) || y_offset[i] > sb->bytes || ybytes > sb->bytes - y_offset[i]) {
            set_last_error("qmatmul_sharded_push_batch: item %d: a buffer is smaller than its shape needs, or its output "
                           "does not lie inside the symmetric buffer at a multiple of 16 bytes", i);
            return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        }
        spans[i] = {y_offset[i], y_offset[i] + ybytes};
        items[i] = QmmArgs{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, static_cast<char*>(sb->view.ptr) + y_offset[i],
                           M[i], K, Nl, bits, group, LUX_DTYPE_BFLOAT16, LUX_DTYPE_BFLOAT16, (int)y_dtype};
        items[i].error = c->err_dev;
    }
    {
        std::vector<std::pair<size_t, size_t>> sorted = spans;
        std::sort(sorted.begin(), sorted.end());
        for (int i = 1; i < n; i++)
            if (sorted[i].first < sorted[i - 1].second) {
                set_last_error("qmatmul_sharded_push_batch: two outputs overlap");
                return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
            }
    }
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    ShardPush sp;
    sp.world = sb->world;
    sp.me = sb->rank;
    sp.ld = (int)ld;
    sp.col0 = sb->rank * Nl;
    sp.inbox_off = (sb->bytes + 255) & ~size_t(255);
    for (int r = 0; r < sb->world; r++) {
        sp.flags[r] = static_cast<uint32_t*>(sb->peer_base[r]);
        sp.y[r] = static_cast<char*>(sb->peer_base[r]) + kHeader;
    }
    // items with M <= 8 and with M > 8 are different instantiations: one sequence of launches each, in item order
    for (int side = 0; side < 2; side++) {
        std::vector<QmmArgs> part;
        std::vector<int> idx;
        for (int i = 0; i < n; i++)
            if ((M[i] > 8) == (side == 1)) {
                part.push_back(items[i]);
                idx.push_back(i);
            }
        for (size_t lo = 0; lo < part.size(); lo += (size_t)qmv_batch_max()) {
            const int cnt = (int)std::min(part.size() - lo, (size_t)qmv_batch_max());
            const char* name = "";
            cudaError_t e = launch_qmv_batch(part.data() + lo, cnt, c->dev->sm_count, c->stream, &name, &sp);
            if (e == cudaErrorNotSupported) {  // K split over CTAs, ...: one push per item
                cudaGetLastError();
                for (int j = 0; j < cnt; j++) {
                    LuxBackendError le = push_decode_at(sb, part[lo + j], y_offset[idx[lo + j]]);
                    if (le != LUX_BACKEND_OK) return le;
                }
                continue;
            }
            if (e != cudaSuccess) return map_cuda_error(e, name);
            c->last_kernel = name;
            c->launches++;  // (not noted as a decode launch: the next decode kernel does not start under it)
        }
    }
    for (int i = 0; i < n; i++)
        as_buf(x[i])->last_stream = as_buf(wq[i])->last_stream = as_buf(scales[i])->last_stream = as_buf(biases[i])->last_stream = c->stream;
    sb->view.last_stream = c->stream;
    return LUX_BACKEND_OK;
}

}  // namespace

void fill_symm_entries(lux_gpu_quant_vtbl* t) {
    t->symm_alloc = symm_alloc;
    t->symm_export = symm_export;
    t->symm_attach = symm_attach;
    t->symm_buffer = symm_buffer;
    t->symm_free = symm_free;
    t->qmatmul_sharded_push = qmatmul_sharded_push;
    t->qmatmul_sharded_push_batch = qmatmul_sharded_push_batch;
    t->qmatmul_sharded_push_pro = qmatmul_sharded_push_pro;
}

}  // namespace luxcuda
