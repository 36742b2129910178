// Internal types of the CUDA backend plugin: per-device state (caching
// allocator, stream pool), contexts, buffers, and the launch interfaces of the
// kernels.  Nothing here crosses the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "lux_cuda_quant.h"

namespace luxcuda {

// ---------------------------------------------------------------------------
// error plumbing: CUDA errors never escape as exceptions; they become a
// LuxBackendError and a thread-local message.
// ---------------------------------------------------------------------------
void set_last_error(const char* fmt, ...);
const char* last_error();
LuxBackendError map_cuda_error(cudaError_t e, const char* what);

#define LUX_CUDA_TRY(expr)                                                        \
    do {                                                                          \
        cudaError_t _e = (expr);                                                  \
        if (_e != cudaSuccess) return ::luxcuda::map_cuda_error(_e, #expr);       \
    } while (0)

// ---------------------------------------------------------------------------
// Per-device state.  Shared (ref-counted) by every context and every buffer of
// that device, so a buffer outlives the context that allocated it: the core
// frees tensors after it has destroyed their context (src/gpu_core.cpp:216-233).
// ---------------------------------------------------------------------------
struct Block {
    void* ptr = nullptr;
    size_t size = 0;
    cudaStream_t last_stream = nullptr;  // stream the block was last used on
    cudaEvent_t idle = nullptr;          // recorded on last_stream when the block was freed
    bool has_event = false;
};

class DeviceState {
public:
    explicit DeviceState(int device);
    ~DeviceState();
    DeviceState(const DeviceState&) = delete;

    int device() const { return device_; }

    // Caching allocator.  Sizes are rounded to 512 B below 1 MiB and to 2 MiB
    // above; a freed block is kept and handed to the next request of a fitting
    // size (at most 25 % slack for large blocks).  Reuse on another stream
    // first waits for the event recorded at free time.
    Block* acquire(size_t bytes, cudaStream_t stream, cudaError_t* err);
    void release(Block* b, cudaStream_t stream);
    void trim();
    void stats(uint64_t* reserved, uint64_t* in_use, uint64_t* driver_allocs);

    cudaStream_t acquire_stream();
    void release_stream(cudaStream_t s);

    // L2 flush buffer (lazy, 256 MiB)
    void* flush_buffer(size_t* bytes, cudaError_t* err);

    int sm_count = 0;
    size_t l2_bytes = 0;
    size_t smem_optin = 0;
    cudaDeviceProp prop{};

private:
    static size_t round_size(size_t bytes);
    int device_;
    std::mutex mu_;
    std::multimap<size_t, Block*> free_;
    std::vector<cudaStream_t> stream_pool_;
    std::vector<cudaStream_t> all_streams_;
    uint64_t reserved_ = 0, in_use_ = 0, driver_allocs_ = 0;
    void* flush_ = nullptr;
    size_t flush_bytes_ = 0;
};

std::shared_ptr<DeviceState> device_state(int device, cudaError_t* err);

constexpr uint32_t kCtxMagic = 0x4C435458u;  // "LCTX"
constexpr uint32_t kBufMagic = 0x4C425546u;  // "LBUF"
constexpr uint32_t kKernMagic = 0x4C4B524Eu; // "LKRN"
constexpr int kTimerSlots = 16;

struct Context {
    uint32_t magic = kCtxMagic;
    std::shared_ptr<DeviceState> dev;
    cudaStream_t stream = nullptr;
    cudaEvent_t timers[kTimerSlots] = {};
    // split-K workspace of the decode GEMV (partials + arrival counters), grown on demand
    Block* qmv_ws = nullptr;
    size_t qmv_ws_bytes = 0;
    // Outgrown workspaces stay allocated until the context goes: launches recorded in CUDA graphs keep
    // using the block they were recorded with.
    std::vector<Block*> qmv_ws_retired;
    // scratch of the prefill GEMM (partial accumulators of tiles shared between CTAs + their flags)
    Block* qmm_ws = nullptr;
    // A kernel that gives up on a bounded wait says so here (page-locked host memory mapped into the device's
    // address space, one word per context): the context's next sync / copy-to-host reads and clears it.
    int* err_host = nullptr;
    int* err_dev = nullptr;
    const char* last_kernel = "";
    std::atomic<uint64_t> launches{0};
    std::atomic<uint64_t> copies{0};  // memcpy / memset enqueues
    // Chain of decode kernels: a decode kernel may start fetching its weights while the previous kernel of
    // the stream drains (programmatic dependent launch) only if that kernel is a decode kernel of this
    // context, is the last thing the context enqueued, and does not write those weights.
    uint64_t chain_launches = ~0ull, chain_copies = 0;  // the two counters right after the last decode launch
    const char* chain_out_lo = nullptr;                 // what that launch writes
    const char* chain_out_hi = nullptr;
    bool stream_exposed = false;  // the host holds the raw stream: it may enqueue work the context cannot see
    std::mutex mu;  // one thread at a time per context
};

// The stream a buffer was last used on.  Every entry point assigns it for each buffer it reads or writes (the
// allocator orders the reuse of a freed block behind it), so the number of assignments doubles as a change
// counter: as long as it stands still, nothing has been enqueued that could have written the buffer.
struct LastStream {
    cudaStream_t stream = nullptr;
    uint64_t uses = 0;
    LastStream& operator=(cudaStream_t s) {
        stream = s;
        ++uses;
        return *this;
    }
    LastStream& operator=(const LastStream& o) {
        stream = o.stream;
        ++uses;
        return *this;
    }
    operator cudaStream_t() const { return stream; }
};

struct Buffer {
    uint32_t magic = kBufMagic;
    std::shared_ptr<DeviceState> dev;
    Block* block = nullptr;  // null for wrapped (non-owning) buffers
    void* ptr = nullptr;
    size_t bytes = 0;
    LastStream last_stream;
    // kernel_dispatch's parameter block as last read back from this buffer, valid while last_stream.uses stands
    // at params_uses (the dispatch itself does not count as a use of the parameter buffer)
    unsigned char params_copy[64] = {};
    uint64_t params_uses = ~0ull;
    bool exposed = false;  // the host holds the raw device pointer: it may write the buffer behind the plugin's back
};

struct Kernel {
    uint32_t magic = kKernMagic;
    int builtin_id = 0;  // 1 = lux.qmm.affine
};

inline Context* as_ctx(LuxBackendContext* c) {
    auto* p = reinterpret_cast<Context*>(c);
    return (p && p->magic == kCtxMagic) ? p : nullptr;
}
inline Buffer* as_buf(LuxBackendBuffer* b) {
    auto* p = reinterpret_cast<Buffer*>(b);
    return (p && p->magic == kBufMagic) ? p : nullptr;
}

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// ---------------------------------------------------------------------------
// kernel launchers (each enqueues on `stream`, returns the launch status)
// ---------------------------------------------------------------------------
struct QmmArgs {
    const void* x;
    const uint32_t* wq;
    const void* scales;
    const void* biases;
    void* y;
    int M, K, N, bits, group;
    int x_dtype, sb_dtype, y_dtype;  // LuxBackendDtype values
    // decode kernel, M <= 8, bf16: x is computed from the buffer as it is loaded (0: as it is; 1: rms-norm of each
    // row with eps; 2: bf16(sum of the column blocks [0,K), [K,2K), [2K,3K)); x_ld = row stride of the buffer)
    int pro = 0, x_ld = 0;
    float eps = 0.0f;
    // where the kernels raise a time-out of one of their bounded waits: the calling context's word (device
    // address of page-locked, mapped host memory); null: the word shared by the process
    int* error = nullptr;
};

// Column-sharded decode launch: where the finished output tiles go besides this rank's own copy of y.
// world == 1 (the default) means "not sharded".
constexpr int kMaxShardWorld = 8;
// Grid-stride helper kernels cap their grids at a few CTAs per SM of a B200 (2 x 74 SMs); they are correct for any
// count.  The matmul kernels size their grids from the device's own SM count.
constexpr int kGridCapSMs = 148;

struct ShardPush {
    int world = 1, me = 0;
    int ld = 0, col0 = 0;                   // row stride of the full y and this rank's first column (elements)
    size_t inbox_off = 0;                   // byte offset from a rank's y to its inbox (words sent by the peers)
    void* y[kMaxShardWorld] = {};           // every rank's copy of y (own copy at [me])
    uint32_t* flags[kMaxShardWorld] = {};   // every rank's flag words (see qmv_mma.cu)
};

// decode GEMV, bf16 activations: mma.sync m16n8k16 with in-register dequant
bool qmv_mma_supported(const QmmArgs& a, int sm_count);
size_t qmv_mma_workspace_bytes(const QmmArgs& a, int sm_count);
// overlap_prev: launch as a programmatic dependent of the previous kernel in the stream (see Context);
// x_stable: that previous kernel does not write x, which may then be read before the wait for it
cudaError_t launch_qmv_mma(const QmmArgs& a, void* workspace, int sm_count, cudaStream_t stream, const char** name,
                           bool overlap_prev = false, const ShardPush* push = nullptr, bool x_stable = false);
bool decode_may_overlap(const Context* c, const QmmArgs& a);
bool decode_x_stable(const Context* c, const QmmArgs& a);  // the last chain kernel's output does not overlap x
bool chain_is_open(const Context* c);  // the last thing the context enqueued is a chain kernel (decode matmul, rms-norm)
void note_chain_launch(Context* c, const void* out, size_t out_bytes);  // right after such a launch, before counting it
void note_decode_launch(Context* c, const QmmArgs& a);  // call right after a decode launch, before counting it
// decode / small-M, any supported dtype combination: CUDA cores + warp shuffles
cudaError_t launch_qmv_simt(const QmmArgs& a, cudaStream_t stream, const char** name);
// several decode matmuls of one shape (M on one side of 8) as one persistent launch; at most qmv_batch_max() items
int qmv_batch_max();
// push (column-sharded layer, world > 1): every item's y lies inside this rank's symmetric buffer and the launch
// delivers its columns to the same place of every peer's
cudaError_t launch_qmv_batch(const QmmArgs* items, int n, int sm_count, cudaStream_t stream, const char** name,
                             const ShardPush* push = nullptr);
// prefill GEMM, bf16 activations: TMA + tcgen05 + TMEM
bool qmm_tc_supported(const QmmArgs& a, int sm_count);
size_t qmm_tc_workspace_bytes(int sm_count);  // scratch of a launch (flags at its head: zero between launches)
cudaError_t launch_qmm_tc(const QmmArgs& a, void* workspace, int sm_count, cudaStream_t stream, const char** name,
                          const ShardPush* push = nullptr);
// non-zero once a kernel gave up on one of its bounded waits since the last call (clears it)
int take_device_error();
int take_context_error(Context* c);  // the context's own word, read and cleared in one atomic step
int* device_error_word();  // where kernels raise it (null if the mapped word could not be set up)
cudaError_t reset_peer_lost();    // on the current device: waits for peers are attempted again
long long peer_wait_limit_ns();  // limit of a device-side wait for a peer rank (LUXCUDA_PEER_WAIT_MS, default 2000)

cudaError_t launch_dequantize(const uint32_t* wq, const void* scales, const void* biases, void* out, int N, int K,
                              int bits, int group, int sb_dtype, int out_dtype, cudaStream_t stream);
cudaError_t launch_unpack(const uint32_t* wq, uint8_t* q, int N, int K, int bits, cudaStream_t stream);
cudaError_t launch_quantize(const float* w, uint32_t* wq, void* scales, void* biases, int N, int K, int bits,
                            int group, int sb_dtype, cudaStream_t stream);
cudaError_t launch_rms_norm(const void* in, void* out, const float* weight, size_t rows, size_t dim, float eps,
                            int in_dtype, int out_dtype, cudaStream_t stream, bool overlap_prev = false);
// decode-chain elementwise steps (bf16): sum of three column blocks; product of two column blocks + rms-norm
cudaError_t launch_sum3(const void* in, void* out, size_t rows, size_t cols, size_t ld, cudaStream_t stream, bool overlap_prev = false);
cudaError_t launch_mul_rms_norm(const void* in, void* out, size_t rows, size_t cols, size_t ld, float eps, cudaStream_t stream,
                                bool overlap_prev = false);
cudaError_t launch_gather_columns(const void* staging, void* y_full, int world, int M, int n_local, int elem_size,
                                  cudaStream_t stream);
cudaError_t launch_flush(void* buf, size_t bytes, cudaStream_t stream);

enum class BinOp { Add, Sub, Mul, Div };
cudaError_t launch_binary_f32(BinOp op, const float* a, const float* b, float* out, size_t n, cudaStream_t stream);
cudaError_t launch_matmul_f32(const float* a, const float* b, float* out, int M, int K, int N, cudaStream_t stream);
// remaining fp32 tensor ops of the base vtable (ops_tensor.cu); unary op codes: 0 exp, 1 log, 2 sqrt, 3 neg, 4 abs,
// 5 tanh, 6 sigmoid, 7 relu, 8 gelu, 9 copy; reduction op codes: 0 sum, 1 max, 2 min, 3 mean
cudaError_t launch_unary_f32(int op, const float* in, float* out, size_t n, cudaStream_t stream);
cudaError_t launch_transpose_f32(const float* in, float* out, int rows, int cols, cudaStream_t stream);
cudaError_t launch_reduce_rows_f32(int op, const float* in, float* out, size_t outer, size_t inner, cudaStream_t stream);
cudaError_t launch_softmax_f32(const float* in, float* out, size_t batch, size_t dim, bool log, cudaStream_t stream);
cudaError_t launch_layer_norm_f32(const float* in, float* out, const float* gamma, const float* beta, size_t batch, size_t dim,
                                  float eps, cudaStream_t stream);
cudaError_t ntt_device(uint64_t* host_data, size_t n, uint64_t modulus, bool inverse, cudaStream_t stream);

// extension table (quant_api.cu) and sharding (shard.cu)
const lux_gpu_quant_vtbl* quant_vtbl();
LuxBackendError qmatmul_on_stream(Context* c, const QmmArgs& a);
void fill_shard_entries(lux_gpu_quant_vtbl* t);
void fill_symm_entries(lux_gpu_quant_vtbl* t);
LuxBackendError ensure_qmv_workspace(Context* c, size_t bytes);  // scratch of the decode kernel, grown on demand
LuxBackendError ensure_qmm_workspace(Context* c);                // scratch of the prefill GEMM, created on first use

}  // namespace luxcuda
