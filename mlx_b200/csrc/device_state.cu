// Per-device state of the plugin: the caching device allocator that replaces
// the reference CPU backend's malloc/free buffers (src/cpu_backend.cpp:121-146),
// the stream pool, and the error plumbing.
#include <cstdarg>
#include <cstring>

#include "internal.h"

namespace luxcuda {

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
static thread_local char t_err[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    if (getenv("LUXCUDA_TRACE")) fprintf(stderr, "luxcuda: %s\n", t_err);
}
const char* last_error() { return t_err; }

LuxBackendError map_cuda_error(cudaError_t e, const char* what) {
    set_last_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    switch (e) {
        case cudaErrorMemoryAllocation: return LUX_BACKEND_ERROR_OUT_OF_MEMORY;
        case cudaErrorInvalidValue:
        case cudaErrorInvalidDevice: return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
        case cudaErrorNoDevice:
        case cudaErrorDevicesUnavailable:
        case cudaErrorECCUncorrectable:
        case cudaErrorHardwareStackError:
        case cudaErrorIllegalAddress:
        case cudaErrorLaunchFailure: return LUX_BACKEND_ERROR_DEVICE_LOST;
        default: return LUX_BACKEND_ERROR_INTERNAL;
    }
}

// ---------------------------------------------------------------------------
// DeviceState
// ---------------------------------------------------------------------------
static std::mutex g_dev_mu;
static std::map<int, std::weak_ptr<DeviceState>> g_devs;

std::shared_ptr<DeviceState> device_state(int device, cudaError_t* err) {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    auto it = g_devs.find(device);
    if (it != g_devs.end()) {
        if (auto sp = it->second.lock()) return sp;
    }
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e == cudaSuccess && (device < 0 || device >= count)) e = cudaErrorInvalidDevice;
    if (e != cudaSuccess) {
        if (err) *err = e;
        return nullptr;
    }
    std::shared_ptr<DeviceState> sp;
    try {
        sp = std::make_shared<DeviceState>(device);
    } catch (...) {
        if (err) *err = cudaErrorUnknown;
        return nullptr;
    }
    g_devs[device] = sp;
    return sp;
}

DeviceState::DeviceState(int device) : device_(device) {
    DeviceGuard g(device);
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) throw 1;
    sm_count = prop.multiProcessorCount;
    l2_bytes = (size_t)prop.l2CacheSize;
    smem_optin = prop.sharedMemPerBlockOptin;
}

DeviceState::~DeviceState() {
    // Runs when the last context and the last buffer of the device are gone
    // (or at process exit, when the driver may already be shutting down: all
    // calls below tolerate failure).
    DeviceGuard g(device_);
    if (!g.ok) return;
    for (auto& kv : free_) {
        if (kv.second->has_event) cudaEventDestroy(kv.second->idle);
        cudaFree(kv.second->ptr);
        delete kv.second;
    }
    if (flush_) cudaFree(flush_);
    for (auto s : all_streams_) cudaStreamDestroy(s);
}

size_t DeviceState::round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    if (bytes < (1u << 20)) return (bytes + 511) & ~size_t(511);
    const size_t big = size_t(2) << 20;
    return (bytes + big - 1) / big * big;
}

Block* DeviceState::acquire(size_t bytes, cudaStream_t stream, cudaError_t* err) {
    const size_t want = round_size(bytes);
    Block* b = nullptr;
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = free_.lower_bound(want);
        if (it != free_.end()) {
            const size_t limit = want < (1u << 20) ? want * 2 : want + want / 4;
            if (it->first <= limit) {
                b = it->second;
                free_.erase(it);
            }
        }
        if (b) in_use_ += b->size;
    }
    DeviceGuard g(device_);
    if (b) {
        if (b->has_event && b->last_stream != stream) {
            cudaError_t e = cudaStreamWaitEvent(stream, b->idle, 0);
            if (e != cudaSuccess) {  // cannot order: fall back to a full wait
                cudaEventSynchronize(b->idle);
            }
        }
        b->last_stream = stream;
        return b;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        trim();  // give cached blocks back and retry once
        e = cudaMalloc(&p, want);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (err) *err = e;
        return nullptr;
    }
    b = new Block();
    b->ptr = p;
    b->size = want;
    b->last_stream = stream;
    std::lock_guard<std::mutex> lk(mu_);
    reserved_ += want;
    in_use_ += want;
    driver_allocs_++;
    return b;
}

void DeviceState::release(Block* b, cudaStream_t stream) {
    if (!b) return;
    {
        DeviceGuard g(device_);
        if (!b->has_event) b->has_event = cudaEventCreateWithFlags(&b->idle, cudaEventDisableTiming) == cudaSuccess;
        if (b->has_event && stream) {
            if (cudaEventRecord(b->idle, stream) != cudaSuccess) {
                cudaGetLastError();
                cudaStreamSynchronize(stream);
            }
            b->last_stream = stream;
        }
    }
    std::lock_guard<std::mutex> lk(mu_);
    in_use_ -= b->size;
    free_.emplace(b->size, b);
}

void DeviceState::trim() {
    std::multimap<size_t, Block*> victims;
    {
        std::lock_guard<std::mutex> lk(mu_);
        victims.swap(free_);
        for (auto& kv : victims) reserved_ -= kv.first;
    }
    DeviceGuard g(device_);
    for (auto& kv : victims) {
        if (kv.second->has_event) {
            cudaEventSynchronize(kv.second->idle);
            cudaEventDestroy(kv.second->idle);
        }
        cudaFree(kv.second->ptr);
        delete kv.second;
    }
}

void DeviceState::stats(uint64_t* reserved, uint64_t* in_use, uint64_t* driver_allocs) {
    std::lock_guard<std::mutex> lk(mu_);
    if (reserved) *reserved = reserved_;
    if (in_use) *in_use = in_use_;
    if (driver_allocs) *driver_allocs = driver_allocs_;
}

cudaStream_t DeviceState::acquire_stream() {
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (!stream_pool_.empty()) {
            cudaStream_t s = stream_pool_.back();
            stream_pool_.pop_back();
            return s;
        }
    }
    DeviceGuard g(device_);
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(mu_);
    all_streams_.push_back(s);
    return s;
}

void DeviceState::release_stream(cudaStream_t s) {
    if (!s) return;
    std::lock_guard<std::mutex> lk(mu_);
    stream_pool_.push_back(s);
}

void* DeviceState::flush_buffer(size_t* bytes, cudaError_t* err) {
    std::lock_guard<std::mutex> lk(mu_);
    if (!flush_) {
        DeviceGuard g(device_);
        size_t want = l2_bytes ? 2 * l2_bytes : (size_t(256) << 20);
        if (want < (size_t(256) << 20)) want = size_t(256) << 20;
        cudaError_t e = cudaMalloc(&flush_, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            flush_ = nullptr;
            if (err) *err = e;
            return nullptr;
        }
        flush_bytes_ = want;
    }
    if (bytes) *bytes = flush_bytes_;
    return flush_;
}

}  // namespace luxcuda
