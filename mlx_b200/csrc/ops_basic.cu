// Small fp32 ops and the NTT the reference's harness exercises through the
// base vtable (test/test_core.cpp:62-144).  Correctness-first kernels: results
// are bit-identical to the CPU backend (src/cpu_backend.cpp:186-323).
#include "internal.h"

namespace luxcuda {

// ---------------------------------------------------------------------------
// elementwise (cpu_backend.cpp:186-241)
// ---------------------------------------------------------------------------
template <int OP>
__global__ void binary_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                  size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float x = a[i], y = b[i], r;
        if (OP == 0) r = __fadd_rn(x, y);
        else if (OP == 1) r = __fsub_rn(x, y);
        else if (OP == 2) r = __fmul_rn(x, y);
        else r = __fdiv_rn(x, y);
        out[i] = r;
    }
}

cudaError_t launch_binary_f32(BinOp op, const float* a, const float* b, float* out, size_t n, cudaStream_t stream) {
    const int threads = 256;
    size_t blocks = (n + threads - 1) / threads;
    if (blocks > kGridCapSMs * 16) blocks = kGridCapSMs * 16;
    switch (op) {
        case BinOp::Add: binary_f32_kernel<0><<<(unsigned)blocks, threads, 0, stream>>>(a, b, out, n); break;
        case BinOp::Sub: binary_f32_kernel<1><<<(unsigned)blocks, threads, 0, stream>>>(a, b, out, n); break;
        case BinOp::Mul: binary_f32_kernel<2><<<(unsigned)blocks, threads, 0, stream>>>(a, b, out, n); break;
        case BinOp::Div: binary_f32_kernel<3><<<(unsigned)blocks, threads, 0, stream>>>(a, b, out, n); break;
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// dense fp32 matmul, out[M,N] = A[M,K].B[K,N] (cpu_backend.cpp:243-266).
// Each output keeps ONE accumulator that walks k = 0..K-1 in order with a
// separate multiply and add, so the result equals the CPU backend's bit for
// bit; tiles of A and B go through shared memory for reuse only.
// ---------------------------------------------------------------------------
constexpr int MT = 32;
__global__ void matmul_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ out,
                                  int M, int K, int N) {
    __shared__ float As[MT][MT + 1];
    __shared__ float Bs[MT][MT + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int row = blockIdx.y * MT + ty, col = blockIdx.x * MT + tx;
    float sum = 0.0f;
    for (int k0 = 0; k0 < K; k0 += MT) {
        As[ty][tx] = (row < M && k0 + tx < K) ? A[(size_t)row * K + k0 + tx] : 0.0f;
        Bs[ty][tx] = (k0 + ty < K && col < N) ? B[(size_t)(k0 + ty) * N + col] : 0.0f;
        __syncthreads();
        const int kmax = min(MT, K - k0);
        for (int k = 0; k < kmax; k++) sum = __fadd_rn(sum, __fmul_rn(As[ty][k], Bs[k][tx]));
        __syncthreads();
    }
    if (row < M && col < N) out[(size_t)row * N + col] = sum;
}

cudaError_t launch_matmul_f32(const float* a, const float* b, float* out, int M, int K, int N, cudaStream_t stream) {
    dim3 block(MT, MT), grid((N + MT - 1) / MT, (M + MT - 1) / MT);
    matmul_f32_kernel<<<grid, block, 0, stream>>>(a, b, out, M, K, N);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// NTT (cpu_backend.cpp:34-77, 269-323): same radix-2 schedule, same root
// choice, arithmetic mod m through 128-bit products -- integer-exact, so the
// output equals the CPU backend's.  Twiddles w^j are computed by square-and-
// multiply per butterfly instead of the CPU's running product; both are exact.
// ---------------------------------------------------------------------------
__host__ __device__ inline uint64_t mulmod(uint64_t a, uint64_t b, uint64_t m) {
    return (uint64_t)(((unsigned __int128)a * b) % m);
}
__host__ __device__ inline uint64_t addmod(uint64_t a, uint64_t b, uint64_t m) {
    return (uint64_t)(((unsigned __int128)a + b) % m);
}
__host__ __device__ inline uint64_t submod(uint64_t a, uint64_t b, uint64_t m) {
    a %= m;
    b %= m;
    return a >= b ? a - b : m - (b - a);
}
__host__ __device__ inline uint64_t powmod(uint64_t base, uint64_t exp, uint64_t m) {
    uint64_t r = 1;
    base %= m;
    while (exp) {
        if (exp & 1) r = mulmod(r, base, m);
        exp >>= 1;
        base = mulmod(base, base, m);
    }
    return r;
}

__global__ void ntt_bitrev_kernel(uint64_t* data, unsigned n, int logn) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned j = __brev(i) >> (32 - logn);
    if (logn == 0) j = 0;
    if (i < j) {
        uint64_t t = data[i];
        data[i] = data[j];
        data[j] = t;
    }
}
// forward (DIT): u + w^j v, u - w^j v ; inverse (DIF): u + v, (u - v) w^j
__global__ void ntt_stage_kernel(uint64_t* data, unsigned n, unsigned len, uint64_t w, uint64_t m, bool dif) {
    unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n / 2) return;
    const unsigned half = len / 2;
    const unsigned j = t % half, i = (t / half) * len;
    const uint64_t wn = powmod(w, j, m);
    const uint64_t u = data[i + j], v = data[i + j + half];
    if (!dif) {
        const uint64_t tv = mulmod(wn, v, m);
        data[i + j] = addmod(u, tv, m);
        data[i + j + half] = submod(u, tv, m);
    } else {
        data[i + j] = addmod(u, v, m);
        data[i + j + half] = mulmod(submod(u, v, m), wn, m);
    }
}
__global__ void ntt_scale_kernel(uint64_t* data, unsigned n, uint64_t ninv, uint64_t m) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) data[i] = mulmod(data[i], ninv, m);
}

cudaError_t ntt_device(uint64_t* host_data, size_t n, uint64_t modulus, bool inverse, cudaStream_t stream) {
    if (n > (size_t(1) << 30)) return cudaErrorInvalidValue;
    // root choice of cpu_backend.cpp:72-77
    const uint64_t g = modulus == 0xFFFFFFFF00000001ull ? 7 : 3;
    const uint64_t omega = powmod(g, (modulus - 1) / n, modulus);
    int logn = 0;
    while ((size_t(1) << logn) < n) logn++;
    uint64_t* d = nullptr;
    cudaError_t e = cudaMallocAsync(&d, n * sizeof(uint64_t), stream);
    if (e != cudaSuccess) return e;
    const unsigned threads = 256, un = (unsigned)n;
    const unsigned blocks_n = (un + threads - 1) / threads, blocks_h = (un / 2 + threads - 1) / threads;
    e = cudaMemcpyAsync(d, host_data, n * sizeof(uint64_t), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess && n > 1) {
        if (!inverse) {
            ntt_bitrev_kernel<<<blocks_n, threads, 0, stream>>>(d, un, logn);
            for (size_t len = 2; len <= n; len *= 2)
                ntt_stage_kernel<<<blocks_h, threads, 0, stream>>>(d, un, (unsigned)len, powmod(omega, n / len, modulus),
                                                                   modulus, false);
        } else {
            const uint64_t omega_inv = powmod(omega, modulus - 2, modulus);
            for (size_t len = n; len >= 2; len /= 2)
                ntt_stage_kernel<<<blocks_h, threads, 0, stream>>>(d, un, (unsigned)len,
                                                                   powmod(omega_inv, n / len, modulus), modulus, true);
            ntt_bitrev_kernel<<<blocks_n, threads, 0, stream>>>(d, un, logn);
        }
        e = cudaGetLastError();
    }
    if (e == cudaSuccess && inverse)  // the CPU backend scales by n^-1 for every n, including n = 1
        ntt_scale_kernel<<<blocks_n, threads, 0, stream>>>(d, un, powmod(n % modulus, modulus - 2, modulus), modulus);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_data, d, n * sizeof(uint64_t), cudaMemcpyDeviceToHost, stream);
    cudaError_t e2 = cudaFreeAsync(d, stream);
    cudaError_t e3 = cudaStreamSynchronize(stream);
    return e != cudaSuccess ? e : (e2 != cudaSuccess ? e2 : e3);
}

// ---------------------------------------------------------------------------
// L2 flush: overwrite a buffer larger than L2
// ---------------------------------------------------------------------------
__global__ void flush_kernel(uint4* p, size_t n, unsigned v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) p[i] = make_uint4(v, v + 1, v + 2, v + 3);
}
cudaError_t launch_flush(void* buf, size_t bytes, cudaStream_t stream) {
    static unsigned ctr = 0;
    flush_kernel<<<kGridCapSMs * 8, 256, 0, stream>>>((uint4*)buf, bytes / 16, ++ctr);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// column interleave after an all-gather: staging[r][m][n_local] -> y[m][r*n_local + j]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gather_columns_kernel(const T* __restrict__ staging, T* __restrict__ y, int world, int M, int nl) {
    const size_t total = (size_t)world * M * nl;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const int j = (int)(i % nl);
        const size_t t = i / nl;
        const int m = (int)(t % M), r = (int)(t / M);
        y[(size_t)m * world * nl + (size_t)r * nl + j] = staging[i];
    }
}
cudaError_t launch_gather_columns(const void* staging, void* y_full, int world, int M, int n_local, int elem_size,
                                  cudaStream_t stream) {
    size_t total = (size_t)world * M * n_local;
    if (!total) return cudaSuccess;
    // widen to 16-byte elements when the slice width allows it
    const int per16 = 16 / elem_size;
    unsigned blocks;
    auto nblocks = [](size_t n) { size_t b = (n + 255) / 256; return (unsigned)(b > kGridCapSMs * 8 ? kGridCapSMs * 8 : b); };
    if (n_local % per16 == 0 && ((uintptr_t)staging % 16) == 0 && ((uintptr_t)y_full % 16) == 0) {
        blocks = nblocks(total / per16);
        gather_columns_kernel<uint4><<<blocks, 256, 0, stream>>>((const uint4*)staging, (uint4*)y_full, world, M, n_local / per16);
    } else if (elem_size == 2) {
        blocks = nblocks(total);
        gather_columns_kernel<uint16_t><<<blocks, 256, 0, stream>>>((const uint16_t*)staging, (uint16_t*)y_full, world, M, n_local);
    } else {
        blocks = nblocks(total);
        gather_columns_kernel<uint32_t><<<blocks, 256, 0, stream>>>((const uint32_t*)staging, (uint32_t*)y_full, world, M, n_local);
    }
    return cudaGetLastError();
}

}  // namespace luxcuda
