// The remaining fp32 tensor ops of the base vtable (include/lux/gpu/backend_plugin.h:130-178) that the
// core's public API forwards to a backend (src/gpu_core.cpp:430-789): transpose, reductions, softmax,
// unary maps, copy, layer-norm.  The reference CPU backend leaves these slots NULL
// (src/cpu_backend.cpp:333-374); their arithmetic follows the reference's CPU kernels
// (kernels/cpu/tensor_ops.c:144-290, 336-356, 358-464, 470-544).  Simple, correct kernels: they are not on
// the quantized-matmul path and are not tuned.  Row-wise ops use one block per row; a full reduction runs
// in one block so that its summation order is fixed.
#include <cfloat>

#include "internal.h"

namespace luxcuda {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float unary_apply(int op, float x) {
    switch (op) {
        case 0: return expf(x);
        case 1: return logf(x);
        case 2: return sqrtf(x);
        case 3: return -x;
        case 4: return fabsf(x);
        case 5: return tanhf(x);
        case 6: return 1.0f / (1.0f + expf(-x));
        case 7: return x > 0.0f ? x : 0.0f;
        case 8: {  // tanh form, constants of kernels/cpu/tensor_ops.c:277-287
            const float x3 = x * x * x;
            return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x3)));
        }
        default: return x;  // copy
    }
}
__global__ void unary_f32_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n, int op) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = unary_apply(op, in[i]);
}

__global__ void transpose_f32_kernel(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float tile[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y)
        if (r0 + j < rows && c < cols) tile[j][threadIdx.x] = in[(size_t)(r0 + j) * cols + c];
    __syncthreads();
    const int r = r0 + threadIdx.x, c0 = blockIdx.x * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y)
        if (c0 + j < cols && r < rows) out[(size_t)(c0 + j) * rows + r] = tile[threadIdx.x][j];
}

// op: 0 sum, 1 max, 2 min, 3 mean
__device__ __forceinline__ float red_identity(int op) { return op == 1 ? -INFINITY : (op == 2 ? INFINITY : 0.0f); }
__device__ __forceinline__ float red_combine(int op, float a, float b) { return op == 1 ? fmaxf(a, b) : (op == 2 ? fminf(a, b) : a + b); }
__device__ float block_reduce(int op, float v, float* red) {
    for (int o = 16; o; o >>= 1) v = red_combine(op, v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < blockDim.x / 32 ? red[threadIdx.x] : red_identity(op);
        for (int o = 16; o; o >>= 1) t = red_combine(op, t, __shfl_xor_sync(0xffffffffu, t, o));
        if (threadIdx.x == 0) red[0] = t;
    }
    __syncthreads();
    const float r = red[0];
    __syncthreads();
    return r;
}
// one block per row of `inner` elements; out[row] = reduction of the row
__global__ void reduce_rows_f32_kernel(const float* __restrict__ in, float* __restrict__ out, size_t inner, int op) {
    __shared__ float red[32];
    const float* row = in + (size_t)blockIdx.x * inner;
    float v = red_identity(op);
    for (size_t i = threadIdx.x; i < inner; i += blockDim.x) v = red_combine(op, v, row[i]);
    v = block_reduce(op, v, red);
    if (threadIdx.x == 0) out[blockIdx.x] = op == 3 ? (inner ? v / (float)inner : 0.0f) : v;
}

// one block per row: softmax (log = 0) or log-softmax (log = 1), kernels/cpu/tensor_ops.c:470-514
__global__ void softmax_f32_kernel(const float* __restrict__ in, float* __restrict__ out, size_t dim, int log) {
    __shared__ float red[32];
    const float* x = in + (size_t)blockIdx.x * dim;
    float* y = out + (size_t)blockIdx.x * dim;
    float m = -INFINITY;
    for (size_t i = threadIdx.x; i < dim; i += blockDim.x) m = fmaxf(m, x[i]);
    m = block_reduce(1, m, red);
    float s = 0.0f;
    for (size_t i = threadIdx.x; i < dim; i += blockDim.x) s += expf(x[i] - m);
    s = block_reduce(0, s, red);
    if (log) {
        const float ls = logf(s);
        for (size_t i = threadIdx.x; i < dim; i += blockDim.x) y[i] = x[i] - m - ls;
    } else {
        const float inv = 1.0f / s;
        for (size_t i = threadIdx.x; i < dim; i += blockDim.x) y[i] = expf(x[i] - m) * inv;
    }
}

// one block per row: y = (x - mean) / sqrt(var + eps) * gamma + beta, kernels/cpu/tensor_ops.c:520-544
__global__ void layer_norm_f32_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ gamma,
                                      const float* __restrict__ beta, size_t dim, float eps) {
    __shared__ float red[32];
    const float* x = in + (size_t)blockIdx.x * dim;
    float* y = out + (size_t)blockIdx.x * dim;
    float s = 0.0f;
    for (size_t i = threadIdx.x; i < dim; i += blockDim.x) s += x[i];
    const float mean = block_reduce(0, s, red) / (float)dim;
    float v = 0.0f;
    for (size_t i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = x[i] - mean;
        v += d * d;
    }
    const float var = block_reduce(0, v, red) / (float)dim;
    const float inv = 1.0f / sqrtf(var + eps);
    for (size_t i = threadIdx.x; i < dim; i += blockDim.x)
        y[i] = (x[i] - mean) * inv * (gamma ? gamma[i] : 1.0f) + (beta ? beta[i] : 0.0f);
}

}  // namespace

cudaError_t launch_unary_f32(int op, const float* in, float* out, size_t n, cudaStream_t stream) {
    if (!n) return cudaSuccess;
    size_t blocks = (n + kThreads - 1) / kThreads;
    if (blocks > kGridCapSMs * 16) blocks = kGridCapSMs * 16;
    unary_f32_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(in, out, n, op);
    return cudaGetLastError();
}
cudaError_t launch_transpose_f32(const float* in, float* out, int rows, int cols, cudaStream_t stream) {
    if (!rows || !cols) return cudaSuccess;
    dim3 block(32, 8), grid((cols + 31) / 32, (rows + 31) / 32);
    transpose_f32_kernel<<<grid, block, 0, stream>>>(in, out, rows, cols);
    return cudaGetLastError();
}
cudaError_t launch_reduce_rows_f32(int op, const float* in, float* out, size_t outer, size_t inner, cudaStream_t stream) {
    if (!outer) return cudaSuccess;
    reduce_rows_f32_kernel<<<(unsigned)outer, inner > 4096 ? 1024 : kThreads, 0, stream>>>(in, out, inner, op);
    return cudaGetLastError();
}
cudaError_t launch_softmax_f32(const float* in, float* out, size_t batch, size_t dim, bool log, cudaStream_t stream) {
    if (!batch || !dim) return cudaSuccess;
    softmax_f32_kernel<<<(unsigned)batch, kThreads, 0, stream>>>(in, out, dim, log ? 1 : 0);
    return cudaGetLastError();
}
cudaError_t launch_layer_norm_f32(const float* in, float* out, const float* gamma, const float* beta, size_t batch, size_t dim,
                                  float eps, cudaStream_t stream) {
    if (!batch || !dim) return cudaSuccess;
    layer_norm_f32_kernel<<<(unsigned)batch, kThreads, 0, stream>>>(in, out, gamma, beta, dim, eps);
    return cudaGetLastError();
}

}  // namespace luxcuda
