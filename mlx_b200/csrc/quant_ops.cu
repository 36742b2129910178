// Format-level kernels of the quantized path: unpack, dequantise (the
// bit-exactness checks of the packed format run through these), the affine
// min/max quantiser that produces the format, and the row rms-norm used
// between the projections of a layer chain.  None of them is the hot path;
// they are written for exactness and coalesced access, not for peak speed.
#include <cuda_bf16.h>

#include "dequant.cuh"
#include "internal.h"

namespace luxcuda {

__device__ __forceinline__ uint32_t unpack_q(const uint32_t* __restrict__ row, int k, int bits) {
    return bits == 4 ? (row[k >> 3] >> (4 * (k & 7))) & 0xFu : (row[k >> 2] >> (8 * (k & 3))) & 0xFFu;
}
__device__ __forceinline__ float load_sb(const void* p, size_t i, int dtype) {
    return dtype == LUX_DTYPE_BFLOAT16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// one thread per packed word: 8 (4-bit) or 4 (8-bit) outputs, contiguous
__global__ void unpack_kernel(const uint32_t* __restrict__ wq, uint8_t* __restrict__ q, size_t words, int bits) {
    size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; w < words; w += stride) {
        const uint32_t v = wq[w];
        if (bits == 4) {
            uint2 o;
            o.x = (v & 0xF) | ((v >> 4 & 0xF) << 8) | ((v >> 8 & 0xF) << 16) | ((v >> 12 & 0xF) << 24);
            o.y = (v >> 16 & 0xF) | ((v >> 20 & 0xF) << 8) | ((v >> 24 & 0xF) << 16) | ((v >> 28 & 0xF) << 24);
            ((uint2*)q)[w] = o;
        } else {
            ((uint32_t*)q)[w] = v;  // bytes are already in k order (little endian)
        }
    }
}
cudaError_t launch_unpack(const uint32_t* wq, uint8_t* q, int N, int K, int bits, cudaStream_t stream) {
    size_t words = (size_t)N * (K * bits / 32);
    if (!words) return cudaSuccess;
    size_t blocks = (words + 255) / 256;
    if (blocks > kGridCapSMs * 16) blocks = kGridCapSMs * 16;
    unpack_kernel<<<(unsigned)blocks, 256, 0, stream>>>(wq, q, words, bits);
    return cudaGetLastError();
}

// one thread per packed word
template <bool OUT_BF16>
__global__ void dequantize_kernel(const uint32_t* __restrict__ wq, const void* __restrict__ scales,
                                  const void* __restrict__ biases, void* __restrict__ out, int N, int K, int bits,
                                  int group, int sb_dtype) {
    const int wpr = K * bits / 32, per = 32 / bits, gpr = K / group;
    const size_t words = (size_t)N * wpr;
    size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; w < words; w += stride) {
        const int n = (int)(w / wpr), kw = (int)(w % wpr);
        const uint32_t v = wq[w];
        if (OUT_BF16) {
            // same in-register dequantiser as the matmul kernels (dequant.cuh), so the
            // bit-exactness check of the dequantised weights covers their arithmetic
            const size_t gi = (size_t)n * gpr + (kw * per) / group;
            const uint32_t s = ((const uint16_t*)scales)[gi], b = ((const uint16_t*)biases)[gi];
            __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)n * K + (size_t)kw * per;
            const bool fast = scale_fast_ok(s);
            if (bits == 4) {
                uint32_t r[4];
                if (fast) dequant4_fast(v, scale_x2_133(s), scale_x2_129(s), dup_bf16(b), r);
                else dequant4_general(v, dup_bf16(s), dup_bf16(b), r);
                for (int i = 0; i < 4; i++) {  // r[i] = (w^_i, w^_{i+4})
                    ((uint16_t*)o)[i] = (uint16_t)(r[i] & 0xFFFFu);
                    ((uint16_t*)o)[i + 4] = (uint16_t)(r[i] >> 16);
                }
            } else {
                uint32_t r[2];
                if (fast) dequant8_fast(v, scale_x2_133(s), dup_bf16(b), r);
                else dequant8_general(v, dup_bf16(s), dup_bf16(b), r);
                ((uint16_t*)o)[0] = (uint16_t)(r[0] & 0xFFFFu);  // r[0] = (w^_0, w^_2), r[1] = (w^_1, w^_3)
                ((uint16_t*)o)[2] = (uint16_t)(r[0] >> 16);
                ((uint16_t*)o)[1] = (uint16_t)(r[1] & 0xFFFFu);
                ((uint16_t*)o)[3] = (uint16_t)(r[1] >> 16);
            }
        } else {
            for (int j = 0; j < per; j++) {
                const int k = kw * per + j;
                const uint32_t q = (v >> (bits * j)) & ((1u << bits) - 1);
                const size_t gi = (size_t)n * gpr + k / group;
                const float s = load_sb(scales, gi, sb_dtype), b = load_sb(biases, gi, sb_dtype);
                ((float*)out)[(size_t)n * K + k] = __fadd_rn(__fmul_rn(s, (float)q), b);
            }
        }
    }
}
cudaError_t launch_dequantize(const uint32_t* wq, const void* scales, const void* biases, void* out, int N, int K,
                              int bits, int group, int sb_dtype, int out_dtype, cudaStream_t stream) {
    size_t words = (size_t)N * (K * bits / 32);
    if (!words) return cudaSuccess;
    size_t blocks = (words + 255) / 256;
    if (blocks > kGridCapSMs * 16) blocks = kGridCapSMs * 16;
    if (out_dtype == LUX_DTYPE_BFLOAT16)
        dequantize_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(wq, scales, biases, out, N, K, bits, group, sb_dtype);
    else
        dequantize_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(wq, scales, biases, out, N, K, bits, group, sb_dtype);
    return cudaGetLastError();
}

// one warp per group: scale = (max-min)/(2^bits-1) (1 if the group is
// constant), bias = min, both rounded to the storage dtype before
// q = clamp(rint((w - bias)/scale)) is computed.
__global__ void quantize_kernel(const float* __restrict__ w, uint32_t* __restrict__ wq, void* __restrict__ scales,
                                void* __restrict__ biases, int N, int K, int bits, int group, int sb_dtype) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int gpr = K / group;
    const size_t ngroups = (size_t)N * gpr;
    if (warp >= ngroups) return;
    const int n = (int)(warp / gpr), g = (int)(warp % gpr);
    const int E = group / 32;  // elements per lane (1, 2 or 4), contiguous
    const float* p = w + (size_t)n * K + (size_t)g * group + lane * E;
    float v[4];
    float lo = INFINITY, hi = -INFINITY;
    for (int i = 0; i < E; i++) {
        v[i] = p[i];
        lo = fminf(lo, v[i]);
        hi = fmaxf(hi, v[i]);
    }
    for (int o = 16; o; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const int qmax = (1 << bits) - 1;
    float s = __fdiv_rn(__fsub_rn(hi, lo), (float)qmax), b = lo;
    if (s == 0.0f) s = 1.0f;
    if (sb_dtype == LUX_DTYPE_BFLOAT16) {
        const __nv_bfloat16 s16 = __float2bfloat16_rn(s), b16 = __float2bfloat16_rn(b);
        if (lane == 0) {
            ((__nv_bfloat16*)scales)[warp] = s16;
            ((__nv_bfloat16*)biases)[warp] = b16;
        }
        s = __bfloat162float(s16);
        b = __bfloat162float(b16);
    } else if (lane == 0) {
        ((float*)scales)[warp] = s;
        ((float*)biases)[warp] = b;
    }
    uint32_t part = 0;
    const int per = 32 / bits;                // elements per word
    const int k0 = lane * E;                  // position inside the group
    for (int i = 0; i < E; i++) {
        float r = rintf(__fdiv_rn(__fsub_rn(v[i], b), s));
        int q = r < 0.0f ? 0 : (r > (float)qmax ? qmax : (int)r);
        part |= (uint32_t)q << (bits * ((k0 + i) % per));
    }
    const int lanes_per_word = per / E;       // 8,4,2 (4-bit) or 4,2,1 (8-bit)
    for (int o = 1; o < lanes_per_word; o <<= 1) part |= __shfl_xor_sync(0xffffffffu, part, o);
    if (lane % lanes_per_word == 0) {
        const size_t kglob = (size_t)g * group + k0;
        wq[(size_t)n * (K * bits / 32) + kglob / per] = part;
    }
}
cudaError_t launch_quantize(const float* w, uint32_t* wq, void* scales, void* biases, int N, int K, int bits,
                            int group, int sb_dtype, cudaStream_t stream) {
    size_t ngroups = (size_t)N * (K / group);
    if (!ngroups) return cudaSuccess;
    const int warps_per_block = 8;
    size_t blocks = (ngroups + warps_per_block - 1) / warps_per_block;
    quantize_kernel<<<(unsigned)blocks, warps_per_block * 32, 0, stream>>>(w, wq, scales, biases, N, K, bits, group, sb_dtype);
    return cudaGetLastError();
}

// y = x * rsqrt(mean(x^2) + eps) * w, fp32 math (kernels/cpu/tensor_ops.c:546-566).
// One 1024-thread block per row; a thread keeps its (up to kRmsCache) elements in registers between the
// sum of squares and the scaling, so a row is read once.  In a decode chain the kernel is launched as a
// programmatic dependent of the kernel before it: everything it does sits behind griddepcontrol.wait.
constexpr int kRmsThreads = 1024, kRmsCache = 16;
__global__ void __launch_bounds__(kRmsThreads) rms_norm_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                               const float* __restrict__ weight, size_t dim, float eps,
                                                               int in_dtype, int out_dtype) {
    __shared__ float red[32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t r = blockIdx.x;
    const bool cached = dim <= (size_t)kRmsThreads * kRmsCache;
    float v[kRmsCache];
    float ss = 0.0f;
    if (cached) {
#pragma unroll
        for (int j = 0; j < kRmsCache; j++) {
            const size_t i = threadIdx.x + (size_t)j * kRmsThreads;
            v[j] = i < dim ? load_sb(in, r * dim + i, in_dtype) : 0.0f;
            ss = fmaf(v[j], v[j], ss);
        }
    } else {
        for (size_t i = threadIdx.x; i < dim; i += kRmsThreads) {
            const float x = load_sb(in, r * dim + i, in_dtype);
            ss = fmaf(x, x, ss);
        }
    }
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = red[threadIdx.x];
        for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) red[0] = t;
    }
    __syncthreads();
    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(red[0], (float)dim), eps)));
    auto put = [&](size_t i, float x) {
        const float o = __fmul_rn(__fmul_rn(x, inv), weight ? weight[i] : 1.0f);
        if (out_dtype == LUX_DTYPE_BFLOAT16) ((__nv_bfloat16*)out)[r * dim + i] = __float2bfloat16_rn(o);
        else ((float*)out)[r * dim + i] = o;
    };
    if (cached) {
#pragma unroll
        for (int j = 0; j < kRmsCache; j++) {
            const size_t i = threadIdx.x + (size_t)j * kRmsThreads;
            if (i < dim) put(i, v[j]);
        }
    } else {
        for (size_t i = threadIdx.x; i < dim; i += kRmsThreads) put(i, load_sb(in, r * dim + i, in_dtype));
    }
}
cudaError_t launch_rms_norm(const void* in, void* out, const float* weight, size_t rows, size_t dim, float eps,
                            int in_dtype, int out_dtype, cudaStream_t stream, bool overlap_prev) {
    if (!rows || !dim) return cudaSuccess;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kRmsThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_prev ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, rms_norm_kernel, in, out, weight, dim, eps, in_dtype, out_dtype);
}


// ---- the two elementwise steps between the projections of a decode layer, bf16 in, bf16 out ------------
// sum3:        out[r][c] = bf16( in[r][c] + in[r][cols + c] + in[r][2*cols + c] )          (fp32 adds, left to right)
// mul_rms_norm: m[r][c]  = bf16( in[r][c] * in[r][cols + c] ),  out = rms_norm(m) as above (unit weight)
// The inputs are column blocks of one row-major buffer with row stride ld (the output of a fused q|k|v or
// gate|up projection).  One 1024-thread block per row; like rms_norm_kernel the kernels sit behind
// griddepcontrol.wait, so they can be launched as programmatic dependents in a decode chain.
__device__ __forceinline__ float bf16_at(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

__global__ void __launch_bounds__(kRmsThreads) sum3_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                           size_t cols, size_t ld) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const __nv_bfloat16* row = in + (size_t)blockIdx.x * ld;
    for (size_t c = threadIdx.x; c < cols; c += kRmsThreads) {
        const float s = __fadd_rn(__fadd_rn(bf16_at(row, c), bf16_at(row, cols + c)), bf16_at(row, 2 * cols + c));
        out[(size_t)blockIdx.x * cols + c] = __float2bfloat16_rn(s);
    }
}

__global__ void __launch_bounds__(kRmsThreads) mul_rms_norm_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                                   size_t cols, size_t ld, float eps) {
    __shared__ float red[32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const __nv_bfloat16* row = in + (size_t)blockIdx.x * ld;
    const bool cached = cols <= (size_t)kRmsThreads * kRmsCache;
    auto prod = [&](size_t c) { return __bfloat162float(__float2bfloat16_rn(__fmul_rn(bf16_at(row, c), bf16_at(row, cols + c)))); };
    float v[kRmsCache];
    float ss = 0.0f;
    if (cached) {
#pragma unroll
        for (int j = 0; j < kRmsCache; j++) {
            const size_t c = threadIdx.x + (size_t)j * kRmsThreads;
            v[j] = c < cols ? prod(c) : 0.0f;
            ss = fmaf(v[j], v[j], ss);
        }
    } else {
        for (size_t c = threadIdx.x; c < cols; c += kRmsThreads) {
            const float x = prod(c);
            ss = fmaf(x, x, ss);
        }
    }
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = red[threadIdx.x];
        for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) red[0] = t;
    }
    __syncthreads();
    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(red[0], (float)cols), eps)));
    if (cached) {
#pragma unroll
        for (int j = 0; j < kRmsCache; j++) {
            const size_t c = threadIdx.x + (size_t)j * kRmsThreads;
            if (c < cols) out[(size_t)blockIdx.x * cols + c] = __float2bfloat16_rn(__fmul_rn(v[j], inv));
        }
    } else {
        for (size_t c = threadIdx.x; c < cols; c += kRmsThreads) out[(size_t)blockIdx.x * cols + c] = __float2bfloat16_rn(__fmul_rn(prod(c), inv));
    }
}

static cudaError_t launch_row_kernel(const void* kern, void** args, size_t rows, cudaStream_t stream, bool overlap_prev) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kRmsThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_prev ? 1 : 0;
    return cudaLaunchKernelExC(&cfg, kern, args);
}
cudaError_t launch_sum3(const void* in, void* out, size_t rows, size_t cols, size_t ld, cudaStream_t stream, bool overlap_prev) {
    if (!rows || !cols) return cudaSuccess;
    void* args[] = {(void*)&in, (void*)&out, (void*)&cols, (void*)&ld};
    return launch_row_kernel((const void*)sum3_kernel, args, rows, stream, overlap_prev);
}
cudaError_t launch_mul_rms_norm(const void* in, void* out, size_t rows, size_t cols, size_t ld, float eps, cudaStream_t stream,
                                bool overlap_prev) {
    if (!rows || !cols) return cudaSuccess;
    void* args[] = {(void*)&in, (void*)&out, (void*)&cols, (void*)&ld, (void*)&eps};
    return launch_row_kernel((const void*)mul_rms_norm_kernel, args, rows, stream, overlap_prev);
}

}  // namespace luxcuda
