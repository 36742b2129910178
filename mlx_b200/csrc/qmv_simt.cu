// Quantized GEMV on CUDA cores: y[M,N] = x[M,K] . dequant(Wq[N,K])^T for the
// fp32 compute path (x fp32; w^ = fl32(fl32(s*q)+b)) and as the general
// fallback of the bf16 path (w^ = one bf16 FMA) for shapes the tensor-core
// kernels do not take.
//
// One warp owns R consecutive rows of W.  Per step every lane fetches one
// 16-byte piece of each row (32 four-bit or 16 eight-bit weights, all inside
// one quantisation group), dequantises it once, and reuses it for MB rows of
// x; x comes through L1 (it is tiny and read by every warp).  The K-sum of a
// row is split over the 32 lanes and finished with warp shuffles.  HBM-bound:
// algorithmic bytes per row = K*bits/8 + 2*(K/group)*sizeof(scale).
#include <cuda_bf16.h>

#include "internal.h"

namespace luxcuda {

namespace {

template <bool BF16>
struct XT;
template <>
struct XT<false> { using type = float; };
template <>
struct XT<true> { using type = __nv_bfloat16; };

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}


// PER consecutive activations (PER*sizeof(X) bytes, naturally aligned) as fp32
template <int PER, bool XBF16>
__device__ __forceinline__ void load_x(const void* p, float* out) {
    if (XBF16) {
        uint32_t v[PER / 2];
        if (PER == 8) {
            const uint4 t = __ldg((const uint4*)p);
            v[0] = t.x; v[1] = t.y; v[PER / 2 - 2] = t.z; v[PER / 2 - 1] = t.w;
        } else {
            const uint2 t = __ldg((const uint2*)p);
            v[0] = t.x; v[1] = t.y;
        }
#pragma unroll
        for (int i = 0; i < PER / 2; i++) {
            out[2 * i] = __uint_as_float(v[i] << 16);
            out[2 * i + 1] = __uint_as_float(v[i] & 0xFFFF0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < PER / 4; i++) {
            const float4 t = __ldg((const float4*)p + i);
            out[4 * i] = t.x; out[4 * i + 1] = t.y; out[4 * i + 2] = t.z; out[4 * i + 3] = t.w;
        }
    }
}

// BITS in {4,8}; XBF16: compute dtype; R rows per warp; MB x-rows per pass
template <int BITS, bool XBF16, int R, int MB>
__global__ void __launch_bounds__(256)
qmv_simt_kernel(const void* __restrict__ xv, const uint32_t* __restrict__ wq, const void* __restrict__ scales,
                const void* __restrict__ biases, void* __restrict__ yv, int M, int K, int N, int group,
                int sb_dtype, int y_dtype) {
    using X = typename XT<XBF16>::type;
    constexpr int KP = 128 / BITS;  // weights per 16-byte piece
    const X* x = (const X*)xv;
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int n0 = warp * R;
    if (n0 >= N) return;
    const int m0 = blockIdx.y * MB;
    const int wpr = K * BITS / 32, gpr = K / group;
    const int pieces = wpr / 4;

    float acc[R][MB];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < MB; m++) acc[r][m] = 0.0f;

    for (int p = lane; p < pieces; p += 32) {
        const int k0 = p * KP;
        uint4 wv[R];
        float s[R], b[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int n = min(n0 + r, N - 1);
            wv[r] = ldg_stream((const uint4*)(wq + (size_t)n * wpr) + p);
            const size_t gi = (size_t)n * gpr + k0 / group;
            if (sb_dtype == LUX_DTYPE_BFLOAT16) {
                s[r] = __bfloat162float(((const __nv_bfloat16*)scales)[gi]);
                b[r] = __bfloat162float(((const __nv_bfloat16*)biases)[gi]);
            } else {
                s[r] = ((const float*)scales)[gi];
                b[r] = ((const float*)biases)[gi];
            }
        }
#pragma unroll
        for (int w = 0; w < 4; w++) {
            constexpr int PER = 32 / BITS;  // weights per word
            float xr[MB][PER];
#pragma unroll
            for (int m = 0; m < MB; m++) {
                const int mm = min(m0 + m, M - 1);
                const X* xp = x + (size_t)mm * K + k0 + w * PER;
                load_x<PER, XBF16>(xp, xr[m]);
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint32_t word = w == 0 ? wv[r].x : (w == 1 ? wv[r].y : (w == 2 ? wv[r].z : wv[r].w));
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    const uint32_t q = (word >> (BITS * j)) & ((1u << BITS) - 1);
                    float wf;
                    if (XBF16) {
                        wf = __bfloat162float(__hfma(__float2bfloat16_rn((float)q), __float2bfloat16_rn(s[r]),
                                                     __float2bfloat16_rn(b[r])));
                    } else {
                        wf = __fadd_rn(__fmul_rn(s[r], (float)q), b[r]);
                    }
#pragma unroll
                    for (int m = 0; m < MB; m++) acc[r][m] = fmaf(xr[m][j], wf, acc[r][m]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < MB; m++) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && n0 + r < N && m0 + m < M) {
                const size_t idx = (size_t)(m0 + m) * N + n0 + r;
                if (y_dtype == LUX_DTYPE_BFLOAT16) ((__nv_bfloat16*)yv)[idx] = __float2bfloat16_rn(v);
                else ((float*)yv)[idx] = v;
            }
        }
}

template <int BITS, bool XBF16, int R, int MB>
cudaError_t launch_one(const QmmArgs& a, cudaStream_t stream) {
    const int warps = (a.N + R - 1) / R;
    dim3 grid((warps + 7) / 8, (a.M + MB - 1) / MB);
    qmv_simt_kernel<BITS, XBF16, R, MB><<<grid, 256, 0, stream>>>(a.x, a.wq, a.scales, a.biases, a.y, a.M, a.K, a.N,
                                                                  a.group, a.sb_dtype, a.y_dtype);
    return cudaGetLastError();
}

template <int BITS, bool XBF16>
cudaError_t launch_bits(const QmmArgs& a, cudaStream_t stream) {
    const bool wide = a.N >= 16384;
    if (a.M == 1) return wide ? launch_one<BITS, XBF16, 4, 1>(a, stream) : launch_one<BITS, XBF16, 2, 1>(a, stream);
    if (a.M == 2) return launch_one<BITS, XBF16, 2, 2>(a, stream);
    return launch_one<BITS, XBF16, 2, 4>(a, stream);
}

}  // namespace

cudaError_t launch_qmv_simt(const QmmArgs& a, cudaStream_t stream, const char** name) {
    const bool xbf16 = a.x_dtype == LUX_DTYPE_BFLOAT16;
    if (name) *name = xbf16 ? (a.bits == 4 ? "qmv_simt<4,bf16>" : "qmv_simt<8,bf16>")
                            : (a.bits == 4 ? "qmv_simt<4,f32>" : "qmv_simt<8,f32>");
    if (a.bits == 4) return xbf16 ? launch_bits<4, true>(a, stream) : launch_bits<4, false>(a, stream);
    return xbf16 ? launch_bits<8, true>(a, stream) : launch_bits<8, false>(a, stream);
}

}  // namespace luxcuda
