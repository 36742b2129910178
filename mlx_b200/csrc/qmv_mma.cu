// Decode-regime quantized GEMV for bf16 activations, M <= 16:
//   y[M,N] = x[M,K] . dequant(Wq[N,K])^T,  w^ = RNE_bf16(s*q + b)  (one bf16 FMA)
//
// HBM-bound: every packed weight word, scale and bias is read exactly once
// with 256-bit coalesced loads straight into registers, dequantised there and
// fed to mma.sync.m16n8k16 (bf16 x bf16 -> fp32), so the M <= 16 rows of x
// cost no extra instruction per weight.  Algorithmic bytes per output row:
// K*bits/8 + 2*(K/group)*2.
//
// Work decomposition ("task" = 16 rows of W x one k-block of KB = 1024/bits
// columns, 2 KiB of packed weights):
//   * tasks are numbered row-tile major, k-block minor; CTA c of G (one per
//     SM, persistent) takes the contiguous range [c*T/G, (c+1)*T/G), so every
//     SM streams the same number of bytes (+-1 task) whatever N is;
//   * inside a CTA the 16 warps take tasks round-robin; lane (g = lane/4,
//     t = lane%4) loads 32 contiguous bytes of row g and of row g+8, i.e. the
//     KT = 256/bits weights k = kb*KB + t*KT + [0,KT) -- one 256-bit load per
//     row, one quantisation group per load (group >= KT);
//   * the dot product is invariant under a permutation of k applied to both
//     operands, so the eight 4-bit values of a word are used in the order the
//     shift/mask unpack yields them (pairs (i, i+4)) and x is staged into
//     shared memory once per CTA in exactly that fragment order;
//   * each task leaves a 16 x 8*MT fp32 partial in shared memory; when all
//     k-blocks of a row tile are done the partials are summed in k-block order
//     (fixed order => the result does not depend on N, on the number of CTAs
//     or on how the columns of a layer are sharded over GPUs);
//   * a row tile whose k-blocks straddle two or more CTAs goes through a global
//     scratch slot: each CTA exports its partials and bumps an arrival
//     counter; the last arriver sums all of them, again in k-block order, and
//     resets the counter.  No CTA ever waits for another one.
//
// Registers hold three tasks in flight per warp (2 being loaded while 1 is
// computed): 16 warps x 2 x 2 KiB = 64 KiB of loads in flight per SM.
#include <cuda_bf16.h>

#include "internal.h"

namespace luxcuda {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
__device__ __forceinline__ uint32_t ldg_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight 4-bit values of `w` -> four bf16x2 registers, out[i] = (w^_i, w^_{i+4}).
// (w >> 4i) & 0x000F000F | 0x43004300 is the bf16 pair (128+q_i, 128+q_{i+4});
// one FMA by 1.0 with -128 recovers q exactly, one FMA applies scale and bias.
__device__ __forceinline__ void dequant4(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[4]) {
    constexpr uint32_t MASK = 0x000F000Fu, MAGIC = 0x43004300u, ONE = 0x3F803F80u, NEG128 = 0xC300C300u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t v = lop3<0xEA>(w >> (4 * i), MASK, MAGIC);  // (a & b) | c
        out[i] = fma_bf16x2(fma_bf16x2(v, ONE, NEG128), s2, b2);
    }
}
// Four 8-bit values of `w` -> two bf16x2 registers (w^_0, w^_1), (w^_2, w^_3).
// byte | 0x4B000000 is the float 2^23 + q; subtracting 2^23 gives q exactly.
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[2]) {
    const float f0 = __uint_as_float(prmt(w, 0x4B000000u, 0x7540u)) - 8388608.0f;
    const float f1 = __uint_as_float(prmt(w, 0x4B000000u, 0x7541u)) - 8388608.0f;
    const float f2 = __uint_as_float(prmt(w, 0x4B000000u, 0x7542u)) - 8388608.0f;
    const float f3 = __uint_as_float(prmt(w, 0x4B000000u, 0x7543u)) - 8388608.0f;
    uint32_t p01, p23;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p01) : "f"(f1), "f"(f0));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p23) : "f"(f3), "f"(f2));
    out[0] = fma_bf16x2(p01, s2, b2);
    out[1] = fma_bf16x2(p23, s2, b2);
}

template <int BITS, int GPT>
struct Stage {
    uint32_t w[2][8];      // rows g and g+8: 32 bytes of packed weights each
    uint32_t s[2][GPT];    // bf16 scale(s) of the lane's k-range, raw bits
    uint32_t b[2][GPT];
};

struct Params {
    const __nv_bfloat16* x;
    const uint32_t* wq;
    const __nv_bfloat16* scales;
    const __nv_bfloat16* biases;
    void* y;
    float* scratch;          // [G][nkb][128*MT] partials of row tiles shared between CTAs
    unsigned int* counters;  // [G] arrival counters (zero between launches)
    int M, K, N, group, y_bf16;
    int nkb, n_rt;
    long long T;             // n_rt * nkb tasks
};

// BITS: 4 | 8.  MT: number of 8-row blocks of x (M <= 8*MT).  GPT: groups per lane chunk (1 | 2).
template <int BITS, int MT, int GPT>
__global__ void __launch_bounds__(kThreads, 1) qmv_mma_kernel(const Params p) {
    constexpr int KT = 256 / BITS;        // weights per lane per row per task
    constexpr int KB = 4 * KT;            // k-block
    constexpr int XV = BITS == 4 ? 8 : 4; // uint4 of x per lane per task per 8-row block
    extern __shared__ __align__(16) unsigned char smem[];
    uint4* xs = reinterpret_cast<uint4*>(smem);                                   // [MT][nkb][XV][32]
    float4* part = reinterpret_cast<float4*>(smem + (size_t)MT * p.nkb * XV * 512);  // [2][nkb][MT][32]
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int G = gridDim.x, c = blockIdx.x;
    const int nkb = p.nkb;
    const long long t_begin = p.T * c / G, t_end = p.T * (c + 1) / G;
    const size_t row_bytes = (size_t)p.K * BITS / 8;
    const int gpr = p.K / p.group;

    // ---- per-warp task iterators (issue runs two tasks ahead of compute) ----
    // warp takes tasks t_begin + warp + i*kWarps
    long long tau_i = t_begin + warp;                      // next task to issue loads for
    int rt_i = (int)(tau_i / nkb), kb_i = (int)(tau_i % nkb);

    auto issue = [&](Stage<BITS, GPT>& st) {
        if (tau_i < t_end) {
            const int n0 = rt_i * 16;
            const int r0 = min(n0 + g, p.N - 1), r1 = min(n0 + g + 8, p.N - 1);
            const size_t off = (size_t)kb_i * (KB * BITS / 8) + t * 32;
            ldg256(reinterpret_cast<const unsigned char*>(p.wq) + r0 * row_bytes + off, st.w[0]);
            ldg256(reinterpret_cast<const unsigned char*>(p.wq) + r1 * row_bytes + off, st.w[1]);
            const int k0 = kb_i * KB + t * KT;
#pragma unroll
            for (int q = 0; q < GPT; q++) {
                const int gi = (k0 + q * (KT / GPT)) / p.group;
                st.s[0][q] = ldg_u16(p.scales + (size_t)r0 * gpr + gi);
                st.b[0][q] = ldg_u16(p.biases + (size_t)r0 * gpr + gi);
                st.s[1][q] = ldg_u16(p.scales + (size_t)r1 * gpr + gi);
                st.b[1][q] = ldg_u16(p.biases + (size_t)r1 * gpr + gi);
            }
        }
        tau_i += kWarps;
        kb_i += kWarps;
        while (kb_i >= nkb) {
            kb_i -= nkb;
            rt_i++;
        }
    };

    Stage<BITS, GPT> st0, st1, st2;
    issue(st0);
    issue(st1);

    // ---- stage x into shared memory in fragment order (weights already in flight) ----
    {
        const int octs_per_row = p.K / 8;
        const int total = MT * 8 * octs_per_row;
        for (int i = tid; i < total; i += kThreads) {
            const int m = i / octs_per_row, o = i - m * octs_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < p.M) v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K) + o);
            const int mt = m >> 3, gg = m & 7;
            int kb, tt, j, dst_lane;
            if (BITS == 4) {
                kb = o >> 5; tt = (o >> 3) & 3; j = o & 7;
                dst_lane = (gg * 4 + tt) ^ j;
                // order within the octet: (0,4,1,5 | 2,6,3,7)
                uint4 r;
                r.x = prmt(v.x, v.z, 0x5410u);  // x0, x4
                r.y = prmt(v.x, v.z, 0x7632u);  // x1, x5
                r.z = prmt(v.y, v.w, 0x5410u);  // x2, x6
                r.w = prmt(v.y, v.w, 0x7632u);  // x3, x7
                v = r;
            } else {
                kb = o >> 4; tt = (o >> 2) & 3; j = o & 3;
                dst_lane = (gg * 4 + tt) ^ (j * 2);
            }
            xs[(((size_t)mt * nkb + kb) * XV + j) * 32 + dst_lane] = v;
        }
    }
    __syncthreads();

    // ---- main loop ----
    long long tau_c = t_begin + warp;                      // next task to compute
    int rt_c = (int)(tau_c / nkb), kb_c = (int)(tau_c % nkb);
    const int rt_first = (int)(t_begin / nkb);
    const int rt_last = t_end > t_begin ? (int)((t_end - 1) / nkb) : rt_first - 1;
    int cur_tile = rt_first;  // next row tile whose barrier this warp has not passed yet

    // finish row tile rt: reduce the per-k-block partials in order, write y (or export)
    auto tile_end = [&](int rt) {
        const int buf = (rt - rt_first) & 1;
        __syncthreads();
        const long long base = (long long)rt * nkb;
        const int kb_lo = (int)(max(t_begin, base) - base), kb_hi = (int)(min(t_end, base + nkb) - base);
        const float* pf = reinterpret_cast<const float*>(part) + (size_t)buf * nkb * MT * 128;
        const bool whole = kb_lo == 0 && kb_hi == nkb;
        bool reduce_here = whole;
        const float* src = pf;
        size_t src_stride = (size_t)MT * 128;
        if (!whole) {
            // slot = CTA that owns the first task of the tile
            int slot = (int)(base * G / p.T);
            while (slot > 0 && p.T * slot / G > base) slot--;
            while (p.T * (slot + 1) / G <= base) slot++;
            float* sc = p.scratch + (size_t)slot * nkb * MT * 128;
            if (tid < 128 * MT)
                for (int kb = kb_lo; kb < kb_hi; kb++) __stcg(sc + (size_t)kb * MT * 128 + tid, pf[(size_t)kb * MT * 128 + tid]);
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int mine = (unsigned int)(kb_hi - kb_lo);
                const unsigned int old = atomicAdd(p.counters + slot, mine);
                s_last = (old + mine == (unsigned int)nkb);
                if (s_last) p.counters[slot] = 0;  // every contributor has arrived: safe to reset
            }
            __syncthreads();
            reduce_here = s_last != 0;
            if (reduce_here) __threadfence();
            src = sc;
        }
        if (reduce_here && tid < 128 * MT) {
            float sum = 0.0f;
            if (whole) {
                for (int kb = 0; kb < nkb; kb++) sum += src[(size_t)kb * src_stride + tid];
            } else {
                for (int kb = 0; kb < nkb; kb++) sum += __ldcg(src + (size_t)kb * src_stride + tid);
            }
            const int mt = tid >> 7, rem = tid & 127, ln = rem >> 2, ci = rem & 3;
            const int row = rt * 16 + (ln >> 2) + 8 * (ci >> 1);
            const int m = mt * 8 + 2 * (ln & 3) + (ci & 1);
            if (row < p.N && m < p.M) {
                const size_t idx = (size_t)m * p.N + row;
                if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y)[idx] = __float2bfloat16_rn(sum);
                else reinterpret_cast<float*>(p.y)[idx] = sum;
            }
        }
    };

    auto compute = [&](const Stage<BITS, GPT>& st) {
        // pass the barriers of the tiles before this task's tile
        while (cur_tile < rt_c) tile_end(cur_tile++);
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
        uint32_t s2[2][GPT], b2[2][GPT];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int q = 0; q < GPT; q++) {
                s2[r][q] = st.s[r][q] | (st.s[r][q] << 16);
                b2[r][q] = st.b[r][q] | (st.b[r][q] << 16);
            }
        if (BITS == 4) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int q = (GPT == 2 && j >= 4) ? GPT - 1 : 0;
                uint32_t lo[4], hi[4];
                dequant4(st.w[0][j], s2[0][q], b2[0][q], lo);
                dequant4(st.w[1][j], s2[1][q], b2[1][q], hi);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 bx = xs[(((size_t)mt * nkb + kb_c) * XV + j) * 32 + (lane ^ j)];
                    mma_bf16(acc[mt], lo[0], hi[0], lo[1], hi[1], bx.x, bx.y);
                    mma_bf16(acc[mt], lo[2], hi[2], lo[3], hi[3], bx.z, bx.w);
                }
            }
        } else {
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                uint32_t lo0[2], hi0[2], lo1[2], hi1[2];
                dequant8(st.w[0][2 * jj], s2[0][0], b2[0][0], lo0);
                dequant8(st.w[1][2 * jj], s2[1][0], b2[1][0], hi0);
                dequant8(st.w[0][2 * jj + 1], s2[0][0], b2[0][0], lo1);
                dequant8(st.w[1][2 * jj + 1], s2[1][0], b2[1][0], hi1);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 bx = xs[(((size_t)mt * nkb + kb_c) * XV + jj) * 32 + (lane ^ (jj * 2))];
                    mma_bf16(acc[mt], lo0[0], hi0[0], lo0[1], hi0[1], bx.x, bx.y);
                    mma_bf16(acc[mt], lo1[0], hi1[0], lo1[1], hi1[1], bx.z, bx.w);
                }
            }
        }
        const int buf = (rt_c - rt_first) & 1;
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
            part[(((size_t)buf * nkb + kb_c) * MT + mt) * 32 + lane] = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
        tau_c += kWarps;
        kb_c += kWarps;
        while (kb_c >= nkb) {
            kb_c -= nkb;
            rt_c++;
        }
    };

#pragma unroll 1
    while (tau_c < t_end) {
        issue(st2);
        compute(st0);
        if (tau_c >= t_end) break;
        issue(st0);
        compute(st1);
        if (tau_c >= t_end) break;
        issue(st1);
        compute(st2);
    }
    while (cur_tile <= rt_last) tile_end(cur_tile++);
}

struct Plan {
    int nkb, n_rt, grid, mt, gpt;
    long long T;
    size_t smem, scratch_floats;
};

bool make_plan(const QmmArgs& a, int sm_count, Plan* pl) {
    if (a.x_dtype != LUX_DTYPE_BFLOAT16 || a.sb_dtype != LUX_DTYPE_BFLOAT16) return false;
    if (a.M < 1 || a.M > 16 || a.N < 1) return false;
    const int KT = 256 / a.bits, KB = 4 * KT;
    if (a.K % KB) return false;
    int gpt = 1;
    if (a.group < KT) {
        if (KT / a.group != 2) return false;
        gpt = 2;
    } else if (a.group % KT) {
        return false;
    }
    if (a.bits == 8 && gpt != 1) return false;
    const int XV = a.bits == 4 ? 8 : 4;
    pl->mt = a.M <= 8 ? 1 : 2;
    pl->gpt = gpt;
    pl->nkb = a.K / KB;
    pl->n_rt = (a.N + 15) / 16;
    pl->T = (long long)pl->n_rt * pl->nkb;
    pl->grid = (int)std::min<long long>(sm_count, pl->T);
    pl->smem = (size_t)pl->mt * pl->nkb * XV * 512 + (size_t)2 * pl->nkb * pl->mt * 512;
    pl->scratch_floats = (size_t)pl->grid * pl->nkb * pl->mt * 128;
    if (pl->smem > 227 * 1024 - 64) return false;  // 16 B of static shared memory besides
    if (((uintptr_t)a.wq & 31) || ((uintptr_t)a.x & 15)) return false;
    return true;
}

template <int BITS, int MT, int GPT>
cudaError_t launch_t(const Params& p, const Plan& pl, cudaStream_t stream) {
    auto kern = qmv_mma_kernel<BITS, MT, GPT>;
    // opt in to large dynamic shared memory (static + dynamic must stay within the 227 KiB per-block limit)
    static std::atomic<size_t> attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_smem[dev & 63].load() < pl.smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev & 63].store(pl.smem);
    }
    kern<<<pl.grid, kThreads, pl.smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

bool qmv_mma_supported(const QmmArgs& a) {
    Plan pl;
    return make_plan(a, 148, &pl);
}

size_t qmv_mma_workspace_bytes(const QmmArgs& a, int sm_count) {
    Plan pl;
    if (!make_plan(a, sm_count, &pl)) return 0;
    return pl.scratch_floats * sizeof(float) + (size_t)pl.grid * sizeof(unsigned int) + 256;
}

// workspace layout: [counters: grid x u32, padded to 256 B][scratch floats]; the
// counters must be zero before the first launch and are left zero by every launch.
cudaError_t launch_qmv_mma(const QmmArgs& a, void* workspace, int sm_count, cudaStream_t stream, const char** name) {
    Plan pl;
    if (!make_plan(a, sm_count, &pl)) return cudaErrorInvalidValue;
    Params p;
    p.x = (const __nv_bfloat16*)a.x;
    p.wq = a.wq;
    p.scales = (const __nv_bfloat16*)a.scales;
    p.biases = (const __nv_bfloat16*)a.biases;
    p.y = a.y;
    const size_t ctr_bytes = ((size_t)pl.grid * sizeof(unsigned int) + 255) & ~size_t(255);
    p.counters = (unsigned int*)workspace;
    p.scratch = (float*)((unsigned char*)workspace + ctr_bytes);
    p.M = a.M; p.K = a.K; p.N = a.N; p.group = a.group;
    p.y_bf16 = a.y_dtype == LUX_DTYPE_BFLOAT16;
    p.nkb = pl.nkb; p.n_rt = pl.n_rt; p.T = pl.T;
    if (a.bits == 4) {
        if (name) *name = pl.mt == 1 ? "qmv_mma<4,m8>" : "qmv_mma<4,m16>";
        if (pl.mt == 1) return pl.gpt == 1 ? launch_t<4, 1, 1>(p, pl, stream) : launch_t<4, 1, 2>(p, pl, stream);
        return pl.gpt == 1 ? launch_t<4, 2, 1>(p, pl, stream) : launch_t<4, 2, 2>(p, pl, stream);
    }
    if (name) *name = pl.mt == 1 ? "qmv_mma<8,m8>" : "qmv_mma<8,m16>";
    return pl.mt == 1 ? launch_t<8, 1, 1>(p, pl, stream) : launch_t<8, 2, 1>(p, pl, stream);
}

}  // namespace luxcuda
