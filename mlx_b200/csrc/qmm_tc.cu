// Prefill-regime quantized GEMM for bf16 activations (M > 16):
//   y[M,N] = x[M,K] . dequant(Wq[N,K])^T,  w^ = RNE_bf16(s*q + b)  (one bf16 FMA)
// on the 5th-generation tensor cores: tcgen05.mma with the fp32 accumulator in
// tensor memory, operands in shared memory.
//
// Tensor-bound: 2*M*N*K flop per launch; the packed weights (N*K*bits/8 bytes)
// are re-read M/BM times from L2, x (M*K*2 bytes) N/128 times.
//
// The MMA computes the TRANSPOSED tile  D[n, m] = sum_k W^[n, k] * x[m, k]:
//   A operand = 128 rows of W^ (dequantised bf16, K-major, 128-byte swizzle),
//               written into shared memory by the dequantising warps;
//   B operand = BM <= 256 rows of x (K-major, 128-byte swizzle), brought in by
//               TMA (cp.async.bulk.tensor, no multicast);
//   D         = 128 lanes x BM columns of fp32 in TMEM, two buffers so the
//               epilogue of one tile overlaps the main loop of the next.
// With W on the 128-lane side a weight is dequantised once per BM = 256 rows of
// x, which keeps the integer pipe (the scarce one) at about a quarter load.
//
// One persistent CTA per SM, 10 warps:
//   warps 0-3  epilogue: tcgen05.ld their 32 TMEM lanes, round to bf16/fp32,
//              store y[m][n] (32 consecutive n per warp and m);
//   warps 4-7  dequantisers: thread r owns row n0+r of the tile; per k-stage
//              (64 weights) it reads 32/64 packed bytes + scale/bias straight
//              from global memory (prefetched one stage ahead in registers),
//              dequantises (dequant.cuh) and stores 128 bytes of bf16 into the
//              swizzled A tile;
//   warp 8     TMA producer for x;
//   warp 9     allocates TMEM, issues tcgen05.mma (one elected thread) and the
//              commits that release smem stages / publish accumulators.
// Stage hand-over uses mbarriers; every wait is bounded: on a time-out the
// kernel raises an error word (host-visible) and all roles drain and return.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>

#include "dequant.cuh"
#include "internal.h"

namespace luxcuda {

namespace {

constexpr int kBK = 64;            // weights (k) per pipeline stage = one 128-byte swizzle row of bf16
constexpr int kStages = 4;
constexpr int kTileN = 128;        // rows of W per tile (MMA M)
constexpr int kMaxBM = 256;        // rows of x per tile (MMA N)
constexpr int kABytes = kTileN * 128;
constexpr int kDqWarps = 8;         // dequantising warps: kDqWarps/4 threads per row of the tile
constexpr int kDqThreads = kDqWarps * 32;
constexpr int kTpr = kDqWarps / 4; // threads per row
constexpr int kCpt = 8 / kTpr;     // 16-byte output chunks (8 weights) per thread per stage
constexpr int kNumThreads = 128 + kDqThreads + 64;
constexpr int kTmaWarp = 4 + kDqWarps, kMmaWarp = 5 + kDqWarps;
constexpr uint32_t kSpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_ca(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort_flag) when the barrier does not
// flip within the limit or another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        if (mbar_try(b, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// ---- tcgen05 / TMEM ------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                          // leading-dimension byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride-dimension byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                          // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                          // layout: SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: D = F32, A = B = BF16, both K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- TMA -----------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(s32(dst)), "l"(map), "r"(x), "r"(y), "r"(s32(bar)) : "memory");
}

struct GemmParams {
    const uint32_t* wq;
    const __nv_bfloat16* scales;
    const __nv_bfloat16* biases;
    void* y;
    int* error;              // host-visible error word (0 = ok)
    int M, K, N, gshift, y_bf16;
    int bm;                  // rows of x per tile (multiple of 16, <= 256)
    int n_tiles, m_tiles;
    uint32_t tmem_cols;      // allocated TMEM columns (power of two >= 32), 2 accumulators of tmem_cols/2
};

#ifdef QMM_TRACE
__device__ unsigned long long g_qtrace[32];
__device__ __forceinline__ unsigned long long qgt() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define QT_MARK(i) do { if (blockIdx.x == 0) g_qtrace[i] = qgt(); } while (0)
#define QT_BEGIN long long _qt0 = (long long)qgt()
#define QT_ADD(i) do { if (blockIdx.x == 0) { long long _t = (long long)qgt(); atomicAdd(&g_qtrace[i], (unsigned long long)(_t - _qt0)); _qt0 = _t; } } while (0)
#else
#define QT_BEGIN do {} while (0)
#define QT_MARK(i) do {} while (0)
#define QT_ADD(i) do {} while (0)
#endif

struct SmemLayout {
    uint64_t full_a[kStages], full_b[kStages], empty[kStages], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// eight dequantised weights (natural k order) from one 4-bit word / two 8-bit words
template <int BITS, bool fast>
__device__ __forceinline__ uint4 dequant_chunk(const uint32_t* w, uint32_t s_bits, uint32_t b_bits) {
    uint4 o;
    const uint32_t b2 = dup_bf16(b_bits);
    if (BITS == 4) {
        uint32_t r[4];  // r[i] = (w^_i, w^_{i+4})
        if (fast) dequant4_fast(w[0], scale_x2_133(s_bits), scale_x2_129(s_bits), b2, r);
        else dequant4_general(w[0], dup_bf16(s_bits), b2, r);
        o.x = prmt(r[0], r[1], 0x5410u);
        o.y = prmt(r[2], r[3], 0x5410u);
        o.z = prmt(r[0], r[1], 0x7632u);
        o.w = prmt(r[2], r[3], 0x7632u);
    } else {
        uint32_t r0[2], r1[2];  // (w^_0, w^_2), (w^_1, w^_3) of each word
        if (fast) {
            const uint32_t s133 = scale_x2_133(s_bits);
            dequant8_fast(w[0], s133, b2, r0);
            dequant8_fast(w[1], s133, b2, r1);
        } else {
            dequant8_general(w[0], dup_bf16(s_bits), b2, r0);
            dequant8_general(w[1], dup_bf16(s_bits), b2, r1);
        }
        o.x = prmt(r0[0], r0[1], 0x5410u);
        o.y = prmt(r0[0], r0[1], 0x7632u);
        o.z = prmt(r1[0], r1[1], 0x5410u);
        o.w = prmt(r1[0], r1[1], 0x7632u);
    }
    return o;
}

// One thread's share of a k-stage: kCpt chunks of 8 weights -> swizzled 16-byte stores into its A row.
template <int BITS, bool FAST>
__device__ __forceinline__ void dequant_store(const uint32_t* w, const uint32_t* sc, const uint32_t* bi, unsigned char* dst,
                                              int part, int r7) {
    constexpr int WPC = kBK * BITS / 32 / 8;   // packed words per chunk
    constexpr int KPT = kBK / kTpr;
#pragma unroll
    for (int c = 0; c < kCpt; c++) {
        const int q = (KPT > 32 && c >= 4) ? 1 : 0;
        const uint4 v = dequant_chunk<BITS, FAST>(&w[c * WPC], sc[q], bi[q]);
        *reinterpret_cast<uint4*>(dst + (((part * kCpt + c) ^ r7) << 4)) = v;
    }
}
// the general (any scale) variant is kept out of line so the common path stays branch-free and small
template <int BITS>
__device__ __noinline__ void dequant_store_general(const uint32_t* w, const uint32_t* sc, const uint32_t* bi,
                                                   unsigned char* dst, int part, int r7) {
    dequant_store<BITS, false>(w, sc, bi, dst, part, r7);
}

template <int BITS>
__global__ void __launch_bounds__(kNumThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ GemmParams p) {
    constexpr int WPS = kBK * BITS / 32;  // packed words per row per stage: 8 | 16
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;                                  // [kStages][128 rows][128 B], swizzled
    unsigned char* sB = smem + kStages * kABytes;              // [kStages][bm rows][128 B], swizzled (TMA)
    const uint32_t b_bytes = (uint32_t)p.bm * 128;
    SmemLayout* sl = reinterpret_cast<SmemLayout*>(sB + kStages * (size_t)kMaxBM * 128);
    unsigned char* sSB = reinterpret_cast<unsigned char*>(sl) + 256;   // [kDqThreads][2 buffers][scales 16 B | biases 16 B]
    volatile int* abort_flag = &sl->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) QT_MARK(16);
    const int nks = p.K / kBK;
    const int total_tiles = p.n_tiles * p.m_tiles;
    const uint32_t acc_cols = p.tmem_cols / 2;

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&sl->full_a[s], kDqThreads);
            mbar_init(&sl->full_b[s], 1);
            mbar_init(&sl->empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&sl->tmem_full[a], 1);
            mbar_init(&sl->tmem_empty[a], 128);
        }
        sl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(&sl->tmem_base, p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sl->tmem_base;
    if (tid == 0) QT_MARK(17);

    if (warp == kTmaWarp) {
        // ---------------- TMA producer: x tiles ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * p.bm;
                for (int ks = 0; ks < nks; ks++, it++) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    QT_BEGIN;
                    if (!mbar_wait(&sl->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
                    QT_ADD(0);
                    mbar_expect_tx(&sl->full_b[s], b_bytes);
                    tma_load_2d(sB + (size_t)s * kMaxBM * 128, &tmap_x, ks * kBK, m0, &sl->full_b[s]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(kTileN, p.bm);
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, tile_i++) {
                const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
                { QT_BEGIN; if (!mbar_wait(&sl->tmem_empty[acc], acc_ph ^ 1, abort_flag)) break; QT_ADD(4); }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_cols;
                for (int ks = 0; ks < nks; ks++, it++) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    QT_BEGIN;
                    if (!mbar_wait(&sl->full_a[s], ph, abort_flag)) { ok = false; break; }
                    QT_ADD(1);
                    if (!mbar_wait(&sl->full_b[s], ph, abort_flag)) { ok = false; break; }
                    QT_ADD(2);
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(s32(sA + (size_t)s * kABytes));
                    const uint64_t db = umma_desc_sw128(s32(sB + (size_t)s * kMaxBM * 128));
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; kk++)  // 32 bytes (2 x 16 B units) further along K per step
                        tc_mma(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (ks | kk) != 0 ? 1u : 0u);
                    tc_commit(&sl->empty[s]);  // arrives when the MMAs above have finished reading the stage
                    QT_ADD(3);
                }
                if (ok) tc_commit(&sl->tmem_full[acc]);
                QT_MARK(18 + (tile_i & 1));
            }
        }
    } else if (warp >= 4) {
        // ---------------- dequantisers: kTpr threads per row n0 + r, kCpt chunks of 8 weights each ----------------
        const int d = tid - 128;
        const int r = d / kTpr, part = d % kTpr;        // part: which kCpt chunks of the 64-weight stage (adjacent lanes share a row)
        constexpr int WPT = WPS / kTpr;                 // packed words per thread per stage
        constexpr int KPT = kBK / kTpr;                 // weights per thread per stage
        const size_t row_bytes = (size_t)p.K * BITS / 8;
        const int gpr = p.K >> p.gshift;
        const uint32_t row_off = (uint32_t)(r >> 3) * 1024 + (uint32_t)(r & 7) * 128;
        // scales/biases: one strided 2-byte load per row and stage would swamp the L1 tag pipe (every
        // thread is on its own row), so when rows of the scale matrix are 16-byte multiples they are
        // fetched eight groups at a time into a per-thread shared-memory slot
        const bool vec_sb = (gpr & 7) == 0;
        const int sps = (8 << p.gshift) / kBK;          // k-stages covered by eight groups: 4, 8 or 16
        const uint32_t sb_slot = s32(sSB) + d * 64;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int n = min((tile / p.m_tiles) * kTileN + r, p.N - 1);
            const uint32_t* wrow = reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(p.wq) + (size_t)n * row_bytes) + part * WPT;
            const uint16_t* srow = reinterpret_cast<const uint16_t*>(p.scales) + (size_t)n * gpr;
            const uint16_t* brow = reinterpret_cast<const uint16_t*>(p.biases) + (size_t)n * gpr;
            // kPre stages of packed words + scale/bias are kept in flight in registers (the loads are
            // L2 hits, but their latency under load is several k-stages long)
            constexpr int kPre = 4;
            constexpr int NS = KPT > 32 ? 2 : 1;
            uint32_t wr[kPre][WPT], sr[kPre][NS], br[kPre][NS];
            auto fetch = [&](int ks, uint32_t (&w)[WPT], uint32_t (&sc)[NS], uint32_t (&bi)[NS]) {
                if (ks >= nks) return;
#ifdef QMM_NOLOAD_W
                for (int i = 0; i < WPT; i++) w[i] = 0x12345678u * (ks + i);
                if (false)
#endif
                if (WPT >= 4) {
                    // straight into the registers that hold the stage (no copy that would wait for the load)
#pragma unroll
                    for (int i = 0; i < WPT / 4; i++)
                        asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3])
                                     : "l"(wrow + ks * WPS + 4 * i));
                } else {
                    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[WPT - 1]) : "l"(wrow + ks * WPS));
                }
                const int k0 = ks * kBK + part * KPT;
#ifdef QMM_NOLOAD_SB
                sc[0] = 0x3C00; bi[0] = 0xBC00; sc[NS - 1] = 0x3C00; bi[NS - 1] = 0xBC00;
                return;
#endif
                if (vec_sb) {
                    // eight groups of scales and biases at a time, 16-byte cp.async into this thread's slot
                    if ((ks & (sps - 1)) == 0) {
                        const int j = ks / sps;
                        cp_async16_ca(sb_slot + (j & 1) * 32, srow + 8 * j);
                        cp_async16_ca(sb_slot + (j & 1) * 32 + 16, brow + 8 * j);
                    }
                    return;
                }
#pragma unroll
                for (int q = 0; q < NS; q++) {
                    const int gi = (k0 + q * 32) >> p.gshift;
                    sc[q] = __ldg(srow + gi);
                    bi[q] = __ldg(brow + gi);
                }
            };
            int ks_cur = 0;
            auto stage = [&](const uint32_t (&w)[WPT], const uint32_t (&sc)[NS], const uint32_t (&bi)[NS]) -> bool {
                const int s = it % kStages;
                const uint32_t ph = (it / kStages) & 1;
                QT_BEGIN;
                if (!mbar_wait(&sl->empty[s], ph ^ 1, abort_flag)) return false;
                if (d == 0) QT_ADD(8);
                unsigned char* dst = sA + (size_t)s * kABytes + row_off;
                uint32_t scv[NS], biv[NS];
#pragma unroll
                for (int q = 0; q < NS; q++) { scv[q] = sc[q]; biv[q] = bi[q]; }
#ifdef QMM_NOLOAD_SB
                if (false) {
#else
                if (vec_sb) {
#endif
                    const int ks = ks_cur;
                    if ((ks & (sps - 1)) == 0) {  // first stage of a block of eight groups: its copy must have landed
                        asm volatile("cp.async.wait_all;" ::: "memory");
                    }
                    const uint32_t base = sb_slot + ((ks / sps) & 1) * 32;
#pragma unroll
                    for (int q = 0; q < NS; q++) {
                        const uint32_t off = ((((ks & (sps - 1)) * kBK + part * KPT + q * 32) >> p.gshift) << 1);
                        uint16_t sv, bv;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sv) : "r"(base + off));
                        asm volatile("ld.shared.u16 %0, [%1+16];" : "=h"(bv) : "r"(base + off));
                        scv[q] = sv; biv[q] = bv;
                    }
                }
                bool fast = true;
#pragma unroll
                for (int q = 0; q < NS; q++) fast = fast && scale_fast_ok(scv[q]);
                if (fast) dequant_store<BITS, true>(w, scv, biv, dst, part, r & 7);
                else dequant_store_general<BITS>(w, scv, biv, dst, part, r & 7);
                if (d == 0) QT_ADD(9);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA
                mbar_arrive(&sl->full_a[s]);
                if (d == 0) QT_ADD(10);
                it++;
                return true;
            };
#pragma unroll
            for (int i = 0; i < kPre; i++) fetch(i, wr[i], sr[i], br[i]);
            for (int ks = 0; ks < nks && ok; ks += kPre) {
#pragma unroll
                for (int i = 0; i < kPre; i++) {
                    if (ks + i < nks) {
                        ks_cur = ks + i;
                        if (!stage(wr[i], sr[i], br[i])) { ok = false; break; }
                        { QT_BEGIN; fetch(ks + i + kPre, wr[i], sr[i], br[i]); if (d == 0) QT_ADD(11); }
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue: warp w reads TMEM lanes 32w .. 32w+31 ----------------
        uint32_t tile_i = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tile_i++) {
            const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
            const int n = (tile / p.m_tiles) * kTileN + warp * 32 + lane;
            const int m0 = (tile % p.m_tiles) * p.bm;
            QT_BEGIN;
            if (!mbar_wait(&sl->tmem_full[acc], acc_ph, abort_flag)) break;
            if (tid == 0) QT_ADD(12);
            tc_fence_after();
            // this thread: column n of y, rows m0 .. m0+bm-1 (32 consecutive n per warp: 64-byte row segments)
            const int m_end = min(p.bm, p.M - m0);
            for (int c0 = 0; c0 < p.bm; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + acc * acc_cols + c0, v);
                if (n < p.N) {
                    const size_t idx0 = (size_t)(m0 + c0) * p.N + n;
                    if (p.y_bf16) {
                        __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(p.y) + idx0;
                        if (c0 + 32 <= m_end) {
#pragma unroll
                            for (int j = 0; j < 32; j++) yp[(size_t)j * p.N] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (c0 + j < m_end) yp[(size_t)j * p.N] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        }
                    } else {
                        float* yp = reinterpret_cast<float*>(p.y) + idx0;
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (c0 + j < m_end) yp[(size_t)j * p.N] = __uint_as_float(v[j]);
                    }
                }
            }
            if (tid == 0) QT_ADD(13);
            tc_fence_before();
            mbar_arrive(&sl->tmem_empty[acc]);
        }
    }
    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (tid == 0) QT_MARK(20);
    if (tid == 0 && sl->abort_flag) *p.error = 1;
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
}

// ---- host side -------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int* g_error_host = nullptr;  // pinned + mapped: written by kernels that give up on a wait, read by the host
std::once_flag g_error_once;

int* error_word() {
    std::call_once(g_error_once, [] {
        void* p = nullptr;
        if (cudaHostAlloc(&p, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
            g_error_host = static_cast<int*>(p);
            *g_error_host = 0;
        } else {
            cudaGetLastError();
        }
    });
    return g_error_host;
}

struct GemmPlan {
    int bm, m_tiles, n_tiles;
    uint32_t tmem_cols;
    size_t smem;
};

bool make_gemm_plan(const QmmArgs& a, GemmPlan* pl) {
    if (a.x_dtype != LUX_DTYPE_BFLOAT16 || a.sb_dtype != LUX_DTYPE_BFLOAT16) return false;
    if (a.bits != 4 && a.bits != 8) return false;
    if (a.group != 32 && a.group != 64 && a.group != 128) return false;
    if (a.M <= 16 || a.N < 1 || a.K % kBK) return false;
    if (((uintptr_t)a.x | (uintptr_t)a.wq | (uintptr_t)a.scales | (uintptr_t)a.biases | (uintptr_t)a.y) & 15) return false;
    if ((long long)a.N * (a.K / a.group) > (1ll << 31) - 1) return false;
    pl->m_tiles = (a.M + kMaxBM - 1) / kMaxBM;
    pl->bm = (((a.M + pl->m_tiles - 1) / pl->m_tiles) + 15) & ~15;
    pl->n_tiles = (a.N + kTileN - 1) / kTileN;
    uint32_t acc = 32;
    while ((int)acc < pl->bm) acc *= 2;
    pl->tmem_cols = 2 * acc;
    pl->smem = 1024 + (size_t)kStages * (kABytes + kMaxBM * 128) + 256 + (size_t)kDqThreads * 64;
    static_assert(sizeof(SmemLayout) <= 256, "barrier block");
    return encode_tiled_fn() != nullptr;
}

template <int BITS>
cudaError_t launch_gemm_t(const CUtensorMap& tmap, const GemmParams& p, const GemmPlan& pl, int sm_count, cudaStream_t stream) {
    auto kern = qmm_tc_kernel<BITS>;
    static std::atomic<size_t> attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_smem[dev & 63].load() < pl.smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev & 63].store(pl.smem);
    }
    const int grid = std::min(sm_count, pl.m_tiles * pl.n_tiles);
    kern<<<grid, kNumThreads, pl.smem, stream>>>(tmap, p);
    return cudaGetLastError();
}

}  // namespace

bool qmm_tc_supported(const QmmArgs& a) {
    GemmPlan pl;
    return make_gemm_plan(a, &pl);
}

cudaError_t launch_qmm_tc(const QmmArgs& a, int sm_count, cudaStream_t stream, const char** name) {
    GemmPlan pl;
    if (!make_gemm_plan(a, &pl)) return cudaErrorInvalidValue;
    int* err = error_word();
    if (!err) return cudaErrorMemoryAllocation;
    // x as a 2-D tensor [M rows][K], boxes of 64 elements (128 bytes) x bm rows, 128-byte swizzle;
    // rows past M are filled with zeros by the copy engine
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)pl.bm};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled_fn()(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.x), dims, strides, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed (%d)", (int)r);
        return cudaErrorInvalidValue;
    }
    GemmParams p;
    p.wq = a.wq;
    p.scales = (const __nv_bfloat16*)a.scales;
    p.biases = (const __nv_bfloat16*)a.biases;
    p.y = a.y;
    int* derr = nullptr;
    if (cudaHostGetDevicePointer((void**)&derr, err, 0) != cudaSuccess) return cudaGetLastError();
    p.error = derr;
    p.M = a.M; p.K = a.K; p.N = a.N;
    p.gshift = a.group == 32 ? 5 : (a.group == 64 ? 6 : 7);
    p.y_bf16 = a.y_dtype == LUX_DTYPE_BFLOAT16;
    p.bm = pl.bm; p.n_tiles = pl.n_tiles; p.m_tiles = pl.m_tiles; p.tmem_cols = pl.tmem_cols;
    if (a.bits == 4) {
        if (name) *name = "qmm_tc<4>";
        return launch_gemm_t<4>(tmap, p, pl, sm_count, stream);
    }
    if (name) *name = "qmm_tc<8>";
    return launch_gemm_t<8>(tmap, p, pl, sm_count, stream);
}

// Non-zero once a kernel has given up on a bounded wait; reading clears it.
int take_device_error() {
    if (!g_error_host || !*g_error_host) return 0;
    const int v = *g_error_host;
    *g_error_host = 0;
    return v;
}

}  // namespace luxcuda
