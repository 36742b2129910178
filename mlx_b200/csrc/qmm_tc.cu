// Prefill-regime quantized GEMM for bf16 activations (M > 16):
//   y[M,N] = x[M,K] . dequant(Wq[N,K])^T,  w^ = RNE_bf16(s*q + b)  (one bf16 FMA)
// on the 5th-generation tensor cores: tcgen05.mma with the fp32 accumulator in
// tensor memory, operands in shared memory.
//
// Tensor-bound: 2*M*N*K flop per launch; the packed weights (N*K*bits/8 bytes)
// are re-read M/BM times from L2, x (M*K*2 bytes) N/128 times.
//
// The MMA computes the TRANSPOSED tile  D[n, m] = sum_k W^[n, k] * x[m, k]:
//   A operand = 128 rows of W^ (dequantised bf16), written by the dequantising
//               warps straight into TENSOR MEMORY (tcgen05.st): it never
//               touches shared memory, whose bandwidth the B operand needs;
//   B operand = BM <= 256 rows of x (K-major, 128-byte swizzle) in shared
//               memory, brought in by TMA (cp.async.bulk.tensor, no multicast);
//   D         = 128 lanes x BM columns of fp32 in TMEM.
// With W on the 128-lane side a weight is dequantised once per BM = 256 rows of
// x, which keeps the integer pipe (the scarce one) at about a quarter load.
// TMEM (512 columns): D in columns [0, 256), a ring of A k-stages
// (64 weights = 32 columns each) from column 256 on, one slot per k-stage in
// flight.  Shared memory: the matching ring of B stages (32 KiB each).
//
// One persistent CTA per SM, 22 warps:
//   warps 0-7   epilogue: warp w reads TMEM lanes 32*(w%4).., half w/4 of the
//               columns, rounds to bf16/fp32, stores y[m][n];
//   warps 8-19  dequantisers in three groups of four warps: group j owns the
//               pipeline stages = j (mod 3); inside a group warp q owns TMEM lanes
//               32q.. (a warp may only touch its own lane quarter), so thread
//               (q, lane) owns row n0 + 32q + lane.  The group's leader thread
//               brings the group's next 128 rows x 64 packed bytes into the
//               group's own shared-memory slot by TMA (64-byte swizzle, so the
//               row-per-thread reads are bank-conflict free); a thread reads its
//               64 bytes, the group meets at a named barrier, the leader refills
//               the slot for the group's next stage.  (Row-per-thread loads from
//               global memory were one L1 wavefront per lane and kept the load
//               pipe 70-80 % busy; through the slot it is 4 wavefronts per warp.)
//               Scales / biases of a stage are one small vector load per thread,
//               fetched one owned stage ahead.  Then dequantise (dequant.cuh)
//               and write 32 TMEM columns per 64 weights;
//   warp 20     TMA producer for x;
//   warp 21     allocates TMEM, issues tcgen05.mma (one elected thread) and the
//               commits that release A slots / B stages and publish D.
// Hand-over uses mbarriers; every wait is bounded: on a time-out the kernel
// raises an error word (host-visible) and all roles drain and return.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <atomic>

#include "dequant.cuh"
#include "internal.h"

namespace luxcuda {

namespace {

constexpr int kBK = 64;            // weights (k) per pipeline stage = one 128-byte swizzle row of bf16
constexpr int kStagesB = 3;  // k-stages in flight: B in shared memory, A in TMEM, one barrier pair per stage
constexpr int kTileN = 128;        // rows of W per tile (MMA M)
constexpr int kMaxBM = 256;        // rows of x per tile (MMA N)
constexpr int kSub = 2;            // 64-weight sub-blocks per pipeline stage (one barrier round per 128 k)
constexpr int kBBytes = kMaxBM * 128;   // one sub-block of B
constexpr int kEpiStageBytes = 16 * 32 * 2;  // per epilogue warp: 16 rows of y x 32 columns, bf16
constexpr int kWUnitBytes = kTileN * 64;  // one unit of packed weights: 128 rows x 64 bytes (128 k at 4 bit, 64 k at 8 bit)
constexpr int kEpiWarps = 8, kDqGroups = 3, kDqWarps = 4 * kDqGroups;
// A dequantising group goes from stage s straight to stage s + kDqGroups.  Its wait for that slot is by
// phase parity, which cannot tell "freed once more" from "two frees behind": the group must never be able
// to get two ring rounds ahead of the MMA, i.e. kDqGroups <= kStagesB.
static_assert(kDqGroups <= kStagesB, "parity waits would alias");
constexpr int kTmaWarp = kEpiWarps + kDqWarps, kMmaWarp = kTmaWarp + 1;
constexpr int kNumThreads = (kMmaWarp + 1) * 32;
constexpr uint32_t kTmemCols = 512, kAColBase = 256, kAColsPerSub = kBK / 2, kAColsPerSlot = kSub * kAColsPerSub;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr size_t kWsFlagBytes = 1024;  // flag words of the stream-K workspace (one per CTA), ahead of the partials

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
        if (i > 4) __nanosleep(40);  // waiting roles must not steal issue slots from the working ones
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// One look at a barrier, never suspended: the answer comes back some hundred cycles later, which the caller
// can spend on other instructions.
__device__ __forceinline__ bool mbar_test_addr(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Same bound, no back-off: for the one thread whose wake-up latency is on the tensor pipe's critical path.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit * 8; i++) {
        if (mbar_try(b, parity)) return true;
        if ((i & 4095u) == 4095u && *abort_flag) return false;
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
// D[tmem] (+)= A[tmem] * B[smem desc], bf16 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the B descriptor as two words:
// only the low one, which holds the address, changes between calls.
__device__ __forceinline__ void tc_mma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc) {
    asm volatile(
        "{ .reg .pred p; .reg .b64 bd; setp.eq.u32 p, 1, 1; mov.b64 bd, {%2, %3};\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc) : "memory");
}
__device__ __forceinline__ void tc_mma_ts_first(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; .reg .b64 bd; setp.ne.b32 p, %5, 0; mov.b64 bd, {%2, %3};\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane <- 32 registers
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
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
    int world, ld, col0;     // copies of y to write (1 unless column-sharded), their row stride and this rank's first column
    void* y_all[kMaxShardWorld];
    int bm;                  // rows of x per tile (multiple of 16, <= 256)
    int n_tiles, m_tiles;
    float* ws;               // partial accumulators of tiles shared between CTAs: [CTA][bm][128] fp32
    int y_tma;               // pair kernel: y leaves through shared memory; 1: by a TMA store (bf16, one copy of y, N % 8 == 0),
                             // 2: by 16-byte stores into every rank's copy (column-sharded, ld and col0 multiples of 8)
    uint32_t* ws_flags;      // [CTA]: 1 while that CTA's partial waits to be added (zero between launches)
};

// The work of a launch is the sequence of (tile, k-stage) units, tile after tile.  Two schedules:
//   * whole tiles, round robin: CTA c takes tiles c, c + G, c + 2G, ... (neighbouring CTAs work on neighbouring
//     tiles at the same k, which L2 likes); the launch lasts ceil(T/G) tiles;
//   * "stream-K": CTA c takes the units [U*c/G, U*(c+1)/G), so every SM gets the same number of k-stages
//     whatever the number of tiles, at the price of one more epilogue per CTA and of the exchange of partial
//     accumulators described next.  The host picks the cheaper one by a small cost model (make_gemm_plan).
// A CTA's range is a sequence of segments, each a run of stages [s_lo, s_hi) of one tile.  Only its first
// segment can start inside a tile (s_lo > 0): that partial accumulator goes to the CTA's slot of the
// workspace; the CTA that owns the tile's first stages (s_lo == 0) adds the partials of the CTAs after it
// (c+1 .. the owner of the tile's last stage) in its epilogue and writes y.  Those partials are produced
// either at the start of the neighbour's range or, when a range is shorter than a tile, at the same time
// as the head: the head's wait for them is short, and bounded.
template <bool SK>
struct SegIter;
template <>
struct SegIter<true> {  // stream-K: the CTA's range of units, segment by segment
    long long u, u_hi;
    int nst;
    __device__ __forceinline__ void init(long long total_units, int nst_) {
        nst = nst_;
        u = total_units * blockIdx.x / gridDim.x;
        u_hi = total_units * (blockIdx.x + 1) / gridDim.x;
    }
    __device__ __forceinline__ bool valid() const { return u < u_hi; }
    __device__ __forceinline__ int tile() const { return (int)(u / nst); }
    __device__ __forceinline__ int s_lo() const { return (int)(u % nst); }
    __device__ __forceinline__ int s_hi() const { return (int)min((long long)nst, (long long)s_lo() + (u_hi - u)); }
    __device__ __forceinline__ void next() { u += (long long)(s_hi() - s_lo()); }
};
// the CTA whose range holds unit u
__device__ __forceinline__ int cta_of_unit(long long u, long long total_units) {
    return (int)(((u + 1) * gridDim.x - 1) / total_units);
}

struct SmemLayout {
    uint64_t full[kStagesB], empty[kStagesB], wfull[kDqGroups], tmem_full, tmem_empty;
    uint32_t tmem_base;
    int abort_flag;
};

// Barrier `id` over 128 threads that also ANDs a predicate: every participant gets the same answer.
__device__ __forceinline__ bool group_all(int id, bool pred) {
    uint32_t r;
    asm volatile(
        "{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, %2, 128, q; selp.u32 %0, 1, 0, p; }"
        : "=r"(r) : "r"((uint32_t)pred), "r"(id) : "memory");
    return r != 0;
}

__device__ __forceinline__ uint32_t ldg_u16(const uint16_t* p) {  // zero-extended straight into a 32-bit register
    uint32_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// 64 weights of one row (one k-stage) -> 32 registers of bf16 pairs in natural k order
template <int BITS, bool FAST>
__device__ __forceinline__ void dequant_row_stage(const uint32_t* w, uint32_t s0, uint32_t b0, uint32_t s1, uint32_t b1,
                                                  uint32_t (&out)[32]) {
    constexpr int WPC = kBK * BITS / 32 / 8;  // packed words per chunk of 8 weights
#pragma unroll
    for (int c = 0; c < 8; c++) {
        const uint32_t s_bits = c < 4 ? s0 : s1, b_bits = c < 4 ? b0 : b1;
        const uint32_t b2 = dup_bf16(b_bits);
        if (BITS == 4) {
            uint32_t r[4];  // r[i] = (w^_i, w^_{i+4})
            if (FAST) dequant4_fast(w[c], scale_x2_133(s_bits), scale_x2_129(s_bits), b2, r);
            else dequant4_general(w[c], dup_bf16(s_bits), b2, r);
            out[4 * c + 0] = prmt(r[0], r[1], 0x5410u);
            out[4 * c + 1] = prmt(r[2], r[3], 0x5410u);
            out[4 * c + 2] = prmt(r[0], r[1], 0x7632u);
            out[4 * c + 3] = prmt(r[2], r[3], 0x7632u);
        } else {
            uint32_t r0[2], r1[2];  // (w^_0, w^_2), (w^_1, w^_3) of each word
            if (FAST) {
                const uint32_t s133 = scale_x2_133(s_bits);
                dequant8_fast(w[c * WPC], s133, b2, r0);
                dequant8_fast(w[c * WPC + WPC - 1], s133, b2, r1);
            } else {
                dequant8_general(w[c * WPC], dup_bf16(s_bits), b2, r0);
                dequant8_general(w[c * WPC + WPC - 1], dup_bf16(s_bits), b2, r1);
            }
            out[4 * c + 0] = prmt(r0[0], r0[1], 0x5410u);
            out[4 * c + 1] = prmt(r0[0], r0[1], 0x7632u);
            out[4 * c + 2] = prmt(r1[0], r1[1], 0x5410u);
            out[4 * c + 3] = prmt(r1[0], r1[1], 0x7632u);
        }
    }
}
template <int BITS, bool SK>
__global__ void __launch_bounds__(kNumThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
              const __grid_constant__ GemmParams p) {
    constexpr int WPS = kBK * BITS / 32;  // packed words per row per stage: 8 | 16
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sB = smem;  // [kStagesB][bm rows][128 B], swizzled (TMA)
    const uint32_t b_bytes = (uint32_t)p.bm * 128;
    unsigned char* sW = sB + (size_t)kStagesB * kSub * kBBytes;  // [kDqGroups][128 rows][64 B], 64-byte swizzle (TMA)
    unsigned char* sEpi = sW + (size_t)kDqGroups * kWUnitBytes;  // [kEpiWarps][16 rows of x][32 rows of the tile] bf16: the epilogue's transposer
    SmemLayout* sl = reinterpret_cast<SmemLayout*>(sEpi + (size_t)kEpiWarps * kEpiStageBytes);
    volatile int* abort_flag = &sl->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nks = p.K / kBK;                  // 64-weight sub-blocks along K
    const int nst = (nks + kSub - 1) / kSub;    // pipeline stages per tile
    const int total_tiles = p.n_tiles * p.m_tiles;
    const long long total_units = (long long)total_tiles * nst;

    if (tid == 0) {
        for (int s = 0; s < kStagesB; s++) {
            mbar_init(&sl->full[s], 128 + 1);  // 128 dequantising threads + the TMA producer (with its byte count)
            mbar_init(&sl->empty[s], 1);        // one tcgen05.commit
        }
        for (int g = 0; g < kDqGroups; g++) mbar_init(&sl->wfull[g], 1);  // the group leader's expect_tx
        mbar_init(&sl->tmem_full, 1);
        mbar_init(&sl->tmem_empty, kEpiWarps * 32);
        sl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(&sl->tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sl->tmem_base;

    if (warp == kTmaWarp) {
        // ---------------- TMA producer: x tiles ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            uint32_t it = 0;
            bool ok = true;
            SegIter<SK> seg;
            for (seg.init(total_units, nst); seg.valid() && ok; seg.next()) {
                const int tile = seg.tile(), s_hi = seg.s_hi();
                const int m0 = (tile % p.m_tiles) * p.bm;
                for (int st = seg.s_lo(); st < s_hi; st++, it++) {
                    const int sb = it % kStagesB;
                    const uint32_t ph = (it / kStagesB) & 1;
                    const int nsub = min(kSub, nks - st * kSub);
                    if (!mbar_wait(&sl->empty[sb], ph ^ 1, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(&sl->full[sb], b_bytes * nsub);
                    for (int u = 0; u < nsub; u++)
                        tma_load_2d(sB + ((size_t)sb * kSub + u) * kBBytes, &tmap_x, (st * kSub + u) * kBK, m0, &sl->full[sb]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(kTileN, p.bm);
            uint32_t tile_i = 0, slot = 0, phase = 0;
            const uint64_t db0 = umma_desc_sw128(s32(sB));
            const uint32_t b_hi = (uint32_t)(db0 >> 32), b_lo0 = (uint32_t)db0;  // the address is in the low word, 16-byte units
            const uint32_t a0 = tmem_base + kAColBase, bar0 = s32(&sl->full[0]);
            bool ok = true;
            // This thread's instructions are the pipeline's critical path (it shares its scheduler with working
            // warps, and a look at a barrier costs it some hundred cycles even when the phase is long over): the
            // barrier of the NEXT stage is looked at before the MMAs of the current one are issued, the answer read
            // after; an MMA is an add or two and the instruction.
            bool ready = false;
            SegIter<SK> seg;
            for (seg.init(total_units, nst); seg.valid() && ok; seg.next(), tile_i++) {
                const int s_lo = seg.s_lo(), s_hi = seg.s_hi();
                if (!mbar_wait(&sl->tmem_empty, (tile_i & 1) ^ 1, abort_flag)) break;
                tc_fence_after();
                for (int st = s_lo; st < s_hi; st++) {
                    if (!ready && !mbar_wait_spin(&sl->full[slot], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t nslot = slot + 1, nphase = phase;
                    if (nslot == (uint32_t)kStagesB) { nslot = 0; nphase ^= 1; }
                    const bool rn = mbar_test_addr(bar0 + 8 * nslot, nphase);  // (past the CTA's last stage: "not yet", and not used)
                    const uint32_t b_lo = b_lo0 + slot * (uint32_t)(kSub * kBBytes >> 4);
                    const uint32_t a_tmem = a0 + slot * kAColsPerSlot;
                    // 16 k per MMA = 8 TMEM columns of A, 32 bytes of each B row
                    tc_mma_ts_first(tmem_base, a_tmem, b_lo, b_hi, idesc, st != s_lo ? 1u : 0u);
#pragma unroll
                    for (int kk = 1; kk < kBK / 16; kk++) tc_mma_ts_acc(tmem_base, a_tmem + 8 * kk, b_lo + 2 * kk, b_hi, idesc);
                    if (st * kSub + 1 < nks) {  // (the last stage of an odd K has one sub-block)
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; kk++)
                            tc_mma_ts_acc(tmem_base, a_tmem + kAColsPerSub + 8 * kk, b_lo + (kBBytes >> 4) + 2 * kk, b_hi, idesc);
                    }
                    tc_commit(&sl->empty[slot]);  // arrives when the MMAs above have consumed their operands
                    ready = rn;
                    slot = nslot; phase = nphase;
                }
                if (ok) tc_commit(&sl->tmem_full);
            }
        }
    } else if (warp >= kEpiWarps) {
        // ---------------- dequantisers: group grp owns the stages = grp (mod kDqGroups); thread owns row n0 + r ----------------
        constexpr int UPS = BITS == 8 ? 2 : 1;  // weight units (128 rows x 64 packed bytes) per pipeline stage
        const int q = warp & 3, grp = (warp - kEpiWarps) >> 2;
        const int r = q * 32 + lane;
        const bool leader = (q == 0 && lane == 0);
        const int bar_id = 1 + grp;  // named barrier of the group (0 is __syncthreads)
        const int gpr = p.K >> p.gshift;
        const int ng_full = (kSub * kBK) >> p.gshift;  // scale groups per full stage: 4, 2 or 1
        const bool vec_ok = (gpr % ng_full) == 0;      // then a stage's scales of one row are one aligned vector
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + kAColBase;
        // this group's weight unit in shared memory; row r is 64 bytes, its 16-byte chunk c sits at c ^ ((r >> 1) & 3)
        const unsigned char* wrow = sW + (size_t)grp * kWUnitBytes + r * 64;
        const uint32_t wsw = (uint32_t)(r >> 1) & 3u;
        uint64_t* wbar = &sl->wfull[grp];
        uint32_t wround = 0;  // units of this group consumed so far

        // An owned stage: the CTA's stages are counted 0, 1, 2, ... along its range of units (the same count
        // the producer and the MMA issuer keep); group grp owns the counts = grp (mod kDqGroups).
        struct Cur { int tile, st; uint32_t it; };  // tile and stage in the tile of count `it`; tile >= total_tiles: past the end
        const long long u_lo = SK ? total_units * blockIdx.x / gridDim.x : 0;
        const uint32_t u_cnt = SK ? (uint32_t)(total_units * (blockIdx.x + 1) / gridDim.x - u_lo)
                                  : (uint32_t)((total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x * nst);
        const int tile_lo = SK ? (int)(u_lo / nst) : (int)blockIdx.x;  // (the one 64-bit division of the walk)
        const int st_lo = SK ? (int)(u_lo % nst) : 0;
        const int tile_step = SK ? 1 : (int)gridDim.x;
        auto advance = [&](Cur& c, int by) {  // `by` stages further along the CTA's sequence of stages
            c.it += by;
            if (c.it >= u_cnt) {
                c.tile = total_tiles;
                return;
            }
            c.st += by;
            while (c.st >= nst) {
                c.st -= nst;
                c.tile += tile_step;
            }
        };
        auto issue = [&](const Cur& c, int u) {  // leader: bring unit u of stage c into the group's slot
            mbar_expect_tx(wbar, kWUnitBytes);
            tma_load_2d(const_cast<unsigned char*>(sW) + (size_t)grp * kWUnitBytes, &tmap_w,
                        c.st * (kSub * kBK * BITS / 8) + u * 64, (c.tile / p.m_tiles) * kTileN, wbar);
        };
        uint32_t sp[2], bp[2];  // scales / biases of the next owned stage of this row, bf16 pairs in group order
        auto fetch_sb = [&](const Cur& c) {
            const int n = min((c.tile / p.m_tiles) * kTileN + r, p.N - 1);
            const int g0 = (c.st * kSub * kBK) >> p.gshift;
            const int ng = min(gpr - g0, ng_full);
            const uint16_t* sr = reinterpret_cast<const uint16_t*>(p.scales) + (size_t)n * gpr + g0;
            const uint16_t* br = reinterpret_cast<const uint16_t*>(p.biases) + (size_t)n * gpr + g0;
            sp[1] = 0; bp[1] = 0;
            if (vec_ok && ng == ng_full && ng == 4) {
                asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(sp[0]), "=r"(sp[1]) : "l"(sr));
                asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(bp[0]), "=r"(bp[1]) : "l"(br));
            } else if (vec_ok && ng == ng_full && ng == 2) {
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(sp[0]) : "l"(sr));
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(bp[0]) : "l"(br));
            } else {
                sp[0] = ldg_u16(sr); bp[0] = ldg_u16(br);
                if (ng > 1) { sp[0] |= ldg_u16(sr + 1) << 16; bp[0] |= ldg_u16(br + 1) << 16; }
                if (ng > 2) { sp[1] = ldg_u16(sr + 2); bp[1] = ldg_u16(br + 2); }
                if (ng > 3) { sp[1] |= ldg_u16(sr + 3) << 16; bp[1] |= ldg_u16(br + 3) << 16; }
            }
        };

        Cur cur{tile_lo, st_lo, 0u};
        advance(cur, grp);
        if (cur.tile < total_tiles) {
            if (leader) issue(cur, 0);
            fetch_sb(cur);
        }
        bool ok = true;
        while (cur.tile < total_tiles) {
            Cur nxt = cur;
            advance(nxt, kDqGroups);
            const uint32_t it = cur.it;
            const int sa = it % kStagesB;
            const int nsub = min(kSub, nks - cur.st * kSub);
            const uint32_t sc[2] = {sp[0], sp[1]}, bc[2] = {bp[0], bp[1]};
            if (nxt.tile < total_tiles) fetch_sb(nxt);  // three stages ahead of its use
            uint32_t w[16];
            bool group_fail = false;
#pragma unroll
            for (int u = 0; u < kSub; u++) {
                if (u >= nsub) break;
                if (UPS == 2 || u == 0) {
                    const bool got = ok && mbar_wait(wbar, wround & 1, abort_flag);
                    wround++;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const uint4 v = *reinterpret_cast<const uint4*>(wrow + ((c ^ wsw) << 4));
                        w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
                    }
                    // The reads above are generic-proxy accesses, the refill is an async-proxy write: the proxy
                    // fence orders the two (without it a read still in the load pipe could see the next unit).
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    // every thread of the group has its bytes: the slot may be refilled.  The same barrier makes
                    // a failed wait a decision of the whole group, so nobody is left waiting at it.
                    ok = group_all(bar_id, got);
                    if (!ok) { group_fail = true; break; }
                    if (leader) {
                        if (UPS == 2 && u + 1 < nsub) issue(cur, u + 1);
                        else if (nxt.tile < total_tiles) issue(nxt, 0);
                    }
                }
                // scales of the two 32-weight halves of this sub-block
                const int h0 = (2 * u * 32) >> p.gshift, h1 = ((2 * u + 1) * 32) >> p.gshift;
                const uint32_t s0 = (sc[h0 >> 1] >> ((h0 & 1) * 16)) & 0xFFFFu, b0 = (bc[h0 >> 1] >> ((h0 & 1) * 16)) & 0xFFFFu;
                const uint32_t s1 = (sc[h1 >> 1] >> ((h1 & 1) * 16)) & 0xFFFFu, b1 = (bc[h1 >> 1] >> ((h1 & 1) * 16)) & 0xFFFFu;
                uint32_t out[32];
                const uint32_t (&ws)[WPS] = *reinterpret_cast<const uint32_t (*)[WPS]>(&w[BITS == 4 ? 8 * u : 0]);
                if (scale_fast_ok(s0) && scale_fast_ok(s1)) dequant_row_stage<BITS, true>(ws, s0, b0, s1, b1, out);
                else dequant_row_stage<BITS, false>(ws, s0, b0, s1, b1, out);  // whole-block branch: not if-converted
                if (u == 0) {
                    // (every lane waits: with one lane polling for the warp the wake-up came later and the launch
                    // took 3 % longer)
                    const bool freed = ok && mbar_wait(&sl->empty[sa], ((it / kStagesB) & 1) ^ 1, abort_flag);
                    ok = __all_sync(0xFFFFFFFFu, freed);  // tcgen05.st below is warp-collective
                    tc_fence_after();
                }
                __syncwarp();
                if (ok) tmem_st32(lane_addr + sa * kAColsPerSlot + u * kAColsPerSub, out);
            }
            if (ok) {
                tmem_st_wait();  // once per stage: both sub-blocks are in tensor memory
                tc_fence_before();
                mbar_arrive(&sl->full[sa]);
            } else if (!*abort_flag) {
                *abort_flag = 1;
            }
            if (group_fail) break;  // decided by the whole group at its barrier
            cur = nxt;                // a warp that failed alone goes on to the next barrier, where the group ends
        }
    } else {
        // ---------------- epilogue: warp w reads TMEM lanes 32*(w%4).., half w/4 of the column blocks ----------------
        const int q = warp & 3, half = warp >> 2;
        const int nblk = (p.bm + 31) / 32, blk_lo = half ? (nblk + 1) / 2 : 0, blk_hi = half ? nblk : (nblk + 1) / 2;
        const int et = tid;                       // 0 .. 255: the epilogue threads are the first eight warps
        const int nl = q * 32 + lane;             // this thread's row of the tile (TMEM lane)
        constexpr int kEpiBar = 1 + kDqGroups;    // named barrier of the epilogue warps
        uint32_t tile_i = 0;
        bool ok = true;
        SegIter<SK> seg;
        for (seg.init(total_units, nst); seg.valid() && ok; seg.next(), tile_i++) {
            const int tile = seg.tile(), s_lo = seg.s_lo(), s_hi = seg.s_hi();
            const int n = (tile / p.m_tiles) * kTileN + nl;
            const int m0 = (tile % p.m_tiles) * p.bm;
            if (!mbar_wait(&sl->tmem_full, tile_i & 1, abort_flag)) break;
            tc_fence_after();
            const int m_end = min(p.bm, p.M - m0);
            if (s_lo != 0) {
                // The segment starts inside a tile: its accumulator is a partial sum, for the CTA that owns the
                // tile's first stages.  [row of x][row of the tile] fp32 in this CTA's slot, then the flag.
                float* ws = p.ws + (size_t)blockIdx.x * (kTileN * kMaxBM);
                for (int blk = blk_lo; blk < blk_hi; blk++) {
                    const int c0 = blk * 32;
                    uint32_t v[32];
                    __syncwarp();
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
                    // (rows past the tile's last row of x are stored too: the slot has room for them and nobody adds them)
#pragma unroll
                    for (int j = 0; j < 32; j++) __stcg(ws + (size_t)(c0 + j) * kTileN + nl, __uint_as_float(v[j]));
                }
                // The stores of all epilogue threads are ordered before the barrier, the barrier before the release
                // of the flag: whoever acquires the flag sees them.  (No fence per thread: it would wait for the
                // stores, with the accumulator still held.)
                asm volatile("bar.sync %0, %1;" ::"n"(kEpiBar), "n"(kEpiWarps * 32) : "memory");
                if (et == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ws_flags + blockIdx.x), "r"(1u) : "memory");
            } else {
                // The segment starts the tile.  If it does not also end it, the CTAs after this one hold the rest:
                // wait (bounded) for their partials, add them in CTA order, then write y.
                const int c_last = s_hi == nst ? (int)blockIdx.x : cta_of_unit((long long)(tile + 1) * nst - 1, total_units);
                const int parts = c_last - (int)blockIdx.x;
                if (parts > 0) {
                    bool got = true;
                    if (et < parts) {
                        const uint32_t* f = p.ws_flags + blockIdx.x + 1 + et;
                        uint32_t v = 0;
                        for (uint32_t i = 0; i < kSpinLimit * 4; i++) {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                            if (v || ((i & 1023u) == 1023u && *abort_flag)) break;
                            __nanosleep(100);
                        }
                        got = v != 0;
                    }
                    uint32_t all;
                    asm volatile(
                        "{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, %2, %3, q; selp.u32 %0, 1, 0, p; }"
                        : "=r"(all) : "r"((uint32_t)got), "n"(kEpiBar), "n"(kEpiWarps * 32) : "memory");
                    if (!all) {
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                }
                // y[m][n] for this thread's n and `cnt` consecutive rows m0 + c0 + j
                // bf16: the thread holds one column of y (its n) for consecutive rows, but y is contiguous along n.
                // Sixteen rows at a time go through the warp's 1 KB of shared memory, [row][n], and leave as
                // 16-byte stores, eight rows of 64 bytes per instruction, instead of 2-byte stores of one row.
                const bool y_vec = p.y_bf16 && ((p.ld | p.col0) & 7) == 0;
                unsigned char* stg = sEpi + (size_t)warp * kEpiStageBytes;
                const int ncol0 = (tile / p.m_tiles) * kTileN + q * 32 + (lane & 3) * 8;  // first of this thread's 8 columns on the way out
                auto store_rows = [&](const uint32_t* v, int c0, int cnt) {
                    if (y_vec) {
                        {
                            constexpr int h = 0;  // (callers on this path pass sixteen rows)
                            __syncwarp();  // the previous sixteen rows have been read
#pragma unroll
                            for (int j = 0; j < 16; j += 2) {
                                const __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(v[h + j]), __uint_as_float(v[h + j + 1]));
                                *reinterpret_cast<__nv_bfloat16*>(stg + j * 64 + lane * 2) = pr.x;
                                *reinterpret_cast<__nv_bfloat16*>(stg + (j + 1) * 64 + lane * 2) = pr.y;
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 2; i++) {
                                const int row = i * 8 + (lane >> 2), m = c0 + h + row;
                                const uint4 val = *reinterpret_cast<const uint4*>(stg + row * 64 + (lane & 3) * 16);
                                if (m >= m_end || ncol0 >= p.N) continue;
                                const size_t idx = (size_t)(m0 + m) * p.ld + p.col0 + ncol0;
                                if (ncol0 + 8 <= p.N) {
                                    for (int dst = 0; dst < p.world; dst++)
                                        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y_all[dst]) + idx) = val;
                                } else {  // the last columns of y: one by one
                                    const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
                                    for (int dst = 0; dst < p.world; dst++) {
                                        uint16_t* yp = reinterpret_cast<uint16_t*>(p.y_all[dst]) + idx;
#pragma unroll
                                        for (int e = 0; e < 8; e++)
                                            if (ncol0 + e < p.N) yp[e] = (uint16_t)(w4[e >> 1] >> ((e & 1) * 16));
                                    }
                                }
                            }
                        }
                        return;
                    }
                    if (n >= p.N) return;
                    // column-sharded layers: the tile goes into every rank's copy of y (peer stores over NVLink)
                    const size_t idx0 = (size_t)(m0 + c0) * p.ld + p.col0 + n;
                    for (int dst = 0; dst < p.world; dst++) {
                        if (p.y_bf16) {
                            __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(p.y_all[dst]) + idx0;
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < cnt && c0 + j < m_end) yp[(size_t)j * p.ld] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        } else {
                            float* yp = reinterpret_cast<float*>(p.y_all[dst]) + idx0;
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < cnt && c0 + j < m_end) yp[(size_t)j * p.ld] = __uint_as_float(v[j]);
                        }
                    }
                };
                if (parts == 0 && y_vec) {
                    // (requesting the next sixteen columns before the current ones are stored was tried: 3 % slower)
                    for (int c0 = blk_lo * 32; c0 < blk_hi * 32; c0 += 16) {
                        uint32_t v[16];
                        __syncwarp();
                        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
                        store_rows(v, c0, 16);
                    }
                } else if (parts == 0) {
                    for (int blk = blk_lo; blk < blk_hi; blk++) {
                        uint32_t v[32];
                        __syncwarp();
                        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + blk * 32, v);
                        store_rows(v, blk * 32, 32);
                    }
                } else {
                    // 16 rows of x at a time (accumulator + one partial in registers); the partial is requested
                    // before the accumulator is read
                    for (int c0 = blk_lo * 32; c0 < blk_hi * 32; c0 += 16) {
                        uint32_t v[32];
                        float pv[16];
                        const float* ws = p.ws + (size_t)(blockIdx.x + 1) * (kTileN * kMaxBM) + (size_t)c0 * kTileN + nl;
#pragma unroll
                        for (int j = 0; j < 16; j++) pv[j] = __ldcg(ws + (size_t)j * kTileN);
                        __syncwarp();
                        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, reinterpret_cast<uint32_t(&)[16]>(v));
                        for (int pt = 1; pt <= parts; pt++) {
#pragma unroll
                            for (int j = 0; j < 16; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + pv[j]);
                            if (pt < parts) {
                                ws += (size_t)kTileN * kMaxBM;
#pragma unroll
                                for (int j = 0; j < 16; j++) pv[j] = __ldcg(ws + (size_t)j * kTileN);
                            }
                        }
                        store_rows(v, c0, 16);
                    }
                }
                if (parts > 0) {
                    // every epilogue thread has read the partials: their flags go back to zero for the next launch
                    asm volatile("bar.sync %0, %1;" ::"n"(kEpiBar), "n"(kEpiWarps * 32) : "memory");
                    if (et < parts) p.ws_flags[blockIdx.x + 1 + et] = 0;
                }
            }
            tc_fence_before();
            mbar_arrive(&sl->tmem_empty);
        }
    }
    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && sl->abort_flag) *p.error = 1;
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Whole tiles, round robin, as a kernel of its own: the same roles without the bookkeeping of split tiles.  (One
// body for both schedules ran this one 5 % slower, and so did every addition tried here -- 16-byte stores through
// shared memory in the epilogue, the look-ahead of the MMA issuer: the launch is sensitive to the amount of code
// its roles execute side by side.)
template <int BITS>
__global__ void __launch_bounds__(kNumThreads, 1)
qmm_tc_tiles_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
              const __grid_constant__ GemmParams p) {
    constexpr int WPS = kBK * BITS / 32;  // packed words per row per stage: 8 | 16
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sB = smem;  // [kStagesB][bm rows][128 B], swizzled (TMA)
    const uint32_t b_bytes = (uint32_t)p.bm * 128;
    unsigned char* sW = sB + (size_t)kStagesB * kSub * kBBytes;  // [kDqGroups][128 rows][64 B], 64-byte swizzle (TMA)
    SmemLayout* sl = reinterpret_cast<SmemLayout*>(sW + (size_t)kDqGroups * kWUnitBytes);
    volatile int* abort_flag = &sl->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nks = p.K / kBK;                  // 64-weight sub-blocks along K
    const int nst = (nks + kSub - 1) / kSub;    // pipeline stages per tile
    const int total_tiles = p.n_tiles * p.m_tiles;

    if (tid == 0) {
        for (int s = 0; s < kStagesB; s++) {
            mbar_init(&sl->full[s], 128 + 1);  // 128 dequantising threads + the TMA producer (with its byte count)
            mbar_init(&sl->empty[s], 1);        // one tcgen05.commit
        }
        for (int g = 0; g < kDqGroups; g++) mbar_init(&sl->wfull[g], 1);  // the group leader's expect_tx
        mbar_init(&sl->tmem_full, 1);
        mbar_init(&sl->tmem_empty, kEpiWarps * 32);
        sl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(&sl->tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sl->tmem_base;

    if (warp == kTmaWarp) {
        // ---------------- TMA producer: x tiles ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * p.bm;
                for (int st = 0; st < nst; st++, it++) {
                    const int sb = it % kStagesB;
                    const uint32_t ph = (it / kStagesB) & 1;
                    const int nsub = min(kSub, nks - st * kSub);
                    if (!mbar_wait(&sl->empty[sb], ph ^ 1, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(&sl->full[sb], b_bytes * nsub);
                    for (int u = 0; u < nsub; u++)
                        tma_load_2d(sB + ((size_t)sb * kSub + u) * kBBytes, &tmap_x, (st * kSub + u) * kBK, m0, &sl->full[sb]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(kTileN, p.bm);
            uint32_t tile_i = 0, slot = 0, phase = 0;
            const uint64_t db0 = umma_desc_sw128(s32(sB));
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, tile_i++) {
                if (!mbar_wait(&sl->tmem_empty, (tile_i & 1) ^ 1, abort_flag)) break;
                tc_fence_after();
                for (int st = 0; st < nst; st++) {
                    const int nsub = min(kSub, nks - st * kSub);
                    if (!mbar_wait_spin(&sl->full[slot], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    for (int u = 0; u < nsub; u++) {
                        const uint64_t db = db0 + (uint64_t)(slot * kSub + u) * (kBBytes >> 4);
                        const uint32_t a_tmem = tmem_base + kAColBase + slot * kAColsPerSlot + u * kAColsPerSub;
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; kk++)  // 16 k = 8 TMEM columns of A, 32 bytes of each B row
                            tc_mma_ts(tmem_base, a_tmem + 8 * kk, db + 2 * kk, idesc, (st | u | kk) != 0 ? 1u : 0u);
                    }
                    tc_commit(&sl->empty[slot]);  // arrives when the MMAs above have consumed their operands
                    if (++slot == kStagesB) { slot = 0; phase ^= 1; }
                }
                if (ok) tc_commit(&sl->tmem_full);
            }
        }
    } else if (warp >= kEpiWarps) {
        // ---------------- dequantisers: group grp owns the stages = grp (mod kDqGroups); thread owns row n0 + r ----------------
        constexpr int UPS = BITS == 8 ? 2 : 1;  // weight units (128 rows x 64 packed bytes) per pipeline stage
        const int q = warp & 3, grp = (warp - kEpiWarps) >> 2;
        const int r = q * 32 + lane;
        const bool leader = (q == 0 && lane == 0);
        const int bar_id = 1 + grp;  // named barrier of the group (0 is __syncthreads)
        const int gpr = p.K >> p.gshift;
        const int ng_full = (kSub * kBK) >> p.gshift;  // scale groups per full stage: 4, 2 or 1
        const bool vec_ok = (gpr % ng_full) == 0;      // then a stage's scales of one row are one aligned vector
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + kAColBase;
        // this group's weight unit in shared memory; row r is 64 bytes, its 16-byte chunk c sits at c ^ ((r >> 1) & 3)
        const unsigned char* wrow = sW + (size_t)grp * kWUnitBytes + r * 64;
        const uint32_t wsw = (uint32_t)(r >> 1) & 3u;
        uint64_t* wbar = &sl->wfull[grp];
        uint32_t wround = 0;  // units of this group consumed so far

        struct Cur { int tile, st; uint32_t it0; };  // an owned stage: tile, stage in the tile, stage counter at tile start
        auto settle = [&](Cur& c) {  // first stage of c.tile owned by the group; tiles without one are skipped
            while (c.tile < total_tiles) {
                c.st = (int)((grp + kDqGroups - c.it0 % kDqGroups) % kDqGroups);
                if (c.st < nst) break;
                c.tile += gridDim.x;
                c.it0 += nst;
            }
        };
        auto advance = [&](Cur& c) {
            c.st += kDqGroups;
            if (c.st >= nst) {
                c.tile += gridDim.x;
                c.it0 += nst;
                settle(c);
            }
        };
        auto issue = [&](const Cur& c, int u) {  // leader: bring unit u of stage c into the group's slot
            mbar_expect_tx(wbar, kWUnitBytes);
            tma_load_2d(const_cast<unsigned char*>(sW) + (size_t)grp * kWUnitBytes, &tmap_w,
                        c.st * (kSub * kBK * BITS / 8) + u * 64, (c.tile / p.m_tiles) * kTileN, wbar);
        };
        uint32_t sp[2], bp[2];  // scales / biases of the next owned stage of this row, bf16 pairs in group order
        auto fetch_sb = [&](const Cur& c) {
            const int n = min((c.tile / p.m_tiles) * kTileN + r, p.N - 1);
            const int g0 = (c.st * kSub * kBK) >> p.gshift;
            const int ng = min(gpr - g0, ng_full);
            const uint16_t* sr = reinterpret_cast<const uint16_t*>(p.scales) + (size_t)n * gpr + g0;
            const uint16_t* br = reinterpret_cast<const uint16_t*>(p.biases) + (size_t)n * gpr + g0;
            sp[1] = 0; bp[1] = 0;
            if (vec_ok && ng == ng_full && ng == 4) {
                asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(sp[0]), "=r"(sp[1]) : "l"(sr));
                asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(bp[0]), "=r"(bp[1]) : "l"(br));
            } else if (vec_ok && ng == ng_full && ng == 2) {
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(sp[0]) : "l"(sr));
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(bp[0]) : "l"(br));
            } else {
                sp[0] = ldg_u16(sr); bp[0] = ldg_u16(br);
                if (ng > 1) { sp[0] |= ldg_u16(sr + 1) << 16; bp[0] |= ldg_u16(br + 1) << 16; }
                if (ng > 2) { sp[1] = ldg_u16(sr + 2); bp[1] = ldg_u16(br + 2); }
                if (ng > 3) { sp[1] |= ldg_u16(sr + 3) << 16; bp[1] |= ldg_u16(br + 3) << 16; }
            }
        };

        Cur cur{(int)blockIdx.x, 0, 0u};
        settle(cur);
        if (cur.tile < total_tiles) {
            if (leader) issue(cur, 0);
            fetch_sb(cur);
        }
        bool ok = true;
        while (cur.tile < total_tiles) {
            Cur nxt = cur;
            advance(nxt);
            const uint32_t it = cur.it0 + cur.st;
            const int sa = it % kStagesB;
            const int nsub = min(kSub, nks - cur.st * kSub);
            const uint32_t sc[2] = {sp[0], sp[1]}, bc[2] = {bp[0], bp[1]};
            if (nxt.tile < total_tiles) fetch_sb(nxt);  // three stages ahead of its use
            uint32_t w[16];
            bool group_fail = false;
#pragma unroll
            for (int u = 0; u < kSub; u++) {
                if (u >= nsub) break;
                if (UPS == 2 || u == 0) {
                    const bool got = ok && mbar_wait(wbar, wround & 1, abort_flag);
                    wround++;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const uint4 v = *reinterpret_cast<const uint4*>(wrow + ((c ^ wsw) << 4));
                        w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
                    }
                    // The reads above are generic-proxy accesses, the refill is an async-proxy write: the proxy
                    // fence orders the two (without it a read still in the load pipe could see the next unit).
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    // every thread of the group has its bytes: the slot may be refilled.  The same barrier makes
                    // a failed wait a decision of the whole group, so nobody is left waiting at it.
                    ok = group_all(bar_id, got);
                    if (!ok) { group_fail = true; break; }
                    if (leader) {
                        if (UPS == 2 && u + 1 < nsub) issue(cur, u + 1);
                        else if (nxt.tile < total_tiles) issue(nxt, 0);
                    }
                }
                // scales of the two 32-weight halves of this sub-block
                const int h0 = (2 * u * 32) >> p.gshift, h1 = ((2 * u + 1) * 32) >> p.gshift;
                const uint32_t s0 = (sc[h0 >> 1] >> ((h0 & 1) * 16)) & 0xFFFFu, b0 = (bc[h0 >> 1] >> ((h0 & 1) * 16)) & 0xFFFFu;
                const uint32_t s1 = (sc[h1 >> 1] >> ((h1 & 1) * 16)) & 0xFFFFu, b1 = (bc[h1 >> 1] >> ((h1 & 1) * 16)) & 0xFFFFu;
                uint32_t out[32];
                const uint32_t (&ws)[WPS] = *reinterpret_cast<const uint32_t (*)[WPS]>(&w[BITS == 4 ? 8 * u : 0]);
                if (scale_fast_ok(s0) && scale_fast_ok(s1)) dequant_row_stage<BITS, true>(ws, s0, b0, s1, b1, out);
                else dequant_row_stage<BITS, false>(ws, s0, b0, s1, b1, out);  // whole-block branch: not if-converted
                if (u == 0) {
                    const bool freed = ok && mbar_wait(&sl->empty[sa], ((it / kStagesB) & 1) ^ 1, abort_flag);
                    ok = __all_sync(0xFFFFFFFFu, freed);  // tcgen05.st below is warp-collective
                    tc_fence_after();
                }
                __syncwarp();
                if (ok) tmem_st32(lane_addr + sa * kAColsPerSlot + u * kAColsPerSub, out);
            }
            if (ok) {
                tmem_st_wait();  // once per stage: both sub-blocks are in tensor memory
                tc_fence_before();
                mbar_arrive(&sl->full[sa]);
            } else if (!*abort_flag) {
                *abort_flag = 1;
            }
            if (group_fail) break;  // decided by the whole group at its barrier
            cur = nxt;                // a warp that failed alone goes on to the next barrier, where the group ends
        }
    } else {
        // ---------------- epilogue: warp w reads TMEM lanes 32*(w%4).., half w/4 of the column blocks ----------------
        const int q = warp & 3, half = warp >> 2;
        const int nblk = (p.bm + 31) / 32, blk_lo = half ? (nblk + 1) / 2 : 0, blk_hi = half ? nblk : (nblk + 1) / 2;
        uint32_t tile_i = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tile_i++) {
            const int n = (tile / p.m_tiles) * kTileN + q * 32 + lane;
            const int m0 = (tile % p.m_tiles) * p.bm;
            if (!mbar_wait(&sl->tmem_full, tile_i & 1, abort_flag)) break;
            tc_fence_after();
            // this thread: column n of y, rows m0 + c (32 consecutive n per warp: 64-byte row segments)
            const int m_end = min(p.bm, p.M - m0);
            for (int blk = blk_lo; blk < blk_hi; blk++) {
                const int c0 = blk * 32;
                uint32_t v[32];
                __syncwarp();
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
                if (n < p.N) {
                    // column-sharded layers: the tile goes into every rank's copy of y (peer stores over NVLink)
                    const size_t idx0 = (size_t)(m0 + c0) * p.ld + p.col0 + n;
                    for (int dst = 0; dst < p.world; dst++) {
                        if (p.y_bf16) {
                            __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(p.y_all[dst]) + idx0;
                            if (c0 + 32 <= m_end) {
#pragma unroll
                                for (int j = 0; j < 32; j++) yp[(size_t)j * p.ld] = __float2bfloat16_rn(__uint_as_float(v[j]));
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (c0 + j < m_end) yp[(size_t)j * p.ld] = __float2bfloat16_rn(__uint_as_float(v[j]));
                            }
                        } else {
                            float* yp = reinterpret_cast<float*>(p.y_all[dst]) + idx0;
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (c0 + j < m_end) yp[(size_t)j * p.ld] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&sl->tmem_empty);
        }
    }
    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && sl->abort_flag) *p.error = 1;
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster share one MMA stream ------------------------------------
// The MMA is 256 rows of W (128 from each CTA's tensor memory) x bm rows of x, of which each CTA stages half in
// its shared memory; the thread that issues it (in CTA 0) issues for both tensor cores, so the instruction
// stream that bounds a stage is halved per SM, and x takes half the shared memory per stage.
constexpr int kStagesP = 3;                   // k-stages in flight: x halves in shared memory, A in TMEM.  (Four, with
                                              // the 64 KB more of shared memory they take from L1, measured the same or slower.)
constexpr int kPairBBytes = (kMaxBM / 2) * 128;  // one sub-block of this CTA's half of x
constexpr int kPairYBytes = kMaxBM * kTileN * 2; // a finished tile of y as bf16
constexpr int kPairEpiBar = 1 + kDqGroups;       // named barrier of the epilogue warps
static_assert(kDqGroups <= kStagesP, "parity waits would alias");
static_assert(kAColBase + kStagesP * kAColsPerSlot <= kTmemCols, "A ring does not fit");
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // a shared::cluster address with this bit cleared is CTA 0's copy
struct PairSmemLayout {
    uint64_t full[kStagesP], empty[kStagesP], wfull[kDqGroups], tmem_full, tmem_empty;
    uint32_t tmem_base;
    int abort_flag;
};
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {  // whole warp, the same warp in both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on CTA 0's copy of a barrier (from either CTA)
__device__ __forceinline__ void mbar_arrive_cta0(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(s32(b) & kPeerBitMask) : "memory");
}
// arrives once on the barrier at this offset in both CTAs when the MMAs issued so far have completed
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(s32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t z = 0;
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z) : "memory");
}
// a finished tile of y from shared memory ([row of x][128 columns] bf16) to global memory; rows and columns past
// the ends of y are clipped by the copy engine
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(s32(src)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// this CTA's half of an x tile into its own shared memory, completion counted on CTA 0's barrier (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(s32(dst)), "l"(map), "r"(x), "r"(y), "r"(s32(bar) & kPeerBitMask) : "memory");
}

template <int BITS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
qmm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ GemmParams p) {
    constexpr int WPS = kBK * BITS / 32;  // packed words per row per stage: 8 | 16
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sB = smem;  // [kStagesP][kSub][bm/2 rows][128 B], swizzled (TMA): this CTA's half of the x tile
    const uint32_t b_bytes = (uint32_t)(p.bm >> 1) * 128;
    unsigned char* sW = sB + (size_t)kStagesP * kSub * kPairBBytes;  // [kDqGroups][128 rows][64 B], 64-byte swizzle (TMA)
    unsigned char* sY = sW + (size_t)kDqGroups * kWUnitBytes;  // [bm rows of x][128 columns] bf16: a finished tile on its way out
    // (without the staging buffer the shared memory is that much smaller, and L1, which holds the rows' scales and
    // biases over a tile, that much larger: worth 4 % on this kernel)
    PairSmemLayout* sl = reinterpret_cast<PairSmemLayout*>(sY + (p.y_tma ? kPairYBytes : 0));
    uint32_t rank;  // of this CTA in its pair: 0 issues the MMAs of both
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int cl = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);
    volatile int* abort_flag = &sl->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nks = p.K / kBK;                  // 64-weight sub-blocks along K
    const int nst = (nks + kSub - 1) / kSub;    // pipeline stages per tile
    // A pair takes two neighbouring 128-row tiles of W (CTA `rank` the tile 2*np + rank) against the same rows of x;
    // with an odd number of W tiles the last pair's second CTA works on rows past N (zeros in, nothing out).
    const int total_tiles = ((p.n_tiles + 1) >> 1) * p.m_tiles;  // pair tiles
    auto n0_of = [&](int pt) { return ((pt / p.m_tiles) * 2 + (int)rank) * kTileN; };

    if (tid == 0) {
        for (int s = 0; s < kStagesP; s++) {
            // (used in CTA 0 only) the four warps of the owning group in either CTA + CTA 0's TMA producer, whose
            // byte count covers both CTAs' halves of x
            mbar_init(&sl->full[s], 4 + 4 + 1);
            mbar_init(&sl->empty[s], 1);  // one tcgen05.commit, multicast to both CTAs
        }
        for (int g = 0; g < kDqGroups; g++) mbar_init(&sl->wfull[g], 1);  // the group leader's expect_tx
        mbar_init(&sl->tmem_full, 1);
        mbar_init(&sl->tmem_empty, 2 * kEpiWarps);  // (used in CTA 0 only) the epilogue warps of both CTAs
        sl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc_pair(&sl->tmem_base, kTmemCols);  // the same warp of both CTAs
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = sl->tmem_base;

    if (warp == kTmaWarp) {
        // ---------------- TMA producer: x tiles ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cl; tile < total_tiles && ok; tile += ncl) {
                const int m0 = (tile % p.m_tiles) * p.bm + (int)rank * (p.bm >> 1);  // this CTA's half of the rows of x
                for (int st = 0; st < nst; st++, it++) {
                    const int sb = it % kStagesP;
                    const uint32_t ph = (it / kStagesP) & 1;
                    const int nsub = min(kSub, nks - st * kSub);
                    if (!mbar_wait(&sl->empty[sb], ph ^ 1, abort_flag)) { ok = false; break; }
                    // both halves complete on CTA 0's barrier, which expects the bytes of both
                    if (rank == 0) mbar_expect_tx(&sl->full[sb], 2 * b_bytes * nsub);
                    for (int u = 0; u < nsub; u++)
                        tma_load_2d_pair(sB + ((size_t)sb * kSub + u) * kPairBBytes, &tmap_x, (st * kSub + u) * kBK, m0, &sl->full[sb]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc(2 * kTileN, p.bm);  // 256 rows of W over the two CTAs x bm rows of x
            uint32_t tile_i = 0, slot = 0, phase = 0;
            const uint64_t db0 = umma_desc_sw128(s32(sB));
            bool ok = true;
            for (int tile = cl; tile < total_tiles && ok; tile += ncl, tile_i++) {
                if (!mbar_wait(&sl->tmem_empty, (tile_i & 1) ^ 1, abort_flag)) break;
                tc_fence_after();
                for (int st = 0; st < nst; st++) {
                    const int nsub = min(kSub, nks - st * kSub);
                    if (!mbar_wait_spin(&sl->full[slot], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    for (int u = 0; u < nsub; u++) {
                        const uint64_t db = db0 + (uint64_t)(slot * kSub + u) * (kPairBBytes >> 4);
                        const uint32_t a_tmem = tmem_base + kAColBase + slot * kAColsPerSlot + u * kAColsPerSub;
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; kk++)  // 16 k = 8 TMEM columns of A, 32 bytes of each B row
                            tc_mma_ts_pair(tmem_base, a_tmem + 8 * kk, db + 2 * kk, idesc, (st | u | kk) != 0 ? 1u : 0u);
                    }
                    tc_commit_pair(&sl->empty[slot]);  // arrives, in both CTAs, when the MMAs above have consumed their operands
                    if (++slot == kStagesP) { slot = 0; phase ^= 1; }
                }
                if (ok) tc_commit_pair(&sl->tmem_full);
            }
        }
    } else if (warp >= kEpiWarps) {
        // ---------------- dequantisers: group grp owns the stages = grp (mod kDqGroups); thread owns row n0 + r ----------------
        constexpr int UPS = BITS == 8 ? 2 : 1;  // weight units (128 rows x 64 packed bytes) per pipeline stage
        const int q = warp & 3, grp = (warp - kEpiWarps) >> 2;
        const int r = q * 32 + lane;
        const bool leader = (q == 0 && lane == 0);
        const int bar_id = 1 + grp;  // named barrier of the group (0 is __syncthreads)
        const int gpr = p.K >> p.gshift;
        const int ng_full = (kSub * kBK) >> p.gshift;  // scale groups per full stage: 4, 2 or 1
        const bool vec_ok = (gpr % ng_full) == 0;      // then a stage's scales of one row are one aligned vector
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + kAColBase;
        // this group's weight unit in shared memory; row r is 64 bytes, its 16-byte chunk c sits at c ^ ((r >> 1) & 3)
        const unsigned char* wrow = sW + (size_t)grp * kWUnitBytes + r * 64;
        const uint32_t wsw = (uint32_t)(r >> 1) & 3u;
        uint64_t* wbar = &sl->wfull[grp];
        uint32_t wround = 0;  // units of this group consumed so far

        struct Cur { int tile, st; uint32_t it0; };  // an owned stage: tile, stage in the tile, stage counter at tile start
        auto settle = [&](Cur& c) {  // first stage of c.tile owned by the group; tiles without one are skipped
            while (c.tile < total_tiles) {
                c.st = (int)((grp + kDqGroups - c.it0 % kDqGroups) % kDqGroups);
                if (c.st < nst) break;
                c.tile += ncl;
                c.it0 += nst;
            }
        };
        auto advance = [&](Cur& c) {
            c.st += kDqGroups;
            if (c.st >= nst) {
                c.tile += ncl;
                c.it0 += nst;
                settle(c);
            }
        };
        auto issue = [&](const Cur& c, int u) {  // leader: bring unit u of stage c into the group's slot
            mbar_expect_tx(wbar, kWUnitBytes);
            tma_load_2d(const_cast<unsigned char*>(sW) + (size_t)grp * kWUnitBytes, &tmap_w,
                        c.st * (kSub * kBK * BITS / 8) + u * 64, n0_of(c.tile), wbar);
        };
        uint32_t sp[2], bp[2];  // scales / biases of the next owned stage of this row, bf16 pairs in group order
        auto fetch_sb = [&](const Cur& c) {
            const int n = min(n0_of(c.tile) + r, p.N - 1);
            const int g0 = (c.st * kSub * kBK) >> p.gshift;
            const int ng = min(gpr - g0, ng_full);
            const uint16_t* sr = reinterpret_cast<const uint16_t*>(p.scales) + (size_t)n * gpr + g0;
            const uint16_t* br = reinterpret_cast<const uint16_t*>(p.biases) + (size_t)n * gpr + g0;
            sp[1] = 0; bp[1] = 0;
            if (vec_ok && ng == ng_full && ng == 4) {
                asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(sp[0]), "=r"(sp[1]) : "l"(sr));
                asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(bp[0]), "=r"(bp[1]) : "l"(br));
            } else if (vec_ok && ng == ng_full && ng == 2) {
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(sp[0]) : "l"(sr));
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(bp[0]) : "l"(br));
            } else {
                sp[0] = ldg_u16(sr); bp[0] = ldg_u16(br);
                if (ng > 1) { sp[0] |= ldg_u16(sr + 1) << 16; bp[0] |= ldg_u16(br + 1) << 16; }
                if (ng > 2) { sp[1] = ldg_u16(sr + 2); bp[1] = ldg_u16(br + 2); }
                if (ng > 3) { sp[1] |= ldg_u16(sr + 3) << 16; bp[1] |= ldg_u16(br + 3) << 16; }
            }
        };

        Cur cur{cl, 0, 0u};
        settle(cur);
        if (cur.tile < total_tiles) {
            if (leader) issue(cur, 0);
            fetch_sb(cur);
        }
        bool ok = true;
        while (cur.tile < total_tiles) {
            Cur nxt = cur;
            advance(nxt);
            const uint32_t it = cur.it0 + cur.st;
            const int sa = it % kStagesP;
            const int nsub = min(kSub, nks - cur.st * kSub);
            const uint32_t sc[2] = {sp[0], sp[1]}, bc[2] = {bp[0], bp[1]};
            if (nxt.tile < total_tiles) fetch_sb(nxt);  // three stages ahead of its use
            uint32_t w[16];
            bool group_fail = false;
#pragma unroll
            for (int u = 0; u < kSub; u++) {
                if (u >= nsub) break;
                if (UPS == 2 || u == 0) {
                    const bool got = ok && mbar_wait(wbar, wround & 1, abort_flag);
                    wround++;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const uint4 v = *reinterpret_cast<const uint4*>(wrow + ((c ^ wsw) << 4));
                        w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
                    }
                    // The reads above are generic-proxy accesses, the refill is an async-proxy write: the proxy
                    // fence orders the two (without it a read still in the load pipe could see the next unit).
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    // every thread of the group has its bytes: the slot may be refilled.  The same barrier makes
                    // a failed wait a decision of the whole group, so nobody is left waiting at it.
                    ok = group_all(bar_id, got);
                    if (!ok) { group_fail = true; break; }
                    if (leader) {
                        if (UPS == 2 && u + 1 < nsub) issue(cur, u + 1);
                        else if (nxt.tile < total_tiles) issue(nxt, 0);
                    }
                }
                // scales of the two 32-weight halves of this sub-block
                const int h0 = (2 * u * 32) >> p.gshift, h1 = ((2 * u + 1) * 32) >> p.gshift;
                const uint32_t s0 = (sc[h0 >> 1] >> ((h0 & 1) * 16)) & 0xFFFFu, b0 = (bc[h0 >> 1] >> ((h0 & 1) * 16)) & 0xFFFFu;
                const uint32_t s1 = (sc[h1 >> 1] >> ((h1 & 1) * 16)) & 0xFFFFu, b1 = (bc[h1 >> 1] >> ((h1 & 1) * 16)) & 0xFFFFu;
                uint32_t out[32];
                const uint32_t (&ws)[WPS] = *reinterpret_cast<const uint32_t (*)[WPS]>(&w[BITS == 4 ? 8 * u : 0]);
                if (scale_fast_ok(s0) && scale_fast_ok(s1)) dequant_row_stage<BITS, true>(ws, s0, b0, s1, b1, out);
                else dequant_row_stage<BITS, false>(ws, s0, b0, s1, b1, out);  // whole-block branch: not if-converted
                if (u == 0) {
                    const bool freed = ok && mbar_wait(&sl->empty[sa], ((it / kStagesP) & 1) ^ 1, abort_flag);
                    ok = __all_sync(0xFFFFFFFFu, freed);  // tcgen05.st below is warp-collective
                    tc_fence_after();
                }
                __syncwarp();
                if (ok) tmem_st32(lane_addr + sa * kAColsPerSlot + u * kAColsPerSub, out);
            }
            if (ok) {
                tmem_st_wait();  // once per stage: both sub-blocks are in tensor memory
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cta0(&sl->full[sa]);  // one arrival per warp, on the barrier the MMA issuer waits at
            } else if (!*abort_flag) {
                *abort_flag = 1;
            }
            if (group_fail) break;  // decided by the whole group at its barrier
            cur = nxt;                // a warp that failed alone goes on to the next barrier, where the group ends
        }
    } else {
        // ---------------- epilogue: warp w reads TMEM lanes 32*(w%4).., half w/4 of the column blocks ----------------
        const int q = warp & 3, half = warp >> 2;
        const int nblk = (p.bm + 31) / 32, blk_lo = half ? (nblk + 1) / 2 : 0, blk_hi = half ? nblk : (nblk + 1) / 2;
        uint32_t tile_i = 0;
        for (int tile = cl; tile < total_tiles; tile += ncl, tile_i++) {
            const int n = n0_of(tile) + q * 32 + lane;
            const int m0 = (tile % p.m_tiles) * p.bm;
            if (p.y_tma && tile_i > 0) {
                // the copy engine has finished reading the previous tile out of the staging buffer
                if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                asm volatile("bar.sync %0, %1;" ::"n"(kPairEpiBar), "n"(kEpiWarps * 32) : "memory");
            }
            if (!mbar_wait(&sl->tmem_full, tile_i & 1, abort_flag)) break;
            tc_fence_after();
            if (p.y_tma) {
                // The accumulator goes to shared memory as bf16, [row of x][column], and is released at once; the
                // copy engine takes the tile to y while the next tile's MMAs run.
                for (int blk = blk_lo; blk < blk_hi; blk++) {
                    const int c0 = blk * 32;
                    uint32_t v[32];
                    __syncwarp();
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(sY + (size_t)c0 * 256) + q * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 32; j++) dst[j * 128] = __float2bfloat16_rn(__uint_as_float(v[j]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cta0(&sl->tmem_empty);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes, then the copy engine's reads
                asm volatile("bar.sync %0, %1;" ::"n"(kPairEpiBar), "n"(kEpiWarps * 32) : "memory");
                if (p.y_tma == 1) {
                    if (tid == 0 && n0_of(tile) < p.N) tma_store_2d(&tmap_y, sY, n0_of(tile), m0);
                } else {
                    // column-sharded layers: the tile goes into every rank's copy of y, 16 bytes per store (plain
                    // stores: no TMA on a peer's memory), a row of the tile = 16 lanes
                    const int m_end = min(p.bm, p.M - m0);
                    const int ncol = n0_of(tile) + (tid & 15) * 8;
                    for (int row = tid >> 4; row < m_end; row += (kEpiWarps * 32) >> 4) {
                        const uint4 val = *reinterpret_cast<const uint4*>(sY + (size_t)row * 256 + (tid & 15) * 16);
                        if (ncol >= p.N) continue;
                        const size_t idx = (size_t)(m0 + row) * p.ld + p.col0 + ncol;
                        if (ncol + 8 <= p.N) {
                            for (int dst = 0; dst < p.world; dst++)
                                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y_all[dst]) + idx) = val;
                        } else {  // the last columns of y: one by one
                            const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
                            for (int dst = 0; dst < p.world; dst++) {
                                uint16_t* yp = reinterpret_cast<uint16_t*>(p.y_all[dst]) + idx;
#pragma unroll
                                for (int e = 0; e < 8; e++)
                                    if (ncol + e < p.N) yp[e] = (uint16_t)(w4[e >> 1] >> ((e & 1) * 16));
                            }
                        }
                    }
                }
                continue;
            }
            // this thread: column n of y, rows m0 + c (32 consecutive n per warp: 64-byte row segments)
            const int m_end = min(p.bm, p.M - m0);
            for (int blk = blk_lo; blk < blk_hi; blk++) {
                const int c0 = blk * 32;
                uint32_t v[32];
                __syncwarp();
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
                if (n < p.N) {
                    // column-sharded layers: the tile goes into every rank's copy of y (peer stores over NVLink)
                    const size_t idx0 = (size_t)(m0 + c0) * p.ld + p.col0 + n;
                    for (int dst = 0; dst < p.world; dst++) {
                        if (p.y_bf16) {
                            __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(p.y_all[dst]) + idx0;
                            if (c0 + 32 <= m_end) {
#pragma unroll
                                for (int j = 0; j < 32; j++) yp[(size_t)j * p.ld] = __float2bfloat16_rn(__uint_as_float(v[j]));
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (c0 + j < m_end) yp[(size_t)j * p.ld] = __float2bfloat16_rn(__uint_as_float(v[j]));
                            }
                        } else {
                            float* yp = reinterpret_cast<float*>(p.y_all[dst]) + idx0;
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (c0 + j < m_end) yp[(size_t)j * p.ld] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cta0(&sl->tmem_empty);
        }
    }
    // ---------------- teardown ----------------
    if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the last tile has left
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // neither CTA leaves (or frees tensor memory) while the other may still reach into it
    if (tid == 0 && sl->abort_flag) *p.error = 1;
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
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
    int bm, m_tiles, n_tiles, streamk, pair;
    size_t smem;
};

bool make_gemm_plan(const QmmArgs& a, int sm_count, GemmPlan* pl) {
    if (a.x_dtype != LUX_DTYPE_BFLOAT16 || a.sb_dtype != LUX_DTYPE_BFLOAT16) return false;
    if (a.bits != 4 && a.bits != 8) return false;
    if (a.group != 32 && a.group != 64 && a.group != 128) return false;
    if (a.M <= 16 || a.N < 1 || a.K % kBK) return false;
    if (((uintptr_t)a.x | (uintptr_t)a.wq | (uintptr_t)a.scales | (uintptr_t)a.biases | (uintptr_t)a.y) & 15) return false;
    if ((long long)a.N * (a.K / a.group) > (1ll << 31) - 1) return false;
    pl->n_tiles = (a.N + kTileN - 1) / kTileN;
    // rows of x per tile: as many as the MMA takes.  The time of a tile is set by the dequantisation of
    // its 128 x K weights, not by its height, so fewer, taller tiles always win (measured: 176-row tiles
    // for M = 512 were 20 % slower than 256-row tiles although they need one round of tiles less).
    (void)sm_count;
    pl->m_tiles = (a.M + kMaxBM - 1) / kMaxBM;
    pl->bm = (((a.M + pl->m_tiles - 1) / pl->m_tiles) + 15) & ~15;
    pl->smem = 1024 + (size_t)kStagesB * kSub * kBBytes + (size_t)kDqGroups * kWUnitBytes + (size_t)kEpiWarps * kEpiStageBytes +
               sizeof(SmemLayout) + 64;
    // Schedule.  In units of one k-stage of a tile (about 0.8 us) of the whole-tile kernel: an epilogue costs
    // about e = 4 * bm/256 (the accumulator is single: nothing else runs meanwhile), handing over and adding one
    // partial accumulator about 7 * bm/256 more, and a stage of the stream-K kernel about 1.3 (fitted to
    // measurements of both kernels on shapes from 32 to 512 tiles).  Whole tiles: ceil(T/G) * (nst + e).
    // Stream-K: 1.3 * T*nst/G, one epilogue more, and the partials of the tile a CTA starts.  Stream-K wins
    // where the tiles are few against the SMs (a column-sharded slice, a small M).
    {
        const double T = (double)pl->n_tiles * pl->m_tiles, G = sm_count, nst = (a.K / kBK + kSub - 1) / kSub;
        const double e = 4.0 * pl->bm / 256.0, rounds = std::ceil(T / G);
        const double parts = T < G ? std::ceil(G / T) : 1.0;
        const double whole = rounds * (nst + e);
        const double sk = 1.3 * T * nst / G + (rounds + 1.0) * e + 7.0 * pl->bm / 256.0 * parts;
        pl->streamk = sk < whole && T * nst >= G;
        if (const char* env = getenv("LUXCUDA_QMM_SCHEDULE")) pl->streamk = env[0] == 's';  // "streamk" | "tiles" (experiments)
    }
    // Whole tiles on CTA pairs when the tiles about fill the SMs (measured against the one-CTA kernel on the same
    // box: 256 tiles 59.2 against 60.1 us, 512 tiles 110.6 against 116.3, 448 tiles of the 8-bit shape 215 against
    // 243, 112 tiles 60.3 against 64.0; below that the one-CTA kernel is 2-3 % ahead).
    pl->pair = !pl->streamk && (sm_count & 1) == 0 && 10 * pl->n_tiles * pl->m_tiles >= 7 * sm_count;
    if (const char* env = getenv("LUXCUDA_QMM_PAIR")) pl->pair = !pl->streamk && (sm_count & 1) == 0 && env[0] == '1';  // (experiments)
    if (pl->pair)
        pl->smem = 1024 + (size_t)kStagesP * kSub * kPairBBytes + (size_t)kDqGroups * kWUnitBytes + kPairYBytes + sizeof(PairSmemLayout) + 64;
    return encode_tiled_fn() != nullptr;
}

template <int BITS>
cudaError_t launch_gemm_pair_t(const CUtensorMap& tmap, const CUtensorMap& tmap_w, const CUtensorMap& tmap_y, const GemmParams& p, const GemmPlan& pl, int sm_count, cudaStream_t stream) {
    auto kern = qmm_tc_pair_kernel<BITS>;
    static std::atomic<size_t> attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_smem[dev & 63].load() < pl.smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev & 63].store(pl.smem);
    }
    // one pair of CTAs per pair of SMs (the kernel carries its cluster shape), unless there are fewer pair tiles
    const int pairs = ((pl.n_tiles + 1) / 2) * pl.m_tiles;
    const int grid = 2 * std::min(sm_count / 2, pairs);
    kern<<<grid, kNumThreads, pl.smem, stream>>>(tmap, tmap_w, tmap_y, p);
    return cudaGetLastError();
}

template <int BITS, bool SK>
cudaError_t launch_gemm_t(const CUtensorMap& tmap, const CUtensorMap& tmap_w, const GemmParams& p, const GemmPlan& pl, int sm_count, cudaStream_t stream) {
    auto kern = SK ? qmm_tc_kernel<BITS, true> : qmm_tc_tiles_kernel<BITS>;
    static std::atomic<size_t> attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_smem[dev & 63].load() < pl.smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev & 63].store(pl.smem);
    }
    // one CTA per SM, unless the launch has fewer units of work (tiles, or k-stages under stream-K) than that
    const long long units = (long long)pl.m_tiles * pl.n_tiles * (SK ? (p.K / kBK + kSub - 1) / kSub : 1);
    const int grid = (int)std::min<long long>(sm_count, units);
    kern<<<grid, kNumThreads, pl.smem, stream>>>(tmap, tmap_w, p);
    return cudaGetLastError();
}

}  // namespace

bool qmm_tc_supported(const QmmArgs& a, int sm_count) {
    GemmPlan pl;
    return make_gemm_plan(a, sm_count, &pl);
}

// Scratch of a launch: one partial accumulator and one flag word per CTA (see SegIter).  The flags must be zero
// before the first launch; every launch leaves them zero.
size_t qmm_tc_workspace_bytes(int sm_count) { return kWsFlagBytes + (size_t)sm_count * kTileN * kMaxBM * sizeof(float); }

cudaError_t launch_qmm_tc(const QmmArgs& a, void* workspace, int sm_count, cudaStream_t stream, const char** name,
                          const ShardPush* push) {
    GemmPlan pl;
    if (!make_gemm_plan(a, sm_count, &pl) || !workspace || sm_count * sizeof(uint32_t) > kWsFlagBytes) return cudaErrorInvalidValue;
    int* err = a.error ? a.error : error_word();
    if (!err) return cudaErrorMemoryAllocation;
    // x as a 2-D tensor [M rows][K], boxes of 64 elements (128 bytes) x bm rows, 128-byte swizzle;
    // rows past M are filled with zeros by the copy engine
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)(pl.pair ? pl.bm / 2 : pl.bm)};  // (a CTA of a pair stages half the rows)
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled_fn()(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.x), dims, strides, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed (%d)", (int)r);
        return cudaErrorInvalidValue;
    }
    // the packed weights as bytes, [N rows][K*bits/8], boxes of 64 bytes x 128 rows, 64-byte swizzle
    CUtensorMap tmap_w;
    {
        const cuuint64_t wdims[2] = {(cuuint64_t)a.K * a.bits / 8, (cuuint64_t)a.N};
        const cuuint64_t wstrides[1] = {(cuuint64_t)a.K * a.bits / 8};
        const cuuint32_t wbox[2] = {64u, (cuuint32_t)kTileN};
        r = encode_tiled_fn()(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint32_t*>(a.wq), wdims, wstrides, wbox,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_last_error("cuTensorMapEncodeTiled (weights) failed (%d)", (int)r);
            return cudaErrorInvalidValue;
        }
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
    p.world = 1; p.ld = a.N; p.col0 = 0;
    for (int r = 0; r < kMaxShardWorld; r++) p.y_all[r] = nullptr;
    p.y_all[0] = a.y;
    if (push && push->world > 1) {
        if (push->world > kMaxShardWorld) return cudaErrorInvalidValue;
        p.world = push->world; p.ld = push->ld; p.col0 = push->col0;
        // own copy first, then the peers
        int k = 0;
        p.y_all[k++] = push->y[push->me];
        for (int r = 0; r < push->world; r++)
            if (r != push->me) p.y_all[k++] = push->y[r];
    }
    p.bm = pl.bm; p.n_tiles = pl.n_tiles; p.m_tiles = pl.m_tiles;
    p.ws_flags = static_cast<uint32_t*>(workspace);
    p.ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kWsFlagBytes);
    p.y_tma = 0;
    if (pl.pair) {
        // y as a 2-D tensor [M rows][N] of bf16, boxes of 128 columns x bm rows, for the epilogue's TMA store
        CUtensorMap tmap_y = tmap;
        if (p.y_bf16 && p.world == 1 && (a.N & 7) == 0 && !getenv("LUXCUDA_QMM_NO_YTMA")) {
            const cuuint64_t ydims[2] = {(cuuint64_t)a.N, (cuuint64_t)a.M};
            const cuuint64_t ystrides[1] = {(cuuint64_t)a.N * 2};
            const cuuint32_t ybox[2] = {(cuuint32_t)kTileN, (cuuint32_t)pl.bm};
            r = encode_tiled_fn()(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, ydims, ystrides, ybox, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            p.y_tma = r == CUDA_SUCCESS ? 1 : 0;
        } else if (p.y_bf16 && p.world > 1 && ((p.ld | p.col0) & 7) == 0 && !getenv("LUXCUDA_QMM_NO_YTMA")) {
            p.y_tma = 2;
        }
        if (!p.y_tma) pl.smem -= kPairYBytes;
        if (name) *name = a.bits == 4 ? "qmm_tc<4,pairs>" : "qmm_tc<8,pairs>";
        return a.bits == 4 ? launch_gemm_pair_t<4>(tmap, tmap_w, tmap_y, p, pl, sm_count, stream)
                           : launch_gemm_pair_t<8>(tmap, tmap_w, tmap_y, p, pl, sm_count, stream);
    }
    if (a.bits == 4) {
        if (name) *name = pl.streamk ? "qmm_tc<4,stream-k>" : "qmm_tc<4>";
        return pl.streamk ? launch_gemm_t<4, true>(tmap, tmap_w, p, pl, sm_count, stream)
                          : launch_gemm_t<4, false>(tmap, tmap_w, p, pl, sm_count, stream);
    }
    if (name) *name = pl.streamk ? "qmm_tc<8,stream-k>" : "qmm_tc<8>";
    return pl.streamk ? launch_gemm_t<8, true>(tmap, tmap_w, p, pl, sm_count, stream)
                      : launch_gemm_t<8, false>(tmap, tmap_w, p, pl, sm_count, stream);
}

// Device-side address of the host-visible error word (the same on every GPU: portable mapped memory).
int* device_error_word() {
    int* err = error_word();
    int* derr = nullptr;
    if (!err || cudaHostGetDevicePointer((void**)&derr, err, 0) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return derr;
}

int take_context_error(Context* c) {
    if (!c || !c->err_host) return 0;
    return __atomic_exchange_n(c->err_host, 0, __ATOMIC_ACQ_REL);
}

// Non-zero once a kernel has given up on a bounded wait; reading clears it.
int take_device_error() {
    if (!g_error_host || !*g_error_host) return 0;
    return __atomic_exchange_n(g_error_host, 0, __ATOMIC_ACQ_REL);
}

}  // namespace luxcuda
