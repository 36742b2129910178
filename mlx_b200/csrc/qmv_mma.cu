// Decode-regime quantized GEMV for bf16 activations, M <= 16:
//   y[M,N] = x[M,K] . dequant(Wq[N,K])^T,  w^ = RNE_bf16(s*q + b)  (one bf16 FMA)
//
// HBM-bound: every packed weight word, scale and bias is read from HBM exactly
// once.  Algorithmic bytes per output row: K*bits/8 + 2*(K/group)*2.
//
// A 25 MB layer is a ~4 us stream, shorter than the memory latency ramp, so
// the kernel is built to put as many bytes in flight per SM as early as
// possible and never to make one warp wait for another:
//   * "task" = 16 rows of W x one k-block (128 bytes per row: 256 four-bit or
//     128 eight-bit weights) = 2 KiB of packed weights + its scales/biases;
//   * CTA (one per SM, 16 warps) owns a range of 16-row tiles and a range of
//     k-blocks; warp w owns the k-blocks kb_lo + w + 16*s of that range and
//     walks them over the CTA's tiles;
//   * each warp keeps a private ring of task buffers in shared memory (four, or two
//     with 16 rows of x), filled with cp.async (16-byte pieces, L1 bypass): the
//     tasks ahead of the one being computed (2.5 KiB each) are in flight, with no
//     registers tied up and no block-wide barrier in the streaming loop;
//   * lane (g = lane/4, t = lane%4) copies and later reads back exactly its own
//     pieces: rows g and g+8, the 16-byte pieces t and t+4 of the 128-byte
//     k-block row (so each quad copies 64 contiguous bytes per instruction);
//   * weights are dequantised in registers (dequant.cuh) and fed to
//     mma.sync.m16n8k16 (bf16 x bf16 -> fp32): the <= 16 rows of x cost no
//     extra instruction per weight.  The dot product is invariant under a
//     permutation of k applied to both operands, so the weights are used in
//     the order the mask/shift unpack yields them and the x fragments of the
//     warp's k-block are loaded once, in that order, into registers;
//   * every task leaves a 16 x 8*MT fp32 partial in shared memory; at the end
//     of a batch of tiles the partials of a tile are summed in k-block order
//     (fixed order => the result does not depend on N, on the grid or on how
//     the columns of a layer are sharded over GPUs);
//   * when a layer has too few tiles to fill the GPU, K is split over KS CTAs
//     per tile range: each exports its partials to a global scratch slot and
//     bumps the tile's arrival counter; the last arriver sums all of them,
//     again in k-block order, and resets the counter.  Nobody waits.
#include <cuda_bf16.h>

#include <algorithm>

#include "dequant.cuh"
#include "internal.h"

namespace luxcuda {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
// Ring stages per warp.  Up to 8 rows of x: four (three tasks = 7.5 KiB per warp, 120 KiB per SM in flight);
// with 16 rows the partials and the x fragments kept in shared memory leave room for two.
constexpr int ring_depth(int mt) { return mt == 1 ? 4 : 2; }
constexpr int kStageBytes = 2048 + 512;    // 4 x 32 x 16 B of weights + 32 x 16 B of scales/biases
constexpr int ring_bytes(int mt) { return kWarps * ring_depth(mt) * kStageBytes; }
constexpr int kSmemLimit = 227 * 1024 - 256;
constexpr int kMaxTb = 32;                 // tiles per reduction batch (flags array)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Params {
    const __nv_bfloat16* x;
    const uint32_t* wq;
    const __nv_bfloat16* scales;
    const __nv_bfloat16* biases;
    void* y;
    int* error;              // host-visible error word (bounded waits of the sharded path); may be null
    float* scratch;          // [n_rt][nkb][128*MT] partials of k-split tiles
    unsigned int* counters;  // [n_rt] arrival counters (zero between launches)
    int M, K, N, gshift, y_bf16;
    int nkb, n_rt;
    int chunks, ks;          // grid = chunks (tile ranges) x ks (k-block ranges)
    int chained;             // launched as a programmatic dependent of the previous kernel
    int xs_off;              // byte offset in shared memory of the x fragments kept there (16-row variant)
    int yt_off;              // byte offset in shared memory of the tiles staged for the peers (0: not sharded)
    int tb;                  // tiles per reduction batch
    int sb_bytes;            // bytes of scales per row per k-block: 2, 4, 8 or 16
    int ld, col0;            // y row stride and first column (elements): N and 0 unless the layer is column-sharded
    int x_early;             // x is not written by the previous kernel of the stream: it may be read before the wait for it
    int x_ld;                // row stride of x in elements (K unless a prologue reads column blocks of a wider buffer)
    float eps;               // of the rms-norm prologue
    long long peer_wait_ns;  // limit of a wait for a peer (column-sharded launches)
    ShardPush sp;            // sp.world > 1: the finished tiles are also stored into the peers' copies of y
};

// ---- column-sharded layers: all-gather by peer stores -----------------------------------
// Every rank holds the full y[M, ld]; this rank computes columns [col0, col0 + N), stores them into its own
// copy and sends them over NVLink to every peer.  What travels is 8-byte words, 4 bytes of y plus the
// number of the call ("epoch"), written two at a time (each half is a whole word) into the receiver's inbox
// (inbox[sender][row][word], behind y in the same buffer): a word is either absent or complete, so the
// receiver needs no fence and no acknowledgement -- it polls the words, which costs one NVLink traversal
// instead of three (data, ack, flag).  Each CTA, once its own tiles are sent, unpacks its share of the
// inbox into the local y; when the launch ends the local y is whole, so stream order is all a consumer
// needs.  One hand-shake guards the inbox: a rank announces ready[q] = epoch on every peer when its kernel
// of that call has started -- everything it enqueued before has then finished with its y and inbox -- and a
// sender waits for it before its first remote store.  Waits are bounded (Params::peer_wait_ns): on a time-out the
// kernel raises the host-visible error word, stops waiting (in every later launch too) and returns.
// (kFlagDone + q: the number of the last call of which rank q has delivered ALL its columns here -- the batched
// kernel stores straight into the peers' y and announces once per launch, see qmv_batch_kernel)
constexpr int kFlagEpoch = 0, kFlagCtaDone = 1, kFlagReady = 8, kFlagDone = 16;

__device__ __forceinline__ long long now_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys64x2(unsigned long long* p, unsigned long long a, unsigned long long b) {
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_relaxed_sys64x2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Set by the first wait that runs out and never cleared: from then on no launch of this process waits
// for a peer again (a lost peer must cost one time-out, not one per launch); the host sees the error word.
__device__ int g_peer_lost;
__device__ __forceinline__ bool peer_lost() { return *reinterpret_cast<volatile int*>(&g_peer_lost) != 0; }
// true once *flag has reached epoch e (wrap-around safe)
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t e, long long limit_ns) {
    if (peer_lost()) return false;
    const long long t0 = now_ns();
    for (;;) {
        if ((int32_t)(ld_relaxed_sys(flag) - e) >= 0) return true;
        if (now_ns() - t0 > limit_ns) {
            g_peer_lost = 1;
            return false;
        }
        __nanosleep(100);
    }
}
// Send the finished tile (16 columns of every row of y) to the peers' inboxes.
__device__ __forceinline__ void push_tile(const Params& p, uint32_t epoch, int rt, const unsigned char* ytile,
                                          int tid_in_group, int group_threads) {
    const int esz = p.y_bf16 ? 2 : 4, ppt = 2 * esz;  // pairs of words (8 bytes of y) per tile row: 4 | 8
    const int wpr = p.N * esz / 4;                    // words per row of this rank's columns
    const int per_peer = p.M * ppt;
    const unsigned long long stamp = (unsigned long long)epoch << 32;
    // the tile's words (staged in shared memory by store_tile), read once, stored to every peer two at a time:
    // each 8-byte half carries its own stamp, so the 16-byte store need not land as one
    for (int i = tid_in_group; i < per_peer; i += group_threads) {
        const int k2 = i & (ppt - 1), m = i / ppt;
        const uint2 v = reinterpret_cast<const uint2*>(ytile + m * (16 * esz))[k2];
        const size_t off = ((size_t)p.sp.me * p.M + m) * wpr + rt * (2 * ppt) + 2 * k2;
        for (int q = 0; q < p.sp.world; q++)
            if (q != p.sp.me)
                st_relaxed_sys64x2(reinterpret_cast<unsigned long long*>(static_cast<char*>(p.sp.y[q]) + p.sp.inbox_off) + off,
                                   stamp | v.x, stamp | v.y);
    }
}
// This CTA's share of the inbox -> local y.  Returns false if a word did not arrive in time.
// A thread takes pairs of words, four pairs requested at once (a poll is an L2 round trip: one after the
// other they would add up to microseconds); whatever has not arrived yet is polled again.
__device__ __forceinline__ bool unpack_inbox(const Params& p, uint32_t epoch) {
    constexpr int U = 4;
    const int esz = p.y_bf16 ? 2 : 4;
    const int ppr = p.N * esz / 8;  // pairs per row of a rank's columns
    const int total = (p.sp.world - 1) * p.M * ppr;
    const int per_cta = (total + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per_cta, hi = min(total, lo + per_cta);
    char* ylocal = static_cast<char*>(p.sp.y[p.sp.me]);
    const unsigned long long* inbox = reinterpret_cast<const unsigned long long*>(ylocal + p.sp.inbox_off);
    int i = lo + (int)threadIdx.x;
    if (i >= hi) return true;
    // position of pair i: sender (skipping this rank), row, pair in the row; advanced without divisions
    int w = i % ppr, m = (i / ppr) % p.M, s = i / (ppr * p.M);
    bool ok = true;
    while (i < hi && ok) {
        const unsigned long long* slot[U];
        uint2* dst[U];
        unsigned long long v0[U], v1[U];
        int n = 0;
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (i < hi) {
                const int src = s + (s >= p.sp.me);
                slot[u] = inbox + (((size_t)src * p.M + m) * ppr + w) * 2;
                dst[u] = reinterpret_cast<uint2*>(ylocal + ((size_t)m * p.ld + (size_t)src * p.N) * esz + (size_t)w * 8);
                ld_relaxed_sys64x2(slot[u], v0[u], v1[u]);
                n = u + 1;
                i += kThreads;
                w += kThreads;
                while (w >= ppr) {
                    w -= ppr;
                    if (++m == p.M) {
                        m = 0;
                        s++;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (u < n) {
                if ((uint32_t)(v0[u] >> 32) != epoch || (uint32_t)(v1[u] >> 32) != epoch) {
                    const long long t0 = now_ns();
                    for (;;) {
                        ld_relaxed_sys64x2(slot[u], v0[u], v1[u]);
                        if ((uint32_t)(v0[u] >> 32) == epoch && (uint32_t)(v1[u] >> 32) == epoch) break;
                        if (peer_lost() || now_ns() - t0 > p.peer_wait_ns) {
                            g_peer_lost = 1;
                            ok = false;
                            break;
                        }
                    }
                }
                if (ok) *dst[u] = make_uint2((uint32_t)v0[u], (uint32_t)v1[u]);
            }
        }
    }
    return ok;
}

// ytile (column-sharded launches only): the tile's values once more in shared memory, [row of x][16 columns]
// (32 bytes per row of x for bf16, 64 for fp32; 16 rows per tile), from where they are sent to the peers
// without a trip through L2.
template <int MT>
__device__ __forceinline__ void store_tile(const Params& p, int rt, int e, float sum, unsigned char* ytile) {
    const int mt = e >> 7, rem = e & 127, ln = rem >> 2, ci = rem & 3;
    const int r16 = (ln >> 2) + 8 * (ci >> 1);
    const int row = rt * 16 + r16;
    const int m = mt * 8 + 2 * (ln & 3) + (ci & 1);
    if (row < p.N && m < p.M) {
        const size_t idx = (size_t)m * p.ld + p.col0 + row;
        if (p.y_bf16) {
            const __nv_bfloat16 v = __float2bfloat16_rn(sum);
            reinterpret_cast<__nv_bfloat16*>(p.y)[idx] = v;
            if (ytile) reinterpret_cast<__nv_bfloat16*>(ytile + m * 32)[r16] = v;
        } else {
            reinterpret_cast<float*>(p.y)[idx] = sum;
            if (ytile) reinterpret_cast<float*>(ytile + m * 64)[r16] = sum;
        }
    }
}

// Sum n partials (stride floats apart) in order; loads are issued eight at a
// time so their latencies overlap, the additions stay in order.
template <bool GLOBAL>
__device__ __forceinline__ float ordered_sum(const float* src, int n, int stride, float sum) {
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = GLOBAL ? __ldcg(src + (size_t)(i + u) * stride) : src[(i + u) * stride];
#pragma unroll
        for (int u = 0; u < 8; u++) sum += v[u];
    }
    for (; i < n; i++) sum += GLOBAL ? __ldcg(src + (size_t)i * stride) : src[i * stride];
    return sum;
}

// End of a batch of row tiles (all threads call it): sum the per-k-block
// partials of every tile in k-block order and write y.  With K split over
// several CTAs the partials go through the tile's scratch slot and the tile
// is finished by whichever CTA arrives last.
template <int MT>
__device__ __noinline__ void batch_end(const Params& p, const float* part, int first_tile, int ntiles, int kb_lo, int nkl,
                                       int* flags, bool more, bool peers_ready, uint32_t epoch, unsigned char* ytiles) {
    constexpr int E = 128 * MT;  // fp32 elements per partial
    const int tid = threadIdx.x;
    __syncthreads();
    if (p.ks == 1) {
        for (int ti = tid / E; ti < ntiles; ti += kThreads / E)
            store_tile<MT>(p, first_tile + ti, tid % E, ordered_sum<false>(part + ti * nkl * E + tid % E, nkl, E, 0.0f),
                           ytiles ? ytiles + ti * (p.y_bf16 ? 512 : 1024) : nullptr);
    } else {
        for (int ti = 0; ti < ntiles; ti++) {
            float* dst = p.scratch + ((size_t)(first_tile + ti) * p.nkb + kb_lo) * E;
            const float* src = part + ti * nkl * E;
            for (int i = tid; i < nkl * E; i += kThreads) __stcg(dst + i, src[i]);
        }
        __syncthreads();
        if (tid < ntiles) {
            __threadfence();  // cumulative: publishes the CTA's partials (ordered before by the barrier)
            const unsigned int old = atomicAdd(p.counters + first_tile + tid, (unsigned int)nkl);
            const int last = (old + (unsigned int)nkl == (unsigned int)p.nkb);
            if (last) {
                p.counters[first_tile + tid] = 0;  // every contributor has arrived: leave the counter clean
                __threadfence();
            }
            flags[tid] = last;
        }
        __syncthreads();
        for (int ti = tid / E; ti < ntiles; ti += kThreads / E)
            if (flags[ti])
                store_tile<MT>(p, first_tile + ti, tid % E,
                               ordered_sum<true>(p.scratch + (size_t)(first_tile + ti) * p.nkb * E + tid % E, p.nkb, E, 0.0f),
                               ytiles ? ytiles + ti * (p.y_bf16 ? 512 : 1024) : nullptr);
    }
    if (p.sp.world > 1) {
        // the tiles this CTA has just finished go to the peers (unless the hand-shake failed)
        __syncthreads();
        if (peers_ready) {
            constexpr int kGroup = 128;
            for (int ti = tid / kGroup; ti < ntiles; ti += kThreads / kGroup)
                if (p.ks == 1 || flags[ti]) push_tile(p, epoch, first_tile + ti, ytiles + ti * (p.y_bf16 ? 512 : 1024), tid % kGroup, kGroup);
        }
    }
    if (more) __syncthreads();  // the partial buffer and the flags are reused by the next batch
}

// With 16 rows of x the fragments of rows 8..15 live in shared memory (one conflict-free 16-byte read per
// use) instead of 32 more registers per lane: at the 128-register limit the kernel otherwise spills.
constexpr bool kX1Shared = true;

// One task out of the warp's ring stage: 4 x 16 bytes of packed weights per
// lane (rows g, g+8; pieces t, t+4), their scales/biases, times the x fragments.
// stage layout: [piece = r*2+h][lane] 16 B  |  [row 0..15 scales][row 0..15 biases] 16 B each
template <int BITS, int MT, bool FAST>
__device__ __forceinline__ void task_mma(const uint4 (&w)[2][2], const uint32_t (&s)[2][2], const uint32_t (&b)[2][2],
                                         const uint4 (&xr)[MT][BITS == 4 ? 8 : 4], const uint4* xs, float (&acc)[MT][2][4]) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint32_t sa[2], sb[2], b2[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            b2[r] = dup_bf16(b[r][h]);
            sa[r] = FAST ? scale_x2_133(s[r][h]) : dup_bf16(s[r][h]);
            sb[r] = FAST ? scale_x2_129(s[r][h]) : 0u;
        }
        const uint32_t w0[4] = {w[0][h].x, w[0][h].y, w[0][h].z, w[0][h].w};
        const uint32_t w1[4] = {w[1][h].x, w[1][h].y, w[1][h].z, w[1][h].w};
        if (BITS == 4) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo[4], hi[4];
                if (FAST) {
                    dequant4_fast(w0[i], sa[0], sb[0], b2[0], lo);
                    dequant4_fast(w1[i], sa[1], sb[1], b2[1], hi);
                } else {
                    dequant4_general(w0[i], sa[0], b2[0], lo);
                    dequant4_general(w1[i], sa[1], b2[1], hi);
                }
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 bx = (mt == 0 || !kX1Shared) ? xr[mt][h * 4 + i] : xs[(h * 4 + i) * 32];
                    mma_bf16(acc[mt][0], lo[0], hi[0], lo[1], hi[1], bx.x, bx.y);
                    mma_bf16(acc[mt][1], lo[2], hi[2], lo[3], hi[3], bx.z, bx.w);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                uint32_t lo0[2], hi0[2], lo1[2], hi1[2];
                if (FAST) {
                    dequant8_fast(w0[2 * i], sa[0], b2[0], lo0);
                    dequant8_fast(w1[2 * i], sa[1], b2[1], hi0);
                    dequant8_fast(w0[2 * i + 1], sa[0], b2[0], lo1);
                    dequant8_fast(w1[2 * i + 1], sa[1], b2[1], hi1);
                } else {
                    dequant8_general(w0[2 * i], sa[0], b2[0], lo0);
                    dequant8_general(w1[2 * i], sa[1], b2[1], hi0);
                    dequant8_general(w0[2 * i + 1], sa[0], b2[0], lo1);
                    dequant8_general(w1[2 * i + 1], sa[1], b2[1], hi1);
                }
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 bx = (mt == 0 || !kX1Shared) ? xr[mt][h * 2 + i] : xs[(h * 2 + i) * 32];
                    mma_bf16(acc[mt][0], lo0[0], hi0[0], lo0[1], hi0[1], bx.x, bx.y);
                    mma_bf16(acc[mt][1], lo1[0], hi1[0], lo1[1], hi1[1], bx.z, bx.w);
                }
            }
        }
    }
}

// x fragments of k-block kb for lane (g, t), in the order the unpack yields the weights.
//   4-bit: fragment j = h*4+i covers k = kb*256 + h*128 + t*32 + i*8 + (0,4,1,5 | 2,6,3,7)
//   8-bit: fragment j = h*2+i covers k = kb*128 + h*64  + t*16 + i*8 + (0,2,1,3 | 4,6,5,7)
// PRO: what x is -- 0: the buffer as it is; 1: its rms-norm, row by row (the caller scales the fragments, see
// rms_scale); 2: bf16(a + b + c) of the three column blocks [0,K), [K,2K), [2K,3K) of a wider row (fp32 adds,
// left to right, one rounding: the bits of the stand-alone sum3 kernel).
__device__ __forceinline__ uint32_t add3_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    const float lo = __fadd_rn(__fadd_rn(__uint_as_float(a << 16), __uint_as_float(b << 16)), __uint_as_float(c << 16));
    const float hi = __fadd_rn(__fadd_rn(__uint_as_float(a & 0xFFFF0000u), __uint_as_float(b & 0xFFFF0000u)), __uint_as_float(c & 0xFFFF0000u));
    const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint4 ldg_nc_v4(const uint4* src) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src));
    return v;
}
template <int BITS, int MT, int PRO>
__device__ __forceinline__ void load_x_raw(const Params& p, int kb, int g, int t, uint4 (&xr)[MT][BITS == 4 ? 8 : 4]) {
    constexpr int XV = BITS == 4 ? 8 : 4;
    constexpr int KB = 1024 / BITS;
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const int m = mt * 8 + g;
        const __nv_bfloat16* row = p.x + (size_t)m * (PRO == 0 ? p.K : p.x_ld) + kb * KB + t * (KB / 8);
#pragma unroll
        for (int j = 0; j < XV; j++) {
            const int h = j / (XV / 2), i = j % (XV / 2);
            xr[mt][j] = make_uint4(0, 0, 0, 0);
            if (m < p.M) {
                const uint4* src = reinterpret_cast<const uint4*>(row + h * (KB / 2) + i * 8);
                if (PRO == 2) {
                    const uint4 a = ldg_nc_v4(src), b = ldg_nc_v4(reinterpret_cast<const uint4*>(row + p.K + h * (KB / 2) + i * 8)),
                                c = ldg_nc_v4(reinterpret_cast<const uint4*>(row + 2 * p.K + h * (KB / 2) + i * 8));
                    xr[mt][j] = make_uint4(add3_bf16x2(a.x, b.x, c.x), add3_bf16x2(a.y, b.y, c.y), add3_bf16x2(a.z, b.z, c.z),
                                           add3_bf16x2(a.w, b.w, c.w));
                } else {
                    xr[mt][j] = ldg_nc_v4(src);
                }
            }
        }
    }
}
// rms-norm prologue: the sum of squares of this lane's fragments (fp32), and the fragments scaled and rounded
// as the stand-alone rms-norm kernel does it: bf16(fl32(x * inv)).
template <int XV>
__device__ __forceinline__ float sumsq_frags(const uint4 (&xr)[XV]) {
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < XV; j++) {
        const uint32_t w[4] = {xr[j].x, xr[j].y, xr[j].z, xr[j].w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xFFFF0000u);
            ss = fmaf(lo, lo, ss);
            ss = fmaf(hi, hi, ss);
        }
    }
    return ss;
}
__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t v, float inv) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(__fmul_rn(__uint_as_float(v << 16), inv), __fmul_rn(__uint_as_float(v & 0xFFFF0000u), inv));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <int XV>
__device__ __forceinline__ void rms_scale(uint4 (&xr)[XV], float inv) {
#pragma unroll
    for (int j = 0; j < XV; j++)
        xr[j] = make_uint4(scale_bf16x2(xr[j].x, inv), scale_bf16x2(xr[j].y, inv), scale_bf16x2(xr[j].z, inv), scale_bf16x2(xr[j].w, inv));
}
template <int BITS, int MT>
__device__ __forceinline__ void permute_x(uint4 (&xr)[MT][BITS == 4 ? 8 : 4]) {
    constexpr int XV = BITS == 4 ? 8 : 4;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int j = 0; j < XV; j++) {
            const uint4 v = xr[mt][j];
            if (BITS == 4) {
                xr[mt][j].x = prmt(v.x, v.z, 0x5410u);  // x0, x4
                xr[mt][j].y = prmt(v.x, v.z, 0x7632u);  // x1, x5
                xr[mt][j].z = prmt(v.y, v.w, 0x5410u);  // x2, x6
                xr[mt][j].w = prmt(v.y, v.w, 0x7632u);  // x3, x7
            } else {
                xr[mt][j].x = prmt(v.x, v.y, 0x5410u);  // x0, x2
                xr[mt][j].y = prmt(v.x, v.y, 0x7632u);  // x1, x3
                xr[mt][j].z = prmt(v.z, v.w, 0x5410u);  // x4, x6
                xr[mt][j].w = prmt(v.z, v.w, 0x7632u);  // x5, x7
            }
        }
}

// all four scales (raw bf16 bits) usable by the exponent-trick dequantiser?  Packed form of
// scale_fast_ok: exponent field e in [1, 121]  <=>  ((s - 0x80) & 0x7F80) <= 0x3C00 per half.
__device__ __forceinline__ bool scales_fast_ok4(uint32_t s00, uint32_t s01, uint32_t s10, uint32_t s11) {
    const uint32_t a = (((s00 | (s10 << 16)) - 0x00800080u) & 0x7F807F80u) + 0x43804380u;
    const uint32_t b = (((s01 | (s11 << 16)) - 0x00800080u) & 0x7F807F80u) + 0x43804380u;
    return ((a | b) & 0x80008000u) == 0u;
}

// BITS: 4 | 8.  MT: number of 8-row blocks of x (M <= 8*MT).  PRO: prologue applied to x as it is loaded (load_x_raw;
// MT == 1 only).
template <int BITS, int MT, int PRO>
__global__ void __launch_bounds__(kThreads, 1) qmv_mma_kernel(const __grid_constant__ Params p) {
    static_assert(PRO == 0 || MT == 1, "prologues are built for M <= 8");
    constexpr int XV = BITS == 4 ? 8 : 4;  // x fragments (uint4) per lane per k-block per 8-row block
    constexpr int KB = 1024 / BITS;        // weights per k-block (128 bytes per row)
    constexpr int E4 = MT * 32;            // float4 per partial
    constexpr int D = ring_depth(MT);      // ring stages of a warp
    extern __shared__ __align__(16) unsigned char smem[];
    float4* part = reinterpret_cast<float4*>(smem + ring_bytes(MT));   // [tb][nkl][MT][32]; ring: [kWarps][D][kStageBytes]
    // after the partials (MT == 2): the x fragments of rows 8..15, [warp][fragment][lane]
    uint4* xs = reinterpret_cast<uint4*>(smem + p.xs_off) + (threadIdx.x >> 5) * (XV * 32) + (threadIdx.x & 31);
    __shared__ int s_flags[kMaxTb];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ci = blockIdx.x % p.chunks, ksi = blockIdx.x / p.chunks;
    const int rt_lo = (int)((long long)p.n_rt * ci / p.chunks), rt_hi = (int)((long long)p.n_rt * (ci + 1) / p.chunks);
    const int kb_lo = (int)((long long)p.nkb * ksi / p.ks), kb_hi = (int)((long long)p.nkb * (ksi + 1) / p.ks);
    const int nkl = kb_hi - kb_lo;
    const int tb = p.tb;
    const size_t row_bytes = (size_t)p.K * BITS / 8;
    const int gpr = p.K >> p.gshift;   // groups per row
    const int gpk = KB >> p.gshift;    // groups per k-block
    const unsigned char* wbase = reinterpret_cast<const unsigned char*>(p.wq) + t * 16;
    const __nv_bfloat16* sb_src = lane < 16 ? p.scales : p.biases;
    const uint32_t ring_lo = smem_u32(smem) + warp * (D * kStageBytes) + lane * 16;  // this lane's slot, stage 0
    const int tail_tile = (p.N & 15) ? p.n_rt - 1 : -1;  // the tile whose rows must be clamped to N-1
    const bool has_work = kb_lo + warp < kb_hi && rt_lo < rt_hi;

    // The warp's tasks, in order: for each batch of tb tiles, for each of its k-blocks, the tiles of the
    // batch ("run": they share the x fragments of that k-block).  D-1 tasks are in flight while one is
    // computed; the fetch runs that far ahead of the computation, one commit group per task (empty past the end).
    const size_t half_tile = 8 * row_bytes, tile_stride = 16 * row_bytes;
    int f_b0 = rt_lo, f_kb = kb_lo + warp, f_rt = rt_lo;  // the task fetched next
    uint32_t f_dst = ring_lo;                             // and the stage it goes to
    // this lane's sources of that task: rows g and g+8 of the tile (its 16-byte pieces t and t+4 of the k-block),
    // the scales (lanes 0-15) or biases (16-31) of row lane%16.  Inside a run they move by constant strides.
    const unsigned char* f_p0 = nullptr;
    const unsigned char* f_p1 = nullptr;
    const __nv_bfloat16* f_sb = nullptr;
    auto fetch_point = [&]() {
        if (f_rt != tail_tile) {
            f_p0 = wbase + (size_t)(f_rt * 16 + g) * row_bytes + f_kb * 128;
            f_p1 = f_p0 + half_tile;
            f_sb = sb_src + ((f_rt * 16 + (lane & 15)) * gpr + f_kb * gpk);
        } else {  // rows past N read row N-1 (their results are never stored)
            const int n0 = f_rt * 16;
            f_p0 = wbase + (size_t)min(n0 + g, p.N - 1) * row_bytes + f_kb * 128;
            f_p1 = wbase + (size_t)min(n0 + g + 8, p.N - 1) * row_bytes + f_kb * 128;
            f_sb = sb_src + (min(n0 + (lane & 15), p.N - 1) * gpr + f_kb * gpk);
        }
    };
    if (has_work) fetch_point();
    auto fetch_next = [&]() {
        if (has_work && f_b0 < rt_hi) {
            cp_async16(f_dst, f_p0);
            cp_async16(f_dst + 512, f_p0 + 64);
            cp_async16(f_dst + 1024, f_p1);
            cp_async16(f_dst + 1536, f_p1 + 64);
            if (p.sb_bytes == 16) cp_async16(f_dst + 2048, f_sb);
            else if (p.sb_bytes == 8) cp_async8(f_dst + 2048, f_sb);
            else cp_async4(f_dst + 2048, reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(f_sb) & ~uintptr_t(3)));  // a lone scale travels with its neighbour
            // on to the task after it
            f_dst = f_dst + kStageBytes == ring_lo + D * kStageBytes ? ring_lo : f_dst + kStageBytes;
            if (++f_rt == min(f_b0 + tb, rt_hi)) {  // next run: next k-block of the batch, else first k-block of the next batch
                f_kb += kWarps;
                if (f_kb >= kb_hi) {
                    f_kb = kb_lo + warp;
                    f_b0 += tb;
                }
                f_rt = f_b0;
                if (f_b0 < rt_hi) fetch_point();
            } else if (f_rt == tail_tile) {
                fetch_point();
            } else {
                f_p0 += tile_stride;
                f_p1 += tile_stride;
                f_sb += 16 * gpr;
            }
        }
        cp_async_commit();
    };

    // The x fragments of the first k-block are on the critical path of the first task, and a load queues
    // behind whatever the SM has already requested.  When the host knows that the previous kernel of the
    // stream does not write x (or there is none to wait for), they are requested first of all, ahead of the
    // weights; otherwise right after the wait.  (With 16 rows the fragments would have to be held across the
    // fetch code and spill; they stay behind it.)
    constexpr bool kXFirst = MT == 1;
    uint4 xr[MT][XV];
    if (kXFirst && p.x_early && has_work) load_x_raw<BITS, MT, PRO>(p, kb_lo + warp, g, t, xr);
#pragma unroll
    for (int i = 0; i < D - 1; i++) fetch_next();

    // Everything above touched only the weights (and, if the host allowed it, x), which no kernel of the chain
    // writes.  From here on the kernel reads x and uses the scratch, which the previous kernel may have
    // written: wait for it, then let the next kernel of the chain start its own weight fetch.  (Both are
    // no-ops in a plain launch.)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // column-sharded: this call's number, and the word to the peers that our copy of y may be overwritten
    uint32_t epoch = 0;
    bool peers_ready = true, ready_checked = p.sp.world <= 1;
    uint32_t ready_early = 0;  // a peer's ready word as read in mid-kernel (its latency hidden behind the tasks)
    if (p.sp.world > 1) {
        epoch = *reinterpret_cast<volatile uint32_t*>(p.sp.flags[p.sp.me] + kFlagEpoch) + 1;
        // (a relaxed store: it publishes no data of this kernel, only that the kernel has started)
        if (blockIdx.x == 0 && tid < p.sp.world && tid != p.sp.me) st_relaxed_sys(p.sp.flags[tid] + kFlagReady + p.sp.me, epoch);
    }
    if (kXFirst && !p.x_early && has_work) load_x_raw<BITS, MT, PRO>(p, kb_lo + warp, g, t, xr);
    bool x_loaded = kXFirst;  // (of the first run)
    // rms-norm prologue.  The host launches it only when every warp has at most one k-block and K is not split:
    // the fragments just loaded by the 16 warps are then the whole of x, each lane holding 1/4 of a k-block of
    // row g.  Sum of squares per row: the four lanes of a row in the warp, then the warps in order through shared
    // memory; every lane ends up with the factor of its row.
    float rms_inv = 1.0f;
    if (PRO == 1) {
        __shared__ float s_rms[kWarps][8];
        if (!has_work) {
#pragma unroll
            for (int j = 0; j < XV; j++) xr[0][j] = make_uint4(0, 0, 0, 0);
        }
        float ss = sumsq_frags<XV>(xr[0]);
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (t == 0) s_rms[warp][g] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) tot += s_rms[w][g];
        rms_inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps)));
        rms_scale<XV>(xr[0], rms_inv);
    }

    uint32_t src_c = ring_lo;  // stage of the task computed next (this lane's slot)
    uint32_t sboff[2][2];      // byte offsets of this lane's scales inside a stage, by row half r and piece h
#pragma unroll 1
    for (int b0 = rt_lo; b0 < rt_hi; b0 += tb) {
        const int nt = min(tb, rt_hi - b0);
        if (has_work) {
#pragma unroll 1
            for (int kb = kb_lo + warp; kb < kb_hi; kb += kWarps) {
                fetch_next();  // (the run's first fetch goes out ahead of the x loads)
                if (!x_loaded) {
                    load_x_raw<BITS, MT, PRO>(p, kb, g, t, xr);
                    if (PRO == 1) rms_scale<XV>(xr[0], rms_inv);
                }
                x_loaded = false;
                permute_x<BITS, MT>(xr);
                if (MT == 2 && kX1Shared) {
                    __syncwarp();  // (the previous run's reads of xs)
#pragma unroll
                    for (int j = 0; j < XV; j++) xs[j * 32] = xr[MT - 1][j];
                    __syncwarp();
                }
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int slot = g + 8 * r;
                    const int par = p.sb_bytes == 2 ? ((slot * gpr + kb) & 1) : 0;
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        sboff[r][h] = 2048 - lane * 16 + slot * 16 + ((((h * (KB / 2) + t * (KB / 8)) >> p.gshift) + par) << 1);
                }
                if (p.sp.world > 1 && tid < p.sp.world && tid != p.sp.me)
                    ready_early = ld_relaxed_sys(p.sp.flags[p.sp.me] + kFlagReady + tid);  // used at the first push
                float4* dstp = part + (kb - kb_lo) * E4 + lane;
#pragma unroll 1
                for (int rt = b0; rt < b0 + nt; rt++) {
                    if (rt != b0) fetch_next();
                    cp_async_wait<D - 1>();
                    __syncwarp();
                    uint4 w[2][2];
                    uint32_t s[2][2], b[2][2];
#pragma unroll
                    for (int r = 0; r < 2; r++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(w[r][h].x), "=r"(w[r][h].y), "=r"(w[r][h].z), "=r"(w[r][h].w)
                                         : "r"(src_c + (r * 2 + h) * 512));
                            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(s[r][h]) : "r"(src_c + sboff[r][h]));
                            asm volatile("ld.shared.u16 %0, [%1+256];" : "=r"(b[r][h]) : "r"(src_c + sboff[r][h]));
                        }
                    const bool fast = scales_fast_ok4(s[0][0], s[0][1], s[1][0], s[1][1]);
                    float acc[MT][2][4];  // two independent accumulation chains per 8-row block of x
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
#pragma unroll
                        for (int c = 0; c < 2; c++) acc[mt][c][0] = acc[mt][c][1] = acc[mt][c][2] = acc[mt][c][3] = 0.0f;
                    if (__all_sync(0xffffffffu, fast)) task_mma<BITS, MT, true>(w, s, b, xr, xs, acc);
                    else task_mma<BITS, MT, false>(w, s, b, xr, xs, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
                        dstp[mt * 32] = make_float4(acc[mt][0][0] + acc[mt][1][0], acc[mt][0][1] + acc[mt][1][1],
                                                    acc[mt][0][2] + acc[mt][1][2], acc[mt][0][3] + acc[mt][1][3]);
                    dstp += nkl * E4;
                    __syncwarp();  // every lane is done with the stage before it is refilled
                    src_c = src_c + kStageBytes == ring_lo + D * kStageBytes ? ring_lo : src_c + kStageBytes;
                }
            }
        }
        if (!ready_checked) {  // before the first remote store: has every peer started this call?
            ready_checked = true;
            int ok = 1;
            if (tid < p.sp.world && tid != p.sp.me)
                ok = (int32_t)(ready_early - epoch) >= 0 || wait_flag(p.sp.flags[p.sp.me] + kFlagReady + tid, epoch, p.peer_wait_ns);
            peers_ready = __syncthreads_and(ok);
        }
        // End of the batch: sum the per-k-block partials of every tile in k-block order and write y.  The
        // common case stays in line (reads of the parameter block from a function out of line are slow).
        if (p.ks == 1 && p.sp.world <= 1) {
            constexpr int E = 128 * MT;
            __syncthreads();
            for (int ti = tid / E; ti < nt; ti += kThreads / E)
                store_tile<MT>(p, b0 + ti, tid % E,
                               ordered_sum<false>(reinterpret_cast<const float*>(part) + ti * nkl * E + tid % E, nkl, E, 0.0f), nullptr);
            if (b0 + tb < rt_hi) __syncthreads();  // the partial buffer is reused by the next batch
        } else {
            batch_end<MT>(p, reinterpret_cast<const float*>(part), b0, nt, kb_lo, nkl, s_flags, b0 + tb < rt_hi, peers_ready, epoch,
                          p.yt_off ? smem + p.yt_off : nullptr);
        }
    }
    cp_async_wait<0>();
    if (p.sp.world > 1) {
        // the peers' columns: this CTA's share of the inbox goes into the local y; the launch ends when all
        // shares are in.  The last CTA to finish moves the call number on.
        const bool ok = peers_ready && unpack_inbox(p, epoch);
        if (!__syncthreads_and(ok) && tid == 0 && p.error) *p.error = 2;
        if (tid == 0) {
            uint32_t* lf = p.sp.flags[p.sp.me];
            // (a plain count: the next launch reads the call number only after this one has completed)
            if (atomicAdd(lf + kFlagCtaDone, 1u) == gridDim.x - 1) {
                lf[kFlagCtaDone] = 0;
                *reinterpret_cast<volatile uint32_t*>(lf + kFlagEpoch) = epoch;
            }
        }
    }
}

// ---- several matmuls of one shape per launch ------------------------------------------------------------
constexpr int kMaxBatch = 48;
struct BatchItem {
    const __nv_bfloat16* x;
    const uint32_t* wq;
    const __nv_bfloat16* scales;
    const __nv_bfloat16* biases;
    void* y;
    int M;
    uint32_t yoff;  // column-sharded: byte offset of this y inside every rank's symmetric buffer
};
struct BatchParams {
    int n_items;
    int K, N, gshift, y_bf16;
    int nkb, n_rt, chunks, tb, sb_bytes, xs_off;
    BatchItem items[kMaxBatch];
    // column-sharded launches only (SH): N is this rank's share of the columns
    int ld, col0, yt_off;
    int* error;
    long long peer_wait_ns;
    ShardPush sp;
};
template <int BITS, int MT>
__device__ __forceinline__ void load_x_item(const __nv_bfloat16* x, int M, int K, int kb, int g, int t, uint4 (&xr)[MT][BITS == 4 ? 8 : 4]) {
    constexpr int XV = BITS == 4 ? 8 : 4;
    constexpr int KB = 1024 / BITS;
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const int m = mt * 8 + g;
        const __nv_bfloat16* row = x + (size_t)m * K + kb * KB + t * (KB / 8);
#pragma unroll
        for (int j = 0; j < XV; j++) {
            const int h = j / (XV / 2), i = j % (XV / 2);
            xr[mt][j] = make_uint4(0, 0, 0, 0);
            if (m < M) xr[mt][j] = ldg_nc_v4(reinterpret_cast<const uint4*>(row + h * (KB / 2) + i * 8));
        }
    }
}
// ytile (column-sharded launches): the tile's values once more in shared memory, [row of x][16 columns]
template <int MT>
__device__ __forceinline__ void store_tile_item(void* y, int M, int N, int ld, int col0, int y_bf16, int rt, int e, float sum,
                                                unsigned char* ytile) {
    const int mt = e >> 7, rem = e & 127, ln = rem >> 2, ci = rem & 3;
    const int r16 = (ln >> 2) + 8 * (ci >> 1);
    const int row = rt * 16 + r16;
    const int m = mt * 8 + 2 * (ln & 3) + (ci & 1);
    if (row < N && m < M) {
        const size_t idx = (size_t)m * ld + col0 + row;
        if (y_bf16) {
            const __nv_bfloat16 v = __float2bfloat16_rn(sum);
            reinterpret_cast<__nv_bfloat16*>(y)[idx] = v;
            if (ytile) reinterpret_cast<__nv_bfloat16*>(ytile + m * 32)[r16] = v;
        } else {
            reinterpret_cast<float*>(y)[idx] = sum;
            if (ytile) reinterpret_cast<float*>(ytile + m * 64)[r16] = sum;
        }
    }
}

// Several decode matmuls of one shape (K, N, bits, group; M <= 8*MT each) in ONE launch: qmv_mma_kernel's roles and
// arithmetic with a loop over the matmuls around them.  A CTA keeps its range of row tiles through all of them and
// its warps' rings never drain in between: the fetch iterator walks from the last task of one matmul into the
// first of the next, so the start of a launch (first reads of parameters, x and weights) and its tail (the
// ordered sum and the store of y), which are half of a single decode launch, are paid once per launch instead of
// once per matmul -- the sum and the store of a matmul run while the next one's weights are already arriving.
// No K split, no prologue (the host sends such calls one by one).
//
// SH: the layer is column-sharded over ranks and every y lives at the same offset of every rank's symmetric buffer.
// The finished tiles of a matmul (staged in shared memory as they are stored locally) go straight into the peers'
// copies of y, 16 bytes a store, while the warps are already in the next matmul.  The hand-shakes are paid once
// per launch instead of once per matmul: ready[q] as in qmv_mma_kernel (before the first remote store: has every
// peer started this call, i.e. is it done with its y of earlier calls?), and at the end done[q] = call number,
// written by a rank's last CTA to finish -- behind a system-wide fence, every CTA having fenced its own stores
// before it counted itself in -- into every peer's flag words; that CTA then waits (bounded) for the peers' done
// words, so that the launch ends with y whole on this rank and stream order is all a consumer needs.
//
// DEEP (M <= 8, at most 8 bytes of scales per row and k-block): five ring stages per warp instead of four, in stages
// of 2304 bytes (the scales and biases of a row in 8-byte slots instead of 16-byte ones).  Every matmul ends with
// the block meeting twice around the sum and the store; meanwhile the rings stand full and nothing new is requested.
// With four tasks in flight per warp instead of three, a matmul's four or five tasks per warp are (nearly) all on
// their way before the previous matmul's end, so the memory system keeps working through it.
constexpr int kDeepDepth = 5, kDeepStageBytes = 2048 + 256;
template <int BITS, int MT, bool SH, bool DEEP>
__global__ void __launch_bounds__(kThreads, 1) qmv_batch_kernel(const __grid_constant__ BatchParams p) {
    constexpr int XV = BITS == 4 ? 8 : 4;  // x fragments (uint4) per lane per k-block per 8-row block
    constexpr int KB = 1024 / BITS;        // weights per k-block (128 bytes per row)
    constexpr int E4 = MT * 32;            // float4 per partial
    static_assert(!DEEP || MT == 1, "the deep ring is for up to 8 rows of x");
    constexpr int D = DEEP ? kDeepDepth : ring_depth(MT);       // ring stages of a warp
    constexpr int kStageBytes = DEEP ? kDeepStageBytes : luxcuda::kStageBytes;
    constexpr int kSlot = DEEP ? 8 : 16;                         // bytes of a row's scales (and of its biases) in a stage
    extern __shared__ __align__(16) unsigned char smem[];
    float4* part = reinterpret_cast<float4*>(smem + kWarps * D * kStageBytes);   // [tb][nkl][MT][32]; ring: [kWarps][D][kStageBytes]
    // after the partials (MT == 2): the x fragments of rows 8..15, [warp][fragment][lane]
    uint4* xs = reinterpret_cast<uint4*>(smem + p.xs_off) + (threadIdx.x >> 5) * (XV * 32) + (threadIdx.x & 31);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ci = blockIdx.x;
    // The row tiles are dealt out in p.chunks ranges of floor or ceil(n_rt / chunks) tiles, range c = [n_rt*c/chunks,
    // n_rt*(c+1)/chunks).  This CTA takes range (blockIdx.x + i) mod chunks of matmul i: nothing synchronises the CTAs
    // between matmuls, so what counts is a CTA's total over the launch, and rotating the ranges evens out the one
    // tile by which they differ (4 or 5 tiles at 688 tiles on 148 SMs: 7 % between the longest and the average).
    // A range follows from the one before by additions (q, rem = n_rt / chunks, n_rt % chunks; acc = rem*(c+1) mod chunks).
    const int rt_q = p.n_rt / p.chunks, rt_rem = p.n_rt % p.chunks;
    auto next_range = [&](int& c, int& lo, int& hi, int& acc) {
        if (++c == p.chunks) {
            c = 0;
            lo = 0;
            hi = rt_q;
            acc = rt_rem;
        } else {
            lo = hi;
            acc += rt_rem;
            const int e = acc >= p.chunks ? 1 : 0;
            acc -= e ? p.chunks : 0;
            hi = lo + rt_q + e;
        }
    };
    int rt_c = ci, rt_lo = (int)((long long)p.n_rt * ci / p.chunks), rt_hi = (int)((long long)p.n_rt * (ci + 1) / p.chunks);
    int rt_acc = (int)(((long long)rt_rem * (ci + 1)) % p.chunks);
    int f_c = rt_c, f_lo = rt_lo, f_hi = rt_hi, f_acc = rt_acc;  // the same for the matmul whose weights are being fetched
    const int kb_lo = 0, kb_hi = p.nkb;
    const int nkl = kb_hi - kb_lo;
    const int tb = p.tb;
    const size_t row_bytes = (size_t)p.K * BITS / 8;
    const int gpr = p.K >> p.gshift;   // groups per row
    const int gpk = KB >> p.gshift;    // groups per k-block
    // the matmul whose weights are being fetched (f_pi) runs ahead of the one being computed (pi)
    int f_pi = 0;
    const unsigned char* wbase = reinterpret_cast<const unsigned char*>(p.items[0].wq) + t * 16;
    const __nv_bfloat16* sb_src = lane < 16 ? p.items[0].scales : p.items[0].biases;
    const uint32_t ring_lo = smem_u32(smem) + warp * (D * kStageBytes) + lane * 16;  // this lane's slot, stage 0
    const int tail_tile = (p.N & 15) ? p.n_rt - 1 : -1;  // the tile whose rows must be clamped to N-1
    const bool has_work = kb_lo + warp < kb_hi && rt_lo < rt_hi;

    // The warp's tasks, in order: for each batch of tb tiles, for each of its k-blocks, the tiles of the
    // batch ("run": they share the x fragments of that k-block).  D-1 tasks are in flight while one is
    // computed; the fetch runs that far ahead of the computation, one commit group per task (empty past the end).
    const size_t half_tile = 8 * row_bytes, tile_stride = 16 * row_bytes;
    int f_b0 = rt_lo, f_kb = kb_lo + warp, f_rt = rt_lo;  // the task fetched next
    uint32_t f_dst = ring_lo;                             // and the stage it goes to
    // this lane's sources of that task: rows g and g+8 of the tile (its 16-byte pieces t and t+4 of the k-block),
    // the scales (lanes 0-15) or biases (16-31) of row lane%16.  Inside a run they move by constant strides.
    const unsigned char* f_p0 = nullptr;
    const unsigned char* f_p1 = nullptr;
    const __nv_bfloat16* f_sb = nullptr;
    auto fetch_point = [&]() {
        if (f_rt != tail_tile) {
            f_p0 = wbase + (size_t)(f_rt * 16 + g) * row_bytes + f_kb * 128;
            f_p1 = f_p0 + half_tile;
            f_sb = sb_src + ((f_rt * 16 + (lane & 15)) * gpr + f_kb * gpk);
        } else {  // rows past N read row N-1 (their results are never stored)
            const int n0 = f_rt * 16;
            f_p0 = wbase + (size_t)min(n0 + g, p.N - 1) * row_bytes + f_kb * 128;
            f_p1 = wbase + (size_t)min(n0 + g + 8, p.N - 1) * row_bytes + f_kb * 128;
            f_sb = sb_src + (min(n0 + (lane & 15), p.N - 1) * gpr + f_kb * gpk);
        }
    };
    if (has_work) fetch_point();
    auto fetch_next = [&]() {
        if (has_work && f_pi < p.n_items) {
            cp_async16(f_dst, f_p0);
            cp_async16(f_dst + 512, f_p0 + 64);
            cp_async16(f_dst + 1024, f_p1);
            cp_async16(f_dst + 1536, f_p1 + 64);
            const uint32_t sb_dst = f_dst + 2048 - lane * (16 - kSlot);  // (f_dst is this lane's 16-byte slot of the stage)
            if (!DEEP && p.sb_bytes == 16) cp_async16(sb_dst, f_sb);
            else if (p.sb_bytes == 8) cp_async8(sb_dst, f_sb);
            else cp_async4(sb_dst, reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(f_sb) & ~uintptr_t(3)));  // a lone scale travels with its neighbour
            // on to the task after it
            f_dst = f_dst + kStageBytes == ring_lo + D * kStageBytes ? ring_lo : f_dst + kStageBytes;
            if (++f_rt == min(f_b0 + tb, f_hi)) {  // next run: next k-block of the batch, else first k-block of the next batch
                f_kb += kWarps;
                if (f_kb >= kb_hi) {
                    f_kb = kb_lo + warp;
                    f_b0 += tb;
                }
                if (f_b0 >= f_hi && ++f_pi < p.n_items) {  // on to the next matmul: the next range of tiles, its weights
                    next_range(f_c, f_lo, f_hi, f_acc);
                    f_b0 = f_lo;
                    wbase = reinterpret_cast<const unsigned char*>(p.items[f_pi].wq) + t * 16;
                    sb_src = lane < 16 ? p.items[f_pi].scales : p.items[f_pi].biases;
                }
                f_rt = f_b0;
                if (f_pi < p.n_items) fetch_point();
            } else if (f_rt == tail_tile) {
                fetch_point();
            } else {
                f_p0 += tile_stride;
                f_p1 += tile_stride;
                f_sb += 16 * gpr;
            }
        }
        cp_async_commit();
    };

    uint4 xr[MT][XV];
    bool x_ahead = false;  // xr already holds the fragments of the run about to start
#pragma unroll
    for (int i = 0; i < D - 1; i++) fetch_next();
    // column-sharded: this call's number, and the word to the peers that our copies of y may be overwritten
    // (the launch is an ordinary one: whatever this rank enqueued before has finished with them)
    uint32_t epoch = 0;
    bool peers_ready = true, ready_checked = !SH;
    if (SH) {
        epoch = *reinterpret_cast<volatile uint32_t*>(p.sp.flags[p.sp.me] + kFlagEpoch) + 1;
        if (blockIdx.x == 0 && tid < p.sp.world && tid != p.sp.me) st_relaxed_sys(p.sp.flags[tid] + kFlagReady + p.sp.me, epoch);
    }
    unsigned char* const ytiles = SH ? smem + p.yt_off : nullptr;
    const int yt_bytes = p.y_bf16 ? 512 : 1024;  // of a staged tile
    uint32_t src_c = ring_lo;  // stage of the task computed next (this lane's slot)
    uint32_t sboff[2][2];      // byte offsets of this lane's scales inside a stage, by row half r and piece h
#pragma unroll 1
    for (int pi = 0; pi < p.n_items; pi++) {
    if (pi) next_range(rt_c, rt_lo, rt_hi, rt_acc);
    const __nv_bfloat16* x_cur = p.items[pi].x;
    void* y_cur = p.items[pi].y;
    const int M_cur = p.items[pi].M;
#pragma unroll 1
    for (int b0 = rt_lo; b0 < rt_hi; b0 += tb) {
        const int nt = min(tb, rt_hi - b0);
        if (has_work) {
#pragma unroll 1
            for (int kb = kb_lo + warp; kb < kb_hi; kb += kWarps) {
                fetch_next();  // (the run's first fetch goes out ahead of the x loads)
                if (!x_ahead) load_x_item<BITS, MT>(x_cur, M_cur, p.K, kb, g, t, xr);
                x_ahead = false;
                permute_x<BITS, MT>(xr);
                if (MT == 2 && kX1Shared) {
                    __syncwarp();  // (the previous run's reads of xs)
#pragma unroll
                    for (int j = 0; j < XV; j++) xs[j * 32] = xr[MT - 1][j];
                    __syncwarp();
                }
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int slot = g + 8 * r;
                    const int par = p.sb_bytes == 2 ? ((slot * gpr + kb) & 1) : 0;
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        sboff[r][h] = 2048 - lane * 16 + slot * kSlot + ((((h * (KB / 2) + t * (KB / 8)) >> p.gshift) + par) << 1);
                }
                float4* dstp = part + (kb - kb_lo) * E4 + lane;
#pragma unroll 1
                for (int rt = b0; rt < b0 + nt; rt++) {
                    if (rt != b0) fetch_next();
                    cp_async_wait<D - 1>();
                    __syncwarp();
                    uint4 w[2][2];
                    uint32_t s[2][2], b[2][2];
#pragma unroll
                    for (int r = 0; r < 2; r++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(w[r][h].x), "=r"(w[r][h].y), "=r"(w[r][h].z), "=r"(w[r][h].w)
                                         : "r"(src_c + (r * 2 + h) * 512));
                            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(s[r][h]) : "r"(src_c + sboff[r][h]));
                            asm volatile("ld.shared.u16 %0, [%1+%2];" : "=r"(b[r][h]) : "r"(src_c + sboff[r][h]), "n"(16 * kSlot));
                        }
                    const bool fast = scales_fast_ok4(s[0][0], s[0][1], s[1][0], s[1][1]);
                    float acc[MT][2][4];  // two independent accumulation chains per 8-row block of x
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
#pragma unroll
                        for (int c = 0; c < 2; c++) acc[mt][c][0] = acc[mt][c][1] = acc[mt][c][2] = acc[mt][c][3] = 0.0f;
                    if (__all_sync(0xffffffffu, fast)) task_mma<BITS, MT, true>(w, s, b, xr, xs, acc);
                    else task_mma<BITS, MT, false>(w, s, b, xr, xs, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
                        dstp[mt * 32] = make_float4(acc[mt][0][0] + acc[mt][1][0], acc[mt][0][1] + acc[mt][1][1],
                                                    acc[mt][0][2] + acc[mt][1][2], acc[mt][0][3] + acc[mt][1][3]);
                    dstp += nkl * E4;
                    __syncwarp();  // every lane is done with the stage before it is refilled
                    src_c = src_c + kStageBytes == ring_lo + D * kStageBytes ? ring_lo : src_c + kStageBytes;
                }
            }
        }
        // When a matmul is one run of one batch for this warp (K of at most 16 k-blocks, the CTA's tiles in one
        // batch), the x fragments of the NEXT matmul are requested here, before the block meets: their latency is
        // spent in the sum and the store below instead of in front of the next matmul's first task.
        // (With 16 rows of x the fragments held across the block barrier spill: measured 16.5 against 11.2 us.)
        if (MT == 1 && has_work && kb_hi - kb_lo <= kWarps && rt_hi - rt_lo <= tb && pi + 1 < p.n_items) {
            load_x_item<BITS, MT>(p.items[pi + 1].x, p.items[pi + 1].M, p.K, kb_lo + warp, g, t, xr);
            x_ahead = true;
        }
        if (SH && !ready_checked) {  // before the first remote store: has every peer started this call?
            ready_checked = true;
            int ok = 1;
            if (tid < p.sp.world && tid != p.sp.me) ok = wait_flag(p.sp.flags[p.sp.me] + kFlagReady + tid, epoch, p.peer_wait_ns);
            peers_ready = __syncthreads_and(ok);
            if (!peers_ready && tid == 0 && p.error) *p.error = 2;  // nothing is sent; the host learns of it at its next sync
        }
        // End of the batch: sum the per-k-block partials of every tile in k-block order and write y.
        {
            constexpr int E = 128 * MT;
            __syncthreads();
            for (int ti = tid / E; ti < nt; ti += kThreads / E)
                store_tile_item<MT>(y_cur, M_cur, p.N, SH ? p.ld : p.N, SH ? p.col0 : 0, p.y_bf16, b0 + ti, tid % E,
                                    ordered_sum<false>(reinterpret_cast<const float*>(part) + ti * nkl * E + tid % E, nkl, E, 0.0f),
                                    SH ? ytiles + ti * yt_bytes : nullptr);
            __syncthreads();  // the partial buffer is reused by the next batch (of this matmul or the next)
        }
        if (SH && peers_ready) {
            // The staged tiles go to the peers, a 16-byte piece of a row per store.  (The staging area is written
            // again only behind the first barrier of the next batch end, which a thread reaches after these reads.)
            const int esz = p.y_bf16 ? 2 : 4;            // also the number of 16-byte pieces of a tile row
            const int per_tile = M_cur * esz, per_peer = nt * per_tile;
            const int total = per_peer * (p.sp.world - 1);
            const uint32_t yoff = p.items[pi].yoff;
            for (int i = tid; i < total; i += kThreads) {
                int q = i / per_peer;
                const int j = i - q * per_peer;
                q += q >= p.sp.me;
                const int ti = j / per_tile, r = j - ti * per_tile, m = r / esz, k = r - m * esz;
                const uint4 v = *reinterpret_cast<const uint4*>(ytiles + ti * yt_bytes + m * (16 * esz) + k * 16);
                char* dst = static_cast<char*>(p.sp.y[q]) + yoff + ((size_t)m * p.ld + p.col0 + (size_t)(b0 + ti) * 16) * esz + k * 16;
                *reinterpret_cast<uint4*>(dst) = v;
            }
        }
    }
    }
    cp_async_wait<0>();
    if (SH) {
        __syncthreads();  // every remote store of this CTA has been issued
        if (tid == 0) {
            __threadfence_system();  // ... and is ordered before the count below, for every observer
            uint32_t* lf = p.sp.flags[p.sp.me];
            if (atomicAdd(lf + kFlagCtaDone, 1u) == gridDim.x - 1) {  // the last CTA of this rank
                lf[kFlagCtaDone] = 0;
                bool ok = peers_ready;
                if (ok) {
                    __threadfence_system();
                    for (int q = 0; q < p.sp.world; q++)
                        if (q != p.sp.me) st_relaxed_sys(p.sp.flags[q] + kFlagDone + p.sp.me, epoch);
                    for (int q = 0; q < p.sp.world; q++)
                        if (q != p.sp.me) ok = wait_flag(lf + kFlagDone + q, epoch, p.peer_wait_ns) && ok;
                    __threadfence_system();
                }
                if (!ok && p.error) *p.error = 2;
                // (a plain store: the next launch reads the call number only after this one has completed)
                *reinterpret_cast<volatile uint32_t*>(lf + kFlagEpoch) = epoch;
            }
        }
    }
}

struct Plan {
    int nkb, n_rt, mt, chunks, ks, tb, gshift, sb_bytes, xs_off, yt_off;
    size_t smem, scratch_bytes;
};

// Arrival counters of k-split tiles live at the head of the workspace in a region of fixed size, so that
// launches of different shapes that share a workspace agree on where the counters end and the partials begin.
constexpr size_t kCounterBytes = 4096;
constexpr int kMaxSplitTiles = (int)(kCounterBytes / sizeof(unsigned int));

// ring_override: bytes of the warps' rings when the kernel is not the standard one (the batched kernel's deep ring)
bool make_plan(const QmmArgs& a, int sm_count, Plan* pl, bool sharded = false, size_t ring_override = 0) {
    if (a.x_dtype != LUX_DTYPE_BFLOAT16 || a.sb_dtype != LUX_DTYPE_BFLOAT16) return false;
    if (a.bits != 4 && a.bits != 8) return false;
    if (a.M < 1 || a.M > 16 || a.N < 1 || sm_count < 1) return false;
    const int KB = 1024 / a.bits;
    if (a.K % KB) return false;
    if (a.group != 32 && a.group != 64 && a.group != 128) return false;
    pl->gshift = a.group == 32 ? 5 : (a.group == 64 ? 6 : 7);
    const int gpk = KB >> pl->gshift, gpr = a.K >> pl->gshift;
    if (gpk < 1) return false;
    pl->sb_bytes = gpk * 2;
    if (pl->sb_bytes == 2 && (((long long)a.N * gpr) & 1)) return false;  // pairs of scales are copied
    pl->mt = a.M <= 8 ? 1 : 2;
    pl->nkb = a.K / KB;
    pl->n_rt = (a.N + 15) / 16;
    // 32-bit row/group indices and per-matrix byte offsets inside the kernel
    if ((long long)a.N * gpr > (1ll << 30) || (long long)pl->n_rt * pl->nkb > (1ll << 30)) return false;
    // K is split over several CTAs only when the tiles alone cannot fill the GPU and a
    // CTA's 16 warps would each still own more than one k-block
    int ks = 1;
    if (pl->n_rt * 2 <= sm_count) ks = std::max(1, std::min((pl->nkb + kWarps - 1) / kWarps, sm_count / pl->n_rt));
    if (const char* env = getenv("LUXCUDA_QMV_KSPLIT"))
        if (pl->n_rt <= kMaxSplitTiles) ks = std::max(1, std::min(atoi(env), pl->nkb));
    if (pl->n_rt > kMaxSplitTiles) ks = 1;
    pl->ks = ks;
    pl->chunks = std::max(1, std::min(pl->n_rt, sm_count / ks));
    const int tiles_max = (pl->n_rt + pl->chunks - 1) / pl->chunks;
    const int nkl_max = (pl->nkb + ks - 1) / ks;
    const size_t per_tile = (size_t)nkl_max * pl->mt * 512;
    const size_t xs_bytes = pl->mt == 2 ? (size_t)kWarps * (a.bits == 4 ? 8 : 4) * 512 : 0;  // x fragments of rows 8..15
    const size_t ring = ring_override ? ring_override : (size_t)ring_bytes(pl->mt);
    const size_t avail = (size_t)kSmemLimit - ring - xs_bytes;
    // column-sharded launches stage every finished tile once more (16 rows of x x 16 columns) for the peers
    const size_t yt_tile = sharded ? (a.y_dtype == LUX_DTYPE_BFLOAT16 ? 512 : 1024) : 0;
    if (per_tile + yt_tile > avail) return false;
    pl->tb = (int)std::min<size_t>(std::min<size_t>(tiles_max, avail / (per_tile + yt_tile)), kMaxTb);
    pl->xs_off = (int)(ring + pl->tb * per_tile);
    pl->yt_off = sharded ? (int)(pl->xs_off + xs_bytes) : 0;
    pl->smem = ring + pl->tb * per_tile + xs_bytes + (sharded ? pl->tb * yt_tile : 0);
    pl->scratch_bytes = ks > 1 ? (size_t)pl->n_rt * pl->nkb * pl->mt * 128 * sizeof(float) : 0;
    if (((uintptr_t)a.wq & 15) || ((uintptr_t)a.x & 15) || ((uintptr_t)a.scales & 15) || ((uintptr_t)a.biases & 15)) return false;
    return true;
}

template <int BITS, int MT, int PRO>
cudaError_t launch_t(const Params& p, const Plan& pl, cudaStream_t stream, bool overlap_prev) {
    auto kern = qmv_mma_kernel<BITS, MT, PRO>;
    // opt in to large dynamic shared memory (static + dynamic stay within the 227 KiB per-block limit)
    static std::atomic<size_t> attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_smem[dev & 63].load() < pl.smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev & 63].store(pl.smem);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.chunks * pl.ks);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    // As a programmatic dependent the grid may start (and fetch weights) while the previous kernel of the
    // stream drains; everything else in the kernel sits behind its griddepcontrol.wait.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_prev ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

// Clears, on the current device, the mark that a wait for a peer has run out (after which no launch waits for
// peers any more).
cudaError_t reset_peer_lost() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_peer_lost, &zero, sizeof(zero));
}

// Limit of a device-side wait for a peer rank, from LUXCUDA_PEER_WAIT_MS (default 2000 ms).
long long peer_wait_limit_ns() {
    static const long long ns = [] {
        const char* env = getenv("LUXCUDA_PEER_WAIT_MS");
        const long long ms = env ? atoll(env) : 2000;
        return (ms < 1 ? 1 : ms) * 1000000ll;
    }();
    return ns;
}

bool qmv_mma_supported(const QmmArgs& a, int sm_count) {
    Plan pl;
    return make_plan(a, sm_count, &pl);
}

// Scratch memory (global memory beyond inputs and outputs): arrival counters
// (always present, zero between launches) and, when K is split, the partials.
size_t qmv_mma_workspace_bytes(const QmmArgs& a, int sm_count) {
    Plan pl;
    if (!make_plan(a, sm_count, &pl)) return 0;
    return kCounterBytes + pl.scratch_bytes;
}

// workspace layout: [counters: kCounterBytes][partials]; the counters must be zero before the
// first launch and are left zero by every launch.
cudaError_t launch_qmv_mma(const QmmArgs& a, void* workspace, int sm_count, cudaStream_t stream, const char** name,
                           bool overlap_prev, const ShardPush* push, bool x_stable) {
    Plan pl;
    if (!make_plan(a, sm_count, &pl, push && push->world > 1)) return cudaErrorInvalidValue;
    Params p;
    p.x = (const __nv_bfloat16*)a.x;
    p.wq = a.wq;
    p.scales = (const __nv_bfloat16*)a.scales;
    p.biases = (const __nv_bfloat16*)a.biases;
    p.y = a.y;
    p.counters = (unsigned int*)workspace;
    p.scratch = (float*)((unsigned char*)workspace + kCounterBytes);
    p.M = a.M; p.K = a.K; p.N = a.N;
    p.gshift = pl.gshift;
    p.y_bf16 = a.y_dtype == LUX_DTYPE_BFLOAT16;
    p.nkb = pl.nkb; p.n_rt = pl.n_rt;
    p.chunks = pl.chunks; p.ks = pl.ks; p.tb = pl.tb; p.sb_bytes = pl.sb_bytes;
    p.chained = overlap_prev ? 1 : 0;
    p.xs_off = pl.xs_off;
    p.yt_off = pl.yt_off;
    p.ld = a.N; p.col0 = 0;
    p.x_early = (!overlap_prev || x_stable) ? 1 : 0;
    p.x_ld = a.pro ? a.x_ld : a.K;
    p.eps = a.eps;
    if (a.pro) {
        // prologues: M <= 8; the rms-norm needs the whole of x in the first fragments of the CTA's warps
        if (pl.mt != 1 || a.pro < 0 || a.pro > 2 || (a.pro == 1 && (pl.ks != 1 || pl.nkb > kWarps))) return cudaErrorNotSupported;
        if ((a.x_ld & 7) || a.x_ld < (a.pro == 2 ? 3 * a.K : a.K)) return cudaErrorInvalidValue;
    }
    p.error = nullptr;
    p.peer_wait_ns = peer_wait_limit_ns();
    if (push && push->world > 1) {
        if (push->world > kMaxShardWorld || (a.N & 15)) return cudaErrorInvalidValue;  // whole 16-column tiles only
        p.sp = *push;
        p.ld = push->ld; p.col0 = push->col0;
        p.error = a.error ? a.error : device_error_word();
        if (!p.error) return cudaErrorMemoryAllocation;
    }
    if (a.bits == 4) {
        if (name) *name = pl.mt == 2 ? "qmv_mma<4,m16>" : a.pro == 1 ? "qmv_mma<4,m8,rms>" : a.pro == 2 ? "qmv_mma<4,m8,sum3>" : "qmv_mma<4,m8>";
        if (pl.mt == 2) return launch_t<4, 2, 0>(p, pl, stream, overlap_prev);
        return a.pro == 1 ? launch_t<4, 1, 1>(p, pl, stream, overlap_prev)
             : a.pro == 2 ? launch_t<4, 1, 2>(p, pl, stream, overlap_prev) : launch_t<4, 1, 0>(p, pl, stream, overlap_prev);
    }
    if (name) *name = pl.mt == 2 ? "qmv_mma<8,m16>" : a.pro == 1 ? "qmv_mma<8,m8,rms>" : a.pro == 2 ? "qmv_mma<8,m8,sum3>" : "qmv_mma<8,m8>";
    if (pl.mt == 2) return launch_t<8, 2, 0>(p, pl, stream, overlap_prev);
    return a.pro == 1 ? launch_t<8, 1, 1>(p, pl, stream, overlap_prev)
         : a.pro == 2 ? launch_t<8, 1, 2>(p, pl, stream, overlap_prev) : launch_t<8, 1, 0>(p, pl, stream, overlap_prev);
}


// Several matmuls of one shape in one launch (qmv_batch_kernel).  All items: the shape of items[0] but for M, with
// M on the same side of 8; bf16; no K split for that shape.  cudaErrorNotSupported otherwise.
template <int BITS, int MT, bool SH, bool DEEP>
cudaError_t launch_batch_t(const BatchParams& p, const Plan& pl, cudaStream_t stream) {
    auto kern = qmv_batch_kernel<BITS, MT, SH, DEEP>;
    static std::atomic<size_t> attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_smem[dev & 63].load() < pl.smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
        if (e != cudaSuccess) return e;
        attr_smem[dev & 63].store(pl.smem);
    }
    kern<<<pl.chunks, kThreads, pl.smem, stream>>>(p);
    return cudaGetLastError();
}
int qmv_batch_max() { return kMaxBatch; }
cudaError_t launch_qmv_batch(const QmmArgs* items, int n, int sm_count, cudaStream_t stream, const char** name,
                             const ShardPush* push) {
    if (n < 1 || n > kMaxBatch) return cudaErrorInvalidValue;
    const bool sh = push && push->world > 1;
    Plan pl;
    QmmArgs a0 = items[0];
    int mmax = 0;
    for (int i = 0; i < n; i++) mmax = std::max(mmax, items[i].M);
    a0.M = mmax;
    if (!make_plan(a0, sm_count, &pl, sh) || pl.ks != 1) return cudaErrorNotSupported;
    // The deep ring (see the kernel) when a CTA's tiles of a matmul still fit into one batch beside it
    bool deep = false;
    if (pl.mt == 1 && pl.sb_bytes <= 8 && !getenv("LUXCUDA_QMV_BATCH_NO_DEEP")) {
        Plan dp;
        if (make_plan(a0, sm_count, &dp, sh, (size_t)kWarps * kDeepDepth * kDeepStageBytes) && dp.ks == 1 && dp.tb >= pl.tb) {
            pl = dp;
            deep = true;
        }
    }
    BatchParams p;
    p.ld = a0.N; p.col0 = 0; p.yt_off = pl.yt_off;
    p.error = nullptr;
    p.peer_wait_ns = peer_wait_limit_ns();
    if (sh) {
        if (push->world > kMaxShardWorld || (a0.N & 15)) return cudaErrorInvalidValue;  // whole 16-column tiles only
        p.sp = *push;
        p.ld = push->ld; p.col0 = push->col0;
        p.error = a0.error ? a0.error : device_error_word();
        if (!p.error) return cudaErrorMemoryAllocation;
    }
    p.n_items = n;
    p.K = a0.K; p.N = a0.N; p.gshift = pl.gshift;
    p.y_bf16 = a0.y_dtype == LUX_DTYPE_BFLOAT16;
    p.nkb = pl.nkb; p.n_rt = pl.n_rt; p.chunks = pl.chunks; p.tb = pl.tb; p.sb_bytes = pl.sb_bytes; p.xs_off = pl.xs_off;
    for (int i = 0; i < n; i++) {
        const QmmArgs& a = items[i];
        if (a.K != a0.K || a.N != a0.N || a.bits != a0.bits || a.group != a0.group || a.y_dtype != a0.y_dtype ||
            a.x_dtype != LUX_DTYPE_BFLOAT16 || a.sb_dtype != LUX_DTYPE_BFLOAT16 || a.M < 1 || (a.M <= 8) != (mmax <= 8) || a.pro)
            return cudaErrorNotSupported;
        if (((uintptr_t)a.wq | (uintptr_t)a.x | (uintptr_t)a.scales | (uintptr_t)a.biases) & 15) return cudaErrorInvalidValue;
        uint32_t yoff = 0;
        if (sh) {  // the item's y lies inside this rank's symmetric buffer: the peers' copies are at the same offset
            const ptrdiff_t d = static_cast<const char*>(a.y) - static_cast<const char*>(push->y[push->me]);
            if (d < 0 || d > (ptrdiff_t)0xFFFFFFF0ll || (d & 15)) return cudaErrorInvalidValue;
            yoff = (uint32_t)d;
        }
        p.items[i] = BatchItem{(const __nv_bfloat16*)a.x, a.wq, (const __nv_bfloat16*)a.scales, (const __nv_bfloat16*)a.biases, a.y, a.M, yoff};
    }
    if (a0.bits == 4) {
        if (name) *name = sh ? (pl.mt == 1 ? "qmv_batch<4,m8,push>" : "qmv_batch<4,m16,push>") : (pl.mt == 1 ? "qmv_batch<4,m8>" : "qmv_batch<4,m16>");
        if (deep) return sh ? launch_batch_t<4, 1, true, true>(p, pl, stream) : launch_batch_t<4, 1, false, true>(p, pl, stream);
        if (sh) return pl.mt == 1 ? launch_batch_t<4, 1, true, false>(p, pl, stream) : launch_batch_t<4, 2, true, false>(p, pl, stream);
        return pl.mt == 1 ? launch_batch_t<4, 1, false, false>(p, pl, stream) : launch_batch_t<4, 2, false, false>(p, pl, stream);
    }
    if (name) *name = sh ? (pl.mt == 1 ? "qmv_batch<8,m8,push>" : "qmv_batch<8,m16,push>") : (pl.mt == 1 ? "qmv_batch<8,m8>" : "qmv_batch<8,m16>");
    if (deep) return sh ? launch_batch_t<8, 1, true, true>(p, pl, stream) : launch_batch_t<8, 1, false, true>(p, pl, stream);
    if (sh) return pl.mt == 1 ? launch_batch_t<8, 1, true, false>(p, pl, stream) : launch_batch_t<8, 2, true, false>(p, pl, stream);
    return pl.mt == 1 ? launch_batch_t<8, 1, false, false>(p, pl, stream) : launch_batch_t<8, 2, false, false>(p, pl, stream);
}

// ---------------------------------------------------------------------------------
// Decode GEMV without any allocation: the scratch lives in the library image.
// ---------------------------------------------------------------------------------
namespace {
// Arrival counters + k-split partials of the decode kernel, 4 MiB per GPU that loads the
// library (held until the process exits).  Zero at load; every launch leaves the counters zero.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mu;
void* g_static_ptr[64];  // device address of g_static_scratch, per device ordinal

// The array's name is only a host-side handle: the address a kernel may use has to be asked
// for, once per device, with that device current.
cudaError_t static_scratch_ptr(int device, void** out) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_ptr[device] = p;
    }
    *out = g_static_ptr[device];
    return cudaSuccess;
}
}  // namespace
}  // namespace luxcuda

extern "C" LUX_GPU_BACKEND_EXPORT LuxBackendError lux_gpu_cuda_qmatmul_decode_noalloc(
    LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* wq, LuxBackendBuffer* scales, LuxBackendBuffer* biases,
    LuxBackendBuffer* y, int M, int K, int N, int bits, int group, LuxBackendDtype y_dtype) {
    using namespace luxcuda;
    Context* c = as_ctx(ctx);
    Buffer *bx = as_buf(x), *bw = as_buf(wq), *bs = as_buf(scales), *bb = as_buf(biases), *by = as_buf(y);
    if (!c || !bx || !bw || !bs || !bb || !by) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (y_dtype != LUX_DTYPE_BFLOAT16 && y_dtype != LUX_DTYPE_FLOAT32) return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    if (M < 1 || M > 16 || K < 1 || N < 1 || (bits != 4 && bits != 8) || (group != 32 && group != 64 && group != 128) || K % group) {
        set_last_error("qmatmul_decode_noalloc: needs 1 <= M <= 16, bits 4|8, group 32|64|128, K a multiple of group");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    const size_t ys = y_dtype == LUX_DTYPE_BFLOAT16 ? 2 : 4;
    if ((size_t)M * K * 2 > bx->bytes || (size_t)N * K * bits / 8 > bw->bytes || (size_t)N * (K / group) * 2 > bs->bytes ||
        (size_t)N * (K / group) * 2 > bb->bytes || (size_t)M * N * ys > by->bytes) {
        set_last_error("qmatmul_decode_noalloc: a buffer is smaller than its shape needs");
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    QmmArgs a{bx->ptr, (const uint32_t*)bw->ptr, bs->ptr, bb->ptr, by->ptr, M, K, N, bits, group,
              LUX_DTYPE_BFLOAT16, LUX_DTYPE_BFLOAT16, (int)y_dtype};
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->dev->device());
    const size_t need = qmv_mma_workspace_bytes(a, c->dev->sm_count);
    if (need == 0) {
        set_last_error("qmatmul_decode_noalloc: shape not taken by the decode kernel (K must be a multiple of %d)", 1024 / bits);
        return LUX_BACKEND_ERROR_NOT_SUPPORTED;
    }
    if (need > kStaticScratchBytes) {
        set_last_error("qmatmul_decode_noalloc: this shape needs %zu bytes of scratch, the built-in scratch holds %zu",
                       need, kStaticScratchBytes);
        return LUX_BACKEND_ERROR_INVALID_ARGUMENT;
    }
    void* scratch = nullptr;
    cudaError_t e = static_scratch_ptr(c->dev->device(), &scratch);
    if (e != cudaSuccess) return map_cuda_error(e, "cudaGetSymbolAddress(static scratch)");
    const char* name = "";
    e = launch_qmv_mma(a, scratch, c->dev->sm_count, c->stream, &name, decode_may_overlap(c, a), nullptr, decode_x_stable(c, a));
    if (e != cudaSuccess) return map_cuda_error(e, name);
    c->last_kernel = name;
    c->launches++;
    note_decode_launch(c, a);
    bx->last_stream = bw->last_stream = bs->last_stream = bb->last_stream = by->last_stream = c->stream;
    return LUX_BACKEND_OK;
}
