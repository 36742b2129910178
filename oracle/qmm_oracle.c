/*
 * CPU oracle for affine group-wise quantized matmul (4-bit / 8-bit).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing on the product path (the CUDA plugin, its
 * host code, the Python mirror of the plugin interface) may call into this
 * file.  It is the checker for the parity tests and the timed CPU baseline.
 *
 * PARITY UNPINNED: the reference tree (luxfi/mlx "Lux GPU Core") contains no
 * quantized matmul, no pack/unpack routine and no golden vector for one.  The
 * packed format and the rounding rules below are therefore this repository's
 * own specification.  What IS anchored on the reference:
 *   - buffer conventions (row-major, contiguous), argument order
 *     (ctx-less here: in..., out, dims...) and the loop nest of the matmul:
 *     `#pragma omp parallel for collapse(2)` over (i, j) with a sequential
 *     fp32 k-sum and no FMA contraction -- src/cpu_backend.cpp:243-266;
 *   - rms-norm formula y = x / sqrt(mean(x^2) + eps) * w --
 *     kernels/cpu/tensor_ops.c:546-566;
 *   - dtype enum values (FLOAT32 = 0, BFLOAT16 = 2, UINT32 = 5) --
 *     include/lux/gpu/backend_plugin.h:38-47.
 *   tests/test_oracle.py checks that orc_qmatmul_ref() on a
 *   layer equals, bit for bit, the reference's own cpu_op_matmul_f32 applied
 *   to the dequantised dense weights.
 *
 * Format specification
 *   Wq      uint32[N][K*bits/32]        packed along K, least-significant first
 *             4-bit: q[n][k] = (Wq[n][k>>3] >> (4*(k&7))) & 0xF
 *             8-bit: q[n][k] = (Wq[n][k>>2] >> (8*(k&3))) & 0xFF
 *   scales  [N][K/group], biases [N][K/group]   (fp32 or bf16)
 *   w^[n][k] = scales[n][k/group] * q[n][k] + biases[n][k/group]
 *   y[m][n]  = sum_k x[m][k] * w^[n][k]           (y = x . W^T)
 *
 * Rounding specification ("compute dtype" = dtype of x)
 *   x fp32 : w^ = fl32(fl32(s*q) + b)  (two roundings, no FMA); scales/biases
 *            given as bf16 are widened to fp32 first (exact).
 *   x bf16 : scales/biases must be bf16; w^ = the single correctly rounded
 *            (round-to-nearest-even) bf16 of the exact real s*q + b, i.e. what
 *            one bf16 fused multiply-add returns.
 *   accumulate fp32 (order free on the GPU => compared by tolerance);
 *   output fp32, or bf16 by round-to-nearest-even of the fp32 sum.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_F32 0
#define ORC_BF16 2

/* ------------------------------------------------------------------ */
/* bf16 helpers                                                        */
/* ------------------------------------------------------------------ */
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

uint16_t orc_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* Round the exact real number (t + e), |e| <= ulp(t)/2, to fp32 with
 * round-to-odd; a following RNE to bf16 is then the correctly rounded bf16 of
 * the real number (24 >= 8 + 2 bits). */
static float round_odd_f32(double t, double e) {
    float f = (float)t;
    double d = (double)f;
    if (d == t && e == 0.0) return f;
    uint32_t u = f32_bits(f);
    if (u & 1u) return f;
    int above = (t > d) || (t == d && e > 0.0); /* real value above f */
    if ((u & 0x7FFFFFFFu) == 0) { /* f is +-0: smallest subnormal toward the value */
        return bits_f32(above ? 1u : 0x80000001u);
    }
    int neg = (u >> 31) & 1;
    if (above != neg) u += 1; else u -= 1; /* step one ulp toward the real value */
    return bits_f32(u);
}

/* canonical bf16 dequantised weight: RNE_bf16(exact s*q + b) */
static inline uint16_t dq_bf16(uint16_t s16, uint16_t b16, uint32_t q) {
    double s = (double)orc_bf16_to_f32(s16), b = (double)orc_bf16_to_f32(b16);
    double p = s * (double)q;            /* 8-bit x 8-bit significands: exact */
    double t = p + b;
    double bb = t - p;                   /* TwoSum residual (exact) */
    double e = (p - (t - bb)) + (b - bb);
    return orc_f32_to_bf16(round_odd_f32(t, e));
}
/* canonical fp32 dequantised weight: fl(fl(s*q) + b) */
static inline float dq_f32(float s, float b, uint32_t q) {
    float p = s * (float)q;              /* built with -ffp-contract=off: never an FMA */
    return p + b;
}

static inline uint32_t unpack1(const uint32_t* row, int64_t k, int bits) {
    return bits == 4 ? (row[k >> 3] >> (4 * (k & 7))) & 0xFu
                     : (row[k >> 2] >> (8 * (k & 3))) & 0xFFu;
}
static inline float load_sb(const void* p, int64_t i, int dtype) {
    return dtype == ORC_BF16 ? orc_bf16_to_f32(((const uint16_t*)p)[i]) : ((const float*)p)[i];
}

/* ------------------------------------------------------------------ */
/* Counter-based RNG (SplitMix64 finaliser over seed + counter)         */
/* ------------------------------------------------------------------ */
static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline uint64_t rng_u64(uint64_t seed, uint64_t ctr) {
    return mix64(seed + (ctr + 1) * 0x9E3779B97F4A7C15ull);
}
static inline double rng_unit(uint64_t seed, uint64_t ctr) { /* (0,1) */
    return ((double)(rng_u64(seed, ctr) >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}
uint64_t orc_seed(uint64_t base, uint64_t a, uint64_t b, uint64_t c, uint64_t d) {
    uint64_t h = mix64(base ^ 0xA0761D6478BD642Full);
    h = mix64(h ^ (a + 0x9E3779B97F4A7C15ull));
    h = mix64(h ^ (b + 0xE7037ED1A0B428DBull));
    h = mix64(h ^ (c + 0x8EBC6AF09C88C6E3ull));
    h = mix64(h ^ (d + 0x589965CC75374CC3ull));
    return h;
}

/* q ~ U{0..2^bits-1}, packed */
void orc_gen_q(uint64_t seed, uint32_t* wq, int64_t N, int64_t K, int bits) {
    int64_t words = N * (K * bits / 32);
    int per = 32 / bits;
#pragma omp parallel for
    for (int64_t w = 0; w < words; w++) {
        uint32_t word = 0;
        for (int j = 0; j < per; j++) {
            uint32_t q = (uint32_t)(rng_u64(seed, (uint64_t)w * per + j) >> 40) & ((1u << bits) - 1);
            word |= q << (bits * j);
        }
        wq[w] = word;
    }
}
void orc_gen_uniform_f32(uint64_t seed, float* out, int64_t n, double lo, double hi) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; i++) out[i] = (float)(lo + (hi - lo) * rng_unit(seed, (uint64_t)i));
}
void orc_gen_normal_f32(uint64_t seed, float* out, int64_t n, double mean, double std) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; i++) {
        double u1 = rng_unit(seed, 2 * (uint64_t)i), u2 = rng_unit(seed, 2 * (uint64_t)i + 1);
        out[i] = (float)(mean + std * sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
    }
}
void orc_round_bf16(const float* in, uint16_t* out, int64_t n) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; i++) out[i] = orc_f32_to_bf16(in[i]);
}
void orc_widen_bf16(const uint16_t* in, float* out, int64_t n) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; i++) out[i] = orc_bf16_to_f32(in[i]);
}

/* ------------------------------------------------------------------ */
/* pack / unpack / dequantise                                           */
/* ------------------------------------------------------------------ */
void orc_unpack(const uint32_t* wq, uint8_t* q, int64_t N, int64_t K, int bits) {
    int64_t wpr = K * bits / 32;
#pragma omp parallel for
    for (int64_t n = 0; n < N; n++)
        for (int64_t k = 0; k < K; k++) q[n * K + k] = (uint8_t)unpack1(wq + n * wpr, k, bits);
}
void orc_pack(const uint8_t* q, uint32_t* wq, int64_t N, int64_t K, int bits) {
    int64_t wpr = K * bits / 32;
    int per = 32 / bits;
#pragma omp parallel for
    for (int64_t n = 0; n < N; n++)
        for (int64_t w = 0; w < wpr; w++) {
            uint32_t word = 0;
            for (int j = 0; j < per; j++)
                word |= ((uint32_t)q[n * K + w * per + j] & ((1u << bits) - 1)) << (bits * j);
            wq[n * wpr + w] = word;
        }
}
/* out_dtype F32: fl(fl(s*q)+b) with s,b widened to fp32.  out_dtype BF16: needs bf16 s,b. */
int orc_dequantize(const uint32_t* wq, const void* scales, const void* biases, void* out,
                   int64_t N, int64_t K, int bits, int group, int sb_dtype, int out_dtype) {
    if ((bits != 4 && bits != 8) || group <= 0 || K % group || (K * bits) % 32) return 1;
    if (out_dtype == ORC_BF16 && sb_dtype != ORC_BF16) return 3;
    int64_t wpr = K * bits / 32, gpr = K / group;
#pragma omp parallel for
    for (int64_t n = 0; n < N; n++)
        for (int64_t k = 0; k < K; k++) {
            uint32_t q = unpack1(wq + n * wpr, k, bits);
            int64_t gi = n * gpr + k / group;
            if (out_dtype == ORC_BF16)
                ((uint16_t*)out)[n * K + k] = dq_bf16(((const uint16_t*)scales)[gi], ((const uint16_t*)biases)[gi], q);
            else
                ((float*)out)[n * K + k] = dq_f32(load_sb(scales, gi, sb_dtype), load_sb(biases, gi, sb_dtype), q);
        }
    return 0;
}

/* ------------------------------------------------------------------ */
/* quantized matmul                                                     */
/* ------------------------------------------------------------------ */
static int check_args(int64_t M, int64_t K, int64_t N, int bits, int group, int x_dtype, int sb_dtype) {
    if (M < 0 || K <= 0 || N < 0) return 1;
    if ((bits != 4 && bits != 8) || group <= 0 || K % group || (K * bits) % 32) return 1;
    if (x_dtype != ORC_F32 && x_dtype != ORC_BF16) return 1;
    if (sb_dtype != ORC_F32 && sb_dtype != ORC_BF16) return 1;
    if (x_dtype == ORC_BF16 && sb_dtype != ORC_BF16) return 3;
    return 0;
}
static inline float wval(const uint32_t* row, const void* S, const void* B, int64_t gbase,
                         int64_t k, int bits, int group, int x_dtype, int sb_dtype) {
    uint32_t q = unpack1(row, k, bits);
    int64_t gi = gbase + k / group;
    if (x_dtype == ORC_BF16)
        return orc_bf16_to_f32(dq_bf16(((const uint16_t*)S)[gi], ((const uint16_t*)B)[gi], q));
    return dq_f32(load_sb(S, gi, sb_dtype), load_sb(B, gi, sb_dtype), q);
}

/* Reference-style quantized matmul: the loop nest of src/cpu_backend.cpp:253-264
 * (collapse(2) over outputs, sequential fp32 k-sum, multiply then add) with
 * unpack + dequantise fused into the dot product.  This is the timed CPU
 * baseline and the "what the reference CPU backend would compute" value. */
int orc_qmatmul_ref(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* y,
                    int64_t M, int64_t K, int64_t N, int bits, int group,
                    int x_dtype, int sb_dtype, int y_dtype) {
    int rc = check_args(M, K, N, bits, group, x_dtype, sb_dtype);
    if (rc) return rc;
    int64_t wpr = K * bits / 32, gpr = K / group;
#pragma omp parallel for collapse(2)
    for (int64_t i = 0; i < M; i++) {
        for (int64_t j = 0; j < N; j++) {
            const uint32_t* row = wq + j * wpr;
            float sum = 0.0f;
            for (int64_t k = 0; k < K; k++) {
                float xv = x_dtype == ORC_BF16 ? orc_bf16_to_f32(((const uint16_t*)x)[i * K + k])
                                               : ((const float*)x)[i * K + k];
                float prod = xv * wval(row, scales, biases, j * gpr, k, bits, group, x_dtype, sb_dtype);
                sum += prod;
            }
            if (y_dtype == ORC_BF16) ((uint16_t*)y)[i * N + j] = orc_f32_to_bf16(sum);
            else ((float*)y)[i * N + j] = sum;
        }
    }
    return 0;
}

/* Same weights and inputs, fp64 accumulation, fp64 output: the "truth" that
 * tolerances are measured against. */
int orc_qmatmul_truth(const void* x, const uint32_t* wq, const void* scales, const void* biases, double* y,
                      int64_t M, int64_t K, int64_t N, int bits, int group, int x_dtype, int sb_dtype) {
    int rc = check_args(M, K, N, bits, group, x_dtype, sb_dtype);
    if (rc) return rc;
    int64_t wpr = K * bits / 32, gpr = K / group;
#pragma omp parallel
    {
        float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for
        for (int64_t j = 0; j < N; j++) {
            for (int64_t k = 0; k < K; k++)
                wrow[k] = wval(wq + j * wpr, scales, biases, j * gpr, k, bits, group, x_dtype, sb_dtype);
            for (int64_t i = 0; i < M; i++) {
                double sum = 0.0;
                if (x_dtype == ORC_BF16) {
                    const uint16_t* xr = (const uint16_t*)x + i * K;
                    for (int64_t k = 0; k < K; k++) sum += (double)orc_bf16_to_f32(xr[k]) * (double)wrow[k];
                } else {
                    const float* xr = (const float*)x + i * K;
                    for (int64_t k = 0; k < K; k++) sum += (double)xr[k] * (double)wrow[k];
                }
                y[i * N + j] = sum;
            }
        }
        free(wrow);
    }
    return 0;
}

/* Faster CPU baseline variant in the same style (row of W dequantised once,
 * reused over the M rows of x; still fp32 multiply-then-add, sequential k).
 * Produces bit-identical results to orc_qmatmul_ref. */
int orc_qmatmul_ref_rowcache(const void* x, const uint32_t* wq, const void* scales, const void* biases, void* y,
                             int64_t M, int64_t K, int64_t N, int bits, int group,
                             int x_dtype, int sb_dtype, int y_dtype) {
    int rc = check_args(M, K, N, bits, group, x_dtype, sb_dtype);
    if (rc) return rc;
    int64_t wpr = K * bits / 32, gpr = K / group;
#pragma omp parallel
    {
        float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for
        for (int64_t j = 0; j < N; j++) {
            for (int64_t k = 0; k < K; k++)
                wrow[k] = wval(wq + j * wpr, scales, biases, j * gpr, k, bits, group, x_dtype, sb_dtype);
            for (int64_t i = 0; i < M; i++) {
                float sum = 0.0f;
                for (int64_t k = 0; k < K; k++) {
                    float xv = x_dtype == ORC_BF16 ? orc_bf16_to_f32(((const uint16_t*)x)[i * K + k])
                                                   : ((const float*)x)[i * K + k];
                    float prod = xv * wrow[k];
                    sum += prod;
                }
                if (y_dtype == ORC_BF16) ((uint16_t*)y)[i * N + j] = orc_f32_to_bf16(sum);
                else ((float*)y)[i * N + j] = sum;
            }
        }
        free(wrow);
    }
    return 0;
}

/* Dense fp32 matmul in exactly the reference's shape: out[M,N] = A[M,K].B[K,N]
 * (src/cpu_backend.cpp:243-266).  Used to cross-check against the compiled
 * reference and to pin orc_qmatmul_ref's accumulation order. */
void orc_matmul_f32(const float* a, const float* b, float* out, int M, int K, int N) {
#pragma omp parallel for collapse(2)
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            float sum = 0.0f;
            for (int k = 0; k < K; k++) {
                float prod = a[(int64_t)i * K + k] * b[(int64_t)k * N + j];
                sum += prod;
            }
            out[(int64_t)i * N + j] = sum;
        }
}

/* rms-norm, formula of kernels/cpu/tensor_ops.c:546-566: fp32 math over a row,
 * y = x * (1/sqrt(mean(x^2)+eps)) * w.  weight may be NULL (= 1).  in/out fp32 or bf16. */
void orc_rms_norm(const void* in, void* out, const float* weight, int64_t rows, int64_t dim, float eps,
                  int in_dtype, int out_dtype) {
#pragma omp parallel for
    for (int64_t r = 0; r < rows; r++) {
        float ss = 0.0f;
        for (int64_t i = 0; i < dim; i++) {
            float v = in_dtype == ORC_BF16 ? orc_bf16_to_f32(((const uint16_t*)in)[r * dim + i]) : ((const float*)in)[r * dim + i];
            ss += v * v;
        }
        float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int64_t i = 0; i < dim; i++) {
            float v = in_dtype == ORC_BF16 ? orc_bf16_to_f32(((const uint16_t*)in)[r * dim + i]) : ((const float*)in)[r * dim + i];
            float o = v * inv * (weight ? weight[i] : 1.0f);
            if (out_dtype == ORC_BF16) ((uint16_t*)out)[r * dim + i] = orc_f32_to_bf16(o);
            else ((float*)out)[r * dim + i] = o;
        }
    }
}

/* Affine min/max quantiser (the producer of the format): per group,
 * scale = (max-min)/(2^bits-1), bias = min, q = clamp(rint((w-bias)/scale)).
 * scales/biases are rounded to sb_dtype BEFORE q is computed. */
int orc_quantize(const float* w, uint32_t* wq, void* scales, void* biases,
                 int64_t N, int64_t K, int bits, int group, int sb_dtype) {
    if ((bits != 4 && bits != 8) || group <= 0 || K % group || (K * bits) % 32) return 1;
    int64_t gpr = K / group, wpr = K * bits / 32;
    int qmax = (1 << bits) - 1;
    memset(wq, 0, sizeof(uint32_t) * (size_t)(N * wpr));
#pragma omp parallel for
    for (int64_t n = 0; n < N; n++)
        for (int64_t g = 0; g < gpr; g++) {
            const float* p = w + n * K + g * group;
            float lo = p[0], hi = p[0];
            for (int i = 1; i < group; i++) { lo = fminf(lo, p[i]); hi = fmaxf(hi, p[i]); }
            float s = (hi - lo) / (float)qmax, b = lo;
            if (s == 0.0f) s = 1.0f;
            if (sb_dtype == ORC_BF16) {
                uint16_t s16 = orc_f32_to_bf16(s), b16 = orc_f32_to_bf16(b);
                ((uint16_t*)scales)[n * gpr + g] = s16; ((uint16_t*)biases)[n * gpr + g] = b16;
                s = orc_bf16_to_f32(s16); b = orc_bf16_to_f32(b16);
            } else { ((float*)scales)[n * gpr + g] = s; ((float*)biases)[n * gpr + g] = b; }
            for (int i = 0; i < group; i++) {
                float r = rintf((p[i] - b) / s);
                int q = r < 0 ? 0 : (r > qmax ? qmax : (int)r);
                int64_t k = g * group + i;
                if (bits == 4) wq[n * wpr + (k >> 3)] |= (uint32_t)q << (4 * (k & 7));
                else wq[n * wpr + (k >> 2)] |= (uint32_t)q << (8 * (k & 3));
            }
        }
    return 0;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
