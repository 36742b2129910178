// In-register dequantisation of packed 4-bit / 8-bit words to bf16x2 pairs,
// w^ = RNE_bf16(scale*q + bias): exactly one bf16 FMA per pair of weights.
//
// Fast path.  A bf16 whose upper 8 bits are zero encodes the integer u in its
// low 8 bits as the value u * 2^-133: the subnormal range (u < 128) and the
// first normal binade (128 <= u < 256) are one linear ramp.  So
//     (word      ) & 0x000F000F   is the pair (q0, q4)        * 2^-133
//     (word      ) & 0x00F000F0   is the pair (q1, q5) * 16   * 2^-133
//     (word >>  8) & 0x000F000F   is the pair (q2, q6)        * 2^-133
//     (word >>  8) & 0x00F000F0   is the pair (q3, q7) * 16   * 2^-133
// (8-bit: (word) & 0x00FF00FF = (q0, q2), (word >> 8) & 0x00FF00FF = (q1, q3))
// and fma(field, scale * 2^133 [or * 2^129], bias) is the exact product
// scale*q plus bias, rounded once -- bit-identical to converting q to bf16
// first.  One shift and four masks per eight weights, no subtract.
// The rescaled scale is the scale with 133 (129) added to its exponent field,
// valid when that field e satisfies 1 <= e <= 121 (normal, below 2^-5).
// Anything else (zero, subnormal, large, inf/nan scales) takes the general
// path: (field | 0x4300) is 128+q, one FMA by 1.0 with -128 recovers q.
#pragma once
#include <cstdint>

namespace luxcuda {

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// scale given as raw bf16 bits (16 bit): may the exponent trick be used?
__device__ __forceinline__ bool scale_fast_ok(uint32_t s_bits) {
    const uint32_t e = (s_bits >> 7) & 0xFFu;
    return e >= 1u && e <= 121u;
}
// Integer helpers written as multiply-adds on purpose: on sm_100 the integer/logic pipe
// issues at half the rate of the FMA pipe and is the busy one in the dequantising
// kernels, so everything that can be phrased as IMAD is kept off it.
__device__ __forceinline__ uint32_t imad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t shr8(uint32_t w) { return w >> 8; }  // (IMAD.HI was measured slower than SHF)
// bf16x2 (s, s) * 2^133 and * 2^129 from raw bf16 bits (16 bit): duplicate + exponent offset
__device__ __forceinline__ uint32_t scale_x2_133(uint32_t s_bits) { return imad(s_bits, 0x00010001u, 0x42804280u); }
__device__ __forceinline__ uint32_t scale_x2_129(uint32_t s_bits) { return imad(s_bits, 0x00010001u, 0x40804080u); }
__device__ __forceinline__ uint32_t dup_bf16(uint32_t bits) { return imad(bits, 0x00010001u, 0u); }

// 4-bit, fast: out[i] = (w^_i, w^_{i+4}), i = 0..3
__device__ __forceinline__ void dequant4_fast(uint32_t w, uint32_t s133, uint32_t s129, uint32_t b2, uint32_t (&out)[4]) {
    const uint32_t w8 = shr8(w);
    out[0] = fma_bf16x2(w & 0x000F000Fu, s133, b2);
    out[1] = fma_bf16x2(w & 0x00F000F0u, s129, b2);
    out[2] = fma_bf16x2(w8 & 0x000F000Fu, s133, b2);
    out[3] = fma_bf16x2(w8 & 0x00F000F0u, s129, b2);
}
// 4-bit, general
__device__ __forceinline__ void dequant4_general(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t v = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;  // (128+q_i, 128+q_{i+4})
        out[i] = fma_bf16x2(fma_bf16x2(v, 0x3F803F80u, 0xC300C300u), s2, b2);
    }
}
// 8-bit, fast: out[0] = (w^_0, w^_2), out[1] = (w^_1, w^_3)
__device__ __forceinline__ void dequant8_fast(uint32_t w, uint32_t s133, uint32_t b2, uint32_t (&out)[2]) {
    out[0] = fma_bf16x2(w & 0x00FF00FFu, s133, b2);
    out[1] = fma_bf16x2(shr8(w) & 0x00FF00FFu, s133, b2);
}
// 8-bit, general: byte | 0x4B000000 is the float 2^23 + q
__device__ __forceinline__ void dequant8_general(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[2]) {
    const float f0 = __uint_as_float(prmt(w, 0x4B000000u, 0x7540u)) - 8388608.0f;
    const float f1 = __uint_as_float(prmt(w, 0x4B000000u, 0x7541u)) - 8388608.0f;
    const float f2 = __uint_as_float(prmt(w, 0x4B000000u, 0x7542u)) - 8388608.0f;
    const float f3 = __uint_as_float(prmt(w, 0x4B000000u, 0x7543u)) - 8388608.0f;
    uint32_t p02, p13;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p02) : "f"(f2), "f"(f0));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p13) : "f"(f3), "f"(f1));
    out[0] = fma_bf16x2(p02, s2, b2);
    out[1] = fma_bf16x2(p13, s2, b2);
}

}  // namespace luxcuda
