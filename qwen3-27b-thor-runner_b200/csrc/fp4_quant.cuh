// BF16 activations -> NVFP4 terms: the arithmetic shared by the stand-alone pre-pass (act_fp4.cu) and the
// GEMV that expands its own activations (decode_fp4.cu, one or two tokens).  See act_fp4.cu for the scheme.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace nvfp4 {
namespace fp4q {

// Two FP32 -> one byte of E2M1 codes, `lo` in the low nibble (round to nearest even, saturating at 6).
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t d;
    asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\tmov.b16 %0, {b, b};\n\t}" : "=h"(d) : "f"(hi), "f"(lo));
    return d;
}
// One byte of E2M1 codes -> two floats.
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
    uint32_t h2;
    asm("{\n\t.reg .b8 b, z;\n\tmov.b16 {b, z}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(h2) : "h"((uint16_t)byte));
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}
// 2^p as an unsigned E4M3 byte, p in [-9, 8].
__device__ __forceinline__ uint32_t ue4m3_pow2(int p) {
    return p >= -6 ? (uint32_t)(p + 7) << 3 : (p == -7 ? 4u : (p == -8 ? 2u : 1u));
}
// The token factor c = 2^(136 - e) that puts the token's largest magnitude (BF16 magnitude bits, biased
// exponent e) into [2^9, 2^10); returns its biased FP32 exponent (1 / c has exponent 254 - that).
__device__ __forceinline__ int token_scale_exponent(unsigned int amax_bf16_bits) {
    int se = 263 - (int)(amax_bf16_bits >> 7);
    return se < 1 ? 1 : (se > 254 ? 254 : se);
}
// 1 / c for the epilogue.  A token that holds an infinity or a NaN has no finite expansion: its factor is NaN, so
// every output of that token is NaN (what FP32 accumulation of such an input gives, up to inf versus NaN) and no
// other token is touched.
__device__ __forceinline__ float token_unscale(unsigned int amax_bf16_bits, int se) {
    return (amax_bf16_bits >> 7) >= 0xFFu ? __uint_as_float(0x7FC00000u) : __uint_as_float((uint32_t)(254 - se) << 23);
}
// Exponent of the first term's scale: the smallest p with bmax <= 6 * 2^p, clamped to the powers of two unsigned E4M3 holds.
__device__ __forceinline__ int first_term_exponent(float bmax) {
    int p0 = -9;
    if (bmax > 0.0f && bmax < 3.0e38f) {
        const uint32_t u = __float_as_uint(bmax * (1.0f / 6.0f));
        p0 = (int)(u >> 23) - 127 + ((u & 0x7FFFFFu) ? 1 : 0);
        if (bmax > 6.0f * __uint_as_float((uint32_t)(p0 + 127) << 23)) ++p0;     // 1/6 is not exact: never let the block exceed 6 s_0
    }
    return p0 < -9 ? -9 : (p0 > 8 ? 8 : p0);
}
// Exponent of term t's scale: s_1 = s_0 / 4, then a factor 8 per term, never below the smallest scale.
__device__ __forceinline__ int term_exponent(int p0, int t) {
    const int p = p0 - (t == 0 ? 0 : 2 + 3 * (t - 1));
    return p < -9 ? -9 : p;
}
// One term of a quarter block (four elements): the two code bytes, the remainder left in r.
__device__ __forceinline__ uint32_t take_term(float (&r)[4], int p) {
    const float s = __uint_as_float((uint32_t)(p + 127) << 23), inv = __uint_as_float((uint32_t)(127 - p) << 23);
    uint32_t w = 0u;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const uint32_t byte = cvt_e2m1x2(r[2 * q] * inv, r[2 * q + 1] * inv) & 0xFFu;
        const float2 d = e2m1x2_to_float2(byte);
        r[2 * q] -= d.x * s;
        r[2 * q + 1] -= d.y * s;
        w |= byte << (8 * q);
    }
    return w;
}

}  // namespace fp4q
}  // namespace nvfp4
