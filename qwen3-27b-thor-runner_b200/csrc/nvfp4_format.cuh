// NVFP4 number formats on the device: E2M1 codes, unsigned-E4M3 block scales, BF16.
// Value semantics follow the reference engine's table and decoder
// (src/engine/dense_gemm_fp4_sm110.cu:24-41): code 8 decodes to +0.0f, the scale
// byte's top bit is ignored, exponent 0 is the 2^-9 subnormal grid and 0x7F is
// 480 (no NaN).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nvfp4 {

// E2M1 magnitude code (3 bits: e e m) -> 0, .5, 1, 1.5, 2, 3, 4, 6.
__device__ __forceinline__ float e2m1_mag(uint32_t code3) {
    // Two byte tables holding 2*value: {0,1,2,3} and {4,6,8,12}.
    const uint32_t tab = (code3 & 4u) ? 0x0C080604u : 0x03020100u;
    return 0.5f * (float)((tab >> ((code3 & 3u) * 8u)) & 0xFFu);
}

// Full 4-bit code -> FP32; codes 8..15 are the negatives except code 8, which is
// +0.0f exactly as in the reference table.
__device__ __forceinline__ float e2m1_lut(uint32_t code4) {
    const float v = e2m1_mag(code4 & 7u);
    return ((code4 & 8u) && (code4 & 7u)) ? -v : v;
}

// Unsigned E4M3 -> FP32, exact.
__device__ __forceinline__ float ue4m3_to_float(uint32_t byte) {
    const uint32_t exp = (byte >> 3) & 0xFu;
    const uint32_t man = byte & 0x7u;
    if (exp == 0u) return (float)man * 1.953125e-3f;             // man * 2^-9
    return __uint_as_float(((exp + 120u) << 23) | (man << 20));  // (1+man/8) * 2^(exp-7)
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

// silu(x) = x / (1 + exp(-x)) in FP32 (src/engine/light_ops.cu:168-170).
__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

// Eight BF16 gate values and eight BF16 up values -> eight BF16 bf16(silu(gate) * up), the
// reference's SwiGLU with its single rounding (src/engine/light_ops.cu:186-187, :1566-1572).
__device__ __forceinline__ uint4 swiglu_bf16x8(uint4 g4, uint4 u4) {
    const uint32_t gv[4] = {g4.x, g4.y, g4.z, g4.w}, uv[4] = {u4.x, u4.y, u4.z, u4.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float g0 = bf16_bits_to_float(gv[j] & 0xFFFFu), g1 = bf16_bits_to_float(gv[j] >> 16);
        const float u0 = bf16_bits_to_float(uv[j] & 0xFFFFu), u1 = bf16_bits_to_float(uv[j] >> 16);
        const __nv_bfloat162 r = __floats2bfloat162_rn(silu(g0) * u0, silu(g1) * u1);
        o[j] = *reinterpret_cast<const uint32_t*>(&r);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Block scales for the f16x2 dequantisation, without a table.  An unsigned E4M3 byte x (bit 7
// ignored) equals the FP16 number whose bit pattern is x << 7, times 2^8: normal codes because
// the exponent bias moves from 7 to 15, the subnormal codes because FP16 subnormals scale the
// same way, and 0x7F gives 480 like the reference's decoder (no NaN code).  Products
// e2m1 * (x << 7 as FP16) are exact in FP16 (at least 2^-18, 2 + 4 significant bits), so the
// kernels multiply by this operand and restore kBlockScaleUnfold once, in their FP32 epilogue.
constexpr float kBlockScaleUnfold = 256.0f;

__device__ __forceinline__ uint32_t mask_scale_bytes(uint32_t four_scale_bytes) { return four_scale_bytes & 0x7F7F7F7Fu; }

// {s, s} as f16x2 with s = ue4m3(byte b of w) / 2^8; w holds four scale bytes, already masked.
__device__ __forceinline__ uint32_t scale_byte_to_f16x2(uint32_t w_masked, int b) {
    uint32_t d;
    const uint32_t sel = 0x4040u | (uint32_t)b | ((uint32_t)b << 8);      // bytes {b, zero, b, zero}
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w_masked), "r"(0u), "r"(sel));
    return d * 128u;                                                      // << 7 inside both halves
}

}  // namespace nvfp4
