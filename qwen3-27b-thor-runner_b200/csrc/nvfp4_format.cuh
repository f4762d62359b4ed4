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

}  // namespace nvfp4
