// Pieces shared by the two mma.sync GEMV kernels (decode_mma.cu: up to 8 tokens per launch with
// resident activations; decode_wide.cu: 9..16 tokens with the activations copied beside the ring).
#pragma once
#include <cstddef>
#include <cstdint>

#include "ptx.cuh"

namespace nvfp4 {
namespace gemv {

constexpr int kRT = 128;                          // rows per half-unit
constexpr int kKC = 256;                          // k elements per half-unit
constexpr int kGroupWarps = 8;                    // warps that share one half-unit (16 rows each)
constexpr int kPackedBytes = kRT * kKC / 2;       // 16384 per half-unit
constexpr int kScaleBytes = kRT * kKC / 16;       // 2048 per half-unit
constexpr int kActBlockBytes = 128 + 16;          // 64 k of FP16 + 16 bytes of padding
constexpr int kActRowBytes = 4 * kActBlockBytes;  // 576 per token per half-unit: four padded 64-k blocks
constexpr int kOutLd = kRT + 4;                   // padded row of the FP32 exchange tile

// Scratch layout (handle workspace): status word, then the per-CTA partial tiles.
constexpr size_t kPartialOffset = 16384;
// Split-tile partials travel as 8-byte {FP32 value, launch epoch} pairs (the data is its own arrival
// flag).  The wide kernel's, [CTA][16 tokens][256 rows], start at kPartialOffset (32 KB per CTA); the
// 8-token kernel's, [CTA][8 tokens][128 rows], at kPairOffset (8 KB per CTA).
constexpr size_t kPairOffset = 6u << 20;
constexpr int kMaxGrid = 256;                     // CTAs of the 8-token kernel whose pairs fit its 2 MB of scratch

// Activation row of one (k-chunk, token): four 64-k blocks of 128 bytes, each followed by 16
// bytes of padding.  Lane (g, t) of a consumer warp reads block t of token g, 16 bytes at a
// time at immediate offsets; with the padding the 8 lanes of a quarter-warp (2 tokens x 4
// blocks) hit 8 different 16-byte bank groups ((4*token + t + chunk) mod 8), no XOR needed.
__device__ __forceinline__ int act_chunk_offset(int c) { return (c >> 3) * kActBlockBytes + (c & 7) * 16; }

// Eight packed E2M1 codes (one 32-bit word, 8 consecutive k of one row) -> four f16x2 registers
// holding e2m1 * (block scale / 2^8), in k order.  The hardware conversion is exact and the
// products are exact in FP16 (2 + 4 significant bits, all within [2^-18, 11.25]).
__device__ __forceinline__ void expand_u32(uint32_t q, uint32_t S, uint32_t (&d)[4]) {
    uint32_t e[4];
    ptx::cvt_e2m1x8_to_f16x2(q, e);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = ptx::mul_f16x2(e[i], S);
}

}  // namespace gemv
}  // namespace nvfp4
