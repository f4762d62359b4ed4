// Activation pre-pass of the NVFP4 tensor-core GEMV (decode_fp4.cu): BF16 activations -> a short sum of
// NVFP4 terms.
//
// tcgen05.mma kind::mxf4nvf4 multiplies NVFP4 by NVFP4 (E2M1 codes, one unsigned E4M3 scale per 16
// elements along K) -- exactly the layout the weights already have in HBM, so they need no
// conversion at all.  The activations are BF16 and must stay at BF16 accuracy, so every token is
// expanded into T NVFP4 "term" rows whose sum reproduces it (T = 5, or 6 where the sixth costs no MMA columns):
//     x * c = q_0 * s_0 + q_1 * s_1 + ... + q_{T-1} * s_{T-1}   (per 16-element block, up to a remainder)
// c is a per-token power of two that puts the token's largest magnitude into [2^9, 2^10); s_0 is the
// smallest power of two with |x c| <= 6 s_0 over the block; s_1 = s_0 / 4, then each next scale is 1/8
// of the one before; q_t is the remainder so far rounded to the nearest E2M1 value (the hardware
// conversion).  After a term the remainder is at most half the local E2M1 spacing (half the
// term's scale for values up to 4), which gives |remainder| <= s_0 / 4096 after five terms and
// s_0 / 32768 after six: 8e-5 and 1e-5 of the block's largest element, whose own BF16 rounding step is 4e-3.
// All scales are powers of two, so every product and every remainder is exact in FP32.  The term
// rows become columns of the MMA's B operand (tokens x T, padded to a multiple of 16); the GEMV's
// epilogue adds the T columns of a token.
//
// Outputs: codes [NCp, K/2] (row c = token * 5 + term; two codes per byte, low nibble = even k), the
// block scales in the order the GEMV moves them into tensor memory (see sfb_offset), and 1 / c per token.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "nvfp4_internal.h"
#include "ptx.cuh"

namespace nvfp4 {
namespace {

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

constexpr int kSliceBlocks = 64;        // 16-element blocks (1024 k) per CTA
constexpr int kPreThreads = 4 * kSliceBlocks;
constexpr int kMaxRowLoads = 4;         // 16-byte loads of the row per thread held in registers at once

// grid: (K slices, tokens).  Every CTA finds the token's largest magnitude over the whole row (cheap, and
// it saves a grid-wide step), then expands its own slice: four threads per 16-element block, four
// elements each (the five terms are a dependent chain per element, so more threads, not longer ones).
// All loads are issued before the first use, so the kernel pays one trip to L2.
// Columns beyond tokens x 5 are never written: whatever an earlier call left there only reaches
// accumulator columns the GEMV's epilogue does not read (stale codes and scales are finite).
template <int TERMS>
__global__ void __launch_bounds__(kPreThreads)
act_to_fp4_kernel(const __nv_bfloat16* __restrict__ A, long long a_stride, int K, int groups,
                  uint8_t* __restrict__ codes, uint8_t* __restrict__ sfb, float* __restrict__ unscale) {
    __shared__ unsigned int s_max;
    const int m = blockIdx.y;
    const int blocks = K / 16;
    if (threadIdx.x == 0) s_max = 0u;
    ptx::griddep_launch_dependents();      // the GEMV behind this kernel may set itself up and start streaming weights
    ptx::griddep_wait();                   // A is the output of the kernel before this one
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(A + (size_t)m * a_stride);
    const int b = blockIdx.x * kSliceBlocks + (threadIdx.x >> 2), part = threadIdx.x & 3;     // block, quarter of it
    const bool live = b < blocks;                          // whole quads are live or not: the shuffles below stay converged
    uint2 own = make_uint2(0u, 0u);
    if (live) own = __ldg(reinterpret_cast<const uint2*>(src + 2 * b) + part);
    unsigned int amax = 0;
    for (int i0 = threadIdx.x; i0 < K / 8; i0 += kPreThreads * kMaxRowLoads) {
        uint4 x[kMaxRowLoads];
#pragma unroll
        for (int j = 0; j < kMaxRowLoads; ++j) {
            const int i = i0 + j * kPreThreads;
            x[j] = i < K / 8 ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < kMaxRowLoads; ++j) {
            const uint32_t v[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) amax = max(amax, max(v[q] & 0x7FFFu, (v[q] >> 16) & 0x7FFFu));
        }
    }
    amax = __reduce_max_sync(0xffffffffu, amax);
    if ((threadIdx.x & 31) == 0 && amax) atomicMax(&s_max, amax);
    __syncthreads();
    // c = 2^(136 - e): the largest element (biased BF16 exponent e) lands in [2^9, 2^10)
    int se = 263 - (int)(s_max >> 7);
    se = se < 1 ? 1 : (se > 254 ? 254 : se);
    const float c = __uint_as_float((uint32_t)se << 23);
    if (blockIdx.x == 0 && threadIdx.x == 0) unscale[m] = __uint_as_float((uint32_t)(254 - se) << 23);
    float r[4];
    r[0] = __uint_as_float(own.x << 16) * c;
    r[1] = __uint_as_float(own.x & 0xFFFF0000u) * c;
    r[2] = __uint_as_float(own.y << 16) * c;
    r[3] = __uint_as_float(own.y & 0xFFFF0000u) * c;
    float bmax = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
    if (live) {
        // p0: smallest p with bmax <= 6 * 2^p, clamped to the unsigned E4M3 range of powers of two
        int p0 = -9;
        if (bmax > 0.0f && bmax < 3.0e38f) {
            const uint32_t u = __float_as_uint(bmax * (1.0f / 6.0f));
            p0 = (int)(u >> 23) - 127 + ((u & 0x7FFFFFu) ? 1 : 0);
            if (bmax > 6.0f * __uint_as_float((uint32_t)(p0 + 127) << 23)) ++p0;     // 1/6 is not exact: never let the block exceed 6 s_0
        }
        p0 = p0 < -9 ? -9 : (p0 > 8 ? 8 : p0);
#pragma unroll
        for (int t = 0; t < TERMS; ++t) {
            int p = p0 - (t == 0 ? 0 : 2 + 3 * (t - 1));
            p = p < -9 ? -9 : p;
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
            const int col = m * TERMS + t;
            *reinterpret_cast<uint16_t*>(codes + (size_t)col * (K / 2) + (size_t)b * 8 + part * 2) = (uint16_t)w;
            if (part == 0) sfb[fp4::sfb_offset(b, col, groups)] = (uint8_t)ue4m3_pow2(p);
        }
    }
}

}  // namespace

cudaError_t launch_act_to_fp4(const void* A, long long a_stride, int M, int K, int terms, int groups, void* codes, void* sfb,
                              float* unscale, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((K / 16 + kSliceBlocks - 1) / kSliceBlocks, M);
    cfg.blockDim = dim3(kPreThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(A);
    uint8_t* c = static_cast<uint8_t*>(codes);
    uint8_t* f = static_cast<uint8_t*>(sfb);
    if (terms == 6) return cudaLaunchKernelEx(&cfg, act_to_fp4_kernel<6>, src, a_stride, K, groups, c, f, unscale);
    if (terms == 5) return cudaLaunchKernelEx(&cfg, act_to_fp4_kernel<5>, src, a_stride, K, groups, c, f, unscale);
    return cudaErrorInvalidValue;
}

}  // namespace nvfp4
