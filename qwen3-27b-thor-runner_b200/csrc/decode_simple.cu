// Scalar CUDA-core dequant-GEMV: the plain, shape-agnostic decode path.
//
// One warp per output row n; lanes stride the row's 16-element scale blocks, so a
// warp reads 256 contiguous packed bytes per step.  Per block: one 8-byte weight
// load, one scale byte, FP32 dot of the 16 products, multiplied by the block scale
// and added to the row sum -- the arithmetic order of the reference's GEMV
// (src/engine/dense_gemm_fp4_sm110.cu:96-141 and :192-240) -- then a shuffle
// reduction, the optional residual in FP32 and a single rounding to BF16.
// Works for any K % 16 == 0 and M <= 16; it is the fallback for shapes the
// TMA-fed kernel does not take and the in-library cross-check of that kernel.
#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"

namespace nvfp4 {
namespace {

constexpr int kWarpsPerBlock = 8;

template <int MT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
decode_simple_kernel(const __nv_bfloat16* __restrict__ A, const uint8_t* __restrict__ packed,
                     const uint8_t* __restrict__ scale, const __nv_bfloat16* residual,
                     __nv_bfloat16* C, float inv_gs, int M, int N, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * kWarpsPerBlock + warp;
    if (n >= N) return;
    const int groups = K >> 4;
    const uint8_t* w_row = packed + (size_t)n * (K >> 1);
    const uint8_t* s_row = scale + (size_t)n * groups;

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

    for (int g = lane; g < groups; g += 32) {
        const float gs = ue4m3_to_float(s_row[g]) * inv_gs;
        const uint2 pk = *reinterpret_cast<const uint2*>(w_row + (size_t)g * 8);
        float w[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            w[j] = e2m1_lut((pk.x >> (4 * j)) & 0xFu);
            w[8 + j] = e2m1_lut((pk.y >> (4 * j)) & 0xFu);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const uint4* ap = reinterpret_cast<const uint4*>(A + (size_t)m * K + ((size_t)g << 4));
                const uint4 a0 = __ldg(ap), a1 = __ldg(ap + 1);
                const uint32_t av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    dot += bf16_bits_to_float(av[j] & 0xFFFFu) * w[2 * j] +
                           bf16_bits_to_float(av[j] >> 16) * w[2 * j + 1];
                }
                acc[m] += dot * gs;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                float v = acc[m];
                if (residual) v += __bfloat162float(residual[(size_t)m * N + n]);
                C[(size_t)m * N + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

}  // namespace

cudaError_t launch_decode_simple(const LinearArgs& a, cudaStream_t s) {
    const dim3 grid((a.N + kWarpsPerBlock - 1) / kWarpsPerBlock), block(kWarpsPerBlock * 32);
    const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(a.A);
    const __nv_bfloat16* R = static_cast<const __nv_bfloat16*>(a.residual);
    __nv_bfloat16* C = static_cast<__nv_bfloat16*>(a.C);
#define NVFP4_LAUNCH(MT) \
    decode_simple_kernel<MT><<<grid, block, 0, s>>>(A, a.packed, a.scale, R, C, a.inv_gs, a.M, a.N, a.K)
    if (a.M <= 1) NVFP4_LAUNCH(1);
    else if (a.M <= 2) NVFP4_LAUNCH(2);
    else if (a.M <= 4) NVFP4_LAUNCH(4);
    else if (a.M <= 8) NVFP4_LAUNCH(8);
    else NVFP4_LAUNCH(16);
#undef NVFP4_LAUNCH
    return cudaGetLastError();
}

}  // namespace nvfp4
