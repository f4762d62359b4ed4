// Whole-matrix dequantisation and SwiGLU: the two small bandwidth kernels beside
// the linear layer.
#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"

namespace nvfp4 {
namespace {

// out[n,k] = bf16( e2m1 * (ue4m3 * inv_gs) ), bit-exact to the reference's
// fp4_dequant_kernel (src/engine/dense_gemm_fp4_sm110.cu:444-467): the block
// scale is multiplied by inv_gs in FP32 first, then by the table value, then
// rounded once.  One thread per scale block: 8 packed bytes in, 32 bytes out.
__global__ void __launch_bounds__(256)
dequant_bf16_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
                    __nv_bfloat16* __restrict__ out, float inv_gs, long long total_groups) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total_groups; g += stride) {
        const float gs = ue4m3_to_float(scale[g]) * inv_gs;
        const uint2 pk = *reinterpret_cast<const uint2*>(packed + g * 8);
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat16 lo0 = __float2bfloat16_rn(e2m1_lut((pk.x >> (8 * j)) & 0xFu) * gs);
            const __nv_bfloat16 hi0 = __float2bfloat16_rn(e2m1_lut((pk.x >> (8 * j + 4)) & 0xFu) * gs);
            const __nv_bfloat16 lo1 = __float2bfloat16_rn(e2m1_lut((pk.y >> (8 * j)) & 0xFu) * gs);
            const __nv_bfloat16 hi1 = __float2bfloat16_rn(e2m1_lut((pk.y >> (8 * j + 4)) & 0xFu) * gs);
            o[j] = (uint32_t)__bfloat16_as_ushort(lo0) | ((uint32_t)__bfloat16_as_ushort(hi0) << 16);
            o[4 + j] = (uint32_t)__bfloat16_as_ushort(lo1) | ((uint32_t)__bfloat16_as_ushort(hi1) << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + g * 16);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// silu(x) = x / (1 + exp(-x)) in FP32, product rounded once to BF16
// (src/engine/light_ops.cu:168-199 and :1542-1577).  gate and up rows are
// row_stride_in elements apart (I for separate tensors, 2I for the merged layout).

__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
              __nv_bfloat16* __restrict__ out, long long row_stride_in, long long row_stride_out, int M, int I) {
    const int vec_per_row = I >> 3;
    const long long total = (long long)M * vec_per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += stride) {
        const int m = (int)(v / vec_per_row), c = (int)(v % vec_per_row) * 8;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gate + (size_t)m * row_stride_in + c);
        const uint4 u4 = *reinterpret_cast<const uint4*>(up + (size_t)m * row_stride_in + c);
        *reinterpret_cast<uint4*>(out + (size_t)m * row_stride_out + c) = swiglu_bf16x8(g4, u4);
    }
    // I % 8 tail columns, scalar.
    const int tail0 = vec_per_row * 8;
    if (tail0 < I) {
        const long long ttotal = (long long)M * (I - tail0);
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ttotal; t += stride) {
            const int m = (int)(t / (I - tail0)), c = tail0 + (int)(t % (I - tail0));
            const float g = __bfloat162float(gate[(size_t)m * row_stride_in + c]);
            const float u = __bfloat162float(up[(size_t)m * row_stride_in + c]);
            out[(size_t)m * row_stride_out + c] = __float2bfloat16_rn(silu(g) * u);
        }
    }
}

int grid_for(long long work_items, int block) {
    long long blocks = (work_items + block - 1) / block;
    const long long cap = 148LL * 16;   // a few waves of 148 SMs; kernels grid-stride beyond it
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

cudaError_t launch_dequant_bf16(const uint8_t* packed, const uint8_t* scale, float inv_gs, int N, int K,
                                void* out, cudaStream_t s) {
    const long long groups = (long long)N * (K >> 4);
    dequant_bf16_kernel<<<grid_for(groups, 256), 256, 0, s>>>(packed, scale, static_cast<__nv_bfloat16*>(out),
                                                            inv_gs, groups);
    return cudaGetLastError();
}

cudaError_t launch_swiglu(const void* gate, const void* up, long long row_stride_in, int M, int I,
                          void* out, long long row_stride_out, cudaStream_t s) {
    const long long vecs = (long long)M * ((I + 7) >> 3);
    swiglu_kernel<<<grid_for(vecs, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gate),
                                                    static_cast<const __nv_bfloat16*>(up),
                                                    static_cast<__nv_bfloat16*>(out), row_stride_in, row_stride_out, M, I);
    return cudaGetLastError();
}

}  // namespace nvfp4
