// Whole-matrix dequantisation, SwiGLU and RMSNorm: the small bandwidth kernels beside
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
// row_stride_in elements apart (I for separate tensors, 2I for the merged layout).  interleaved:
// the input row holds slabs of 16 columns, 8 gate values followed by their 8 up values (the
// output of a linear on row-interleaved gate/up weights); gate points at column 0, up at column 8.

__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
              __nv_bfloat16* __restrict__ out, long long row_stride_in, long long row_stride_out, int M, int I,
              int interleaved) {
    const int vec_per_row = I >> 3;
    const long long total = (long long)M * vec_per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += stride) {
        const int m = (int)(v / vec_per_row), c = (int)(v % vec_per_row) * 8;
        const int cin = interleaved ? 2 * c : c;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gate + (size_t)m * row_stride_in + cin);
        const uint4 u4 = *reinterpret_cast<const uint4*>(up + (size_t)m * row_stride_in + cin);
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

namespace {

// How many block-scale bytes of a weight are 0x7F or 0xFF: 480 to the reference's decoder
// (src/engine/dense_gemm_fp4_sm110.cu:30-41), NaN to the tensor core's FP8 E4M3.  16 bytes per load where the
// pointer allows it, byte by byte for the rest.
__global__ void __launch_bounds__(256)
count_nan_scales_kernel(const uint8_t* __restrict__ scale, long long bytes, unsigned long long* count) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    const long long vecs = (reinterpret_cast<uintptr_t>(scale) & 15u) == 0 ? bytes >> 4 : 0;
    unsigned int n = 0;
    for (long long i = tid; i < vecs; i += nthr) {
        const uint4 x = __ldg(reinterpret_cast<const uint4*>(scale) + i);
        n += (__popc(__vcmpeq4(x.x | 0x80808080u, 0xFFFFFFFFu)) + __popc(__vcmpeq4(x.y | 0x80808080u, 0xFFFFFFFFu)) +
              __popc(__vcmpeq4(x.z | 0x80808080u, 0xFFFFFFFFu)) + __popc(__vcmpeq4(x.w | 0x80808080u, 0xFFFFFFFFu))) >> 3;
    }
    for (long long i = (vecs << 4) + tid; i < bytes; i += nthr) n += (scale[i] & 0x7Fu) == 0x7Fu;
    n = __reduce_add_sync(0xffffffffu, n);
    if ((threadIdx.x & 31) == 0 && n) atomicAdd(count, (unsigned long long)n);
}

}  // namespace

cudaError_t launch_count_nan_scales(const uint8_t* scale, long long bytes, unsigned long long* count, cudaStream_t s) {
    count_nan_scales_kernel<<<grid_for((bytes + 15) >> 4, 256), 256, 0, s>>>(scale, bytes, count);
    return cudaGetLastError();
}

namespace {

// RMSNorm with the centred weight, one CTA per token:
//   out = bf16( (x * rsqrt(mean(x^2) + eps)) * (1 + w) ), FP32 throughout
// (rmsnorm_kernel, src/engine/light_ops.cu:65-106).  With `bias` the row is x + bias first, kept
// unrounded for the norm, and bf16(x + bias) goes back to x (fused_add_rmsnorm_kernel, :270-318).
// 16-byte chunks; a thread keeps up to kNormCache chunks in registers between the two passes and
// reads the row again beyond that.  1/sqrtf and a true division, not the fast-math forms.
constexpr int kNormThreads = 256;
constexpr int kNormCache = 6;                 // x 256 threads x 8 elements = 12288 columns from registers

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(__nv_bfloat16* out, __nv_bfloat16* x, const __nv_bfloat16* __restrict__ bias,
               const __nv_bfloat16* __restrict__ weight, float eps, int K) {
    __shared__ float s_part[kNormThreads / 32];
    __shared__ float s_inv;
    const int tid = threadIdx.x;
    const size_t row = (size_t)blockIdx.x * K;
    const int chunks = K >> 3;
    auto load = [&](int c, float (&v)[8]) {
        const uint4 a = *reinterpret_cast<const uint4*>(x + row + (size_t)c * 8);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(aw[i] << 16);
            v[2 * i + 1] = __uint_as_float(aw[i] & 0xFFFF0000u);
        }
        if (bias) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias + row + (size_t)c * 8));
            const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] += __uint_as_float(bw[i] << 16);
                v[2 * i + 1] += __uint_as_float(bw[i] & 0xFFFF0000u);
            }
        }
    };
    float cache[kNormCache][8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kNormCache; ++j) {
        const int c = tid + j * kNormThreads;
        if (c < chunks) {
            load(c, cache[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(cache[j][i], cache[j][i], ss);
        }
    }
    for (int c = tid + kNormCache * kNormThreads; c < chunks; c += kNormThreads) {
        float v[8];
        load(c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) s_part[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < kNormThreads / 32; ++i) t += s_part[i];
        s_inv = 1.0f / sqrtf(t / (float)K + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    auto store = [&](int c, const float (&v)[8]) {
        const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(weight + (size_t)c * 8));
        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
        uint32_t o[4], r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float w0 = 1.0f + __uint_as_float(ww[i] << 16), w1 = 1.0f + __uint_as_float(ww[i] & 0xFFFF0000u);
            const __nv_bfloat162 y = __floats2bfloat162_rn(v[2 * i] * inv * w0, v[2 * i + 1] * inv * w1);
            o[i] = *reinterpret_cast<const uint32_t*>(&y);
            const __nv_bfloat162 q = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            r[i] = *reinterpret_cast<const uint32_t*>(&q);
        }
        if (bias) *reinterpret_cast<uint4*>(x + row + (size_t)c * 8) = make_uint4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<uint4*>(out + row + (size_t)c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    };
    // the uncached tail first: with a bias its x is still the old value only until it is stored
    for (int c = tid + kNormCache * kNormThreads; c < chunks; c += kNormThreads) {
        float v[8];
        load(c, v);
        store(c, v);
    }
#pragma unroll
    for (int j = 0; j < kNormCache; ++j) {
        const int c = tid + j * kNormThreads;
        if (c < chunks) store(c, cache[j]);
    }
}

}  // namespace

cudaError_t launch_rmsnorm(void* out, void* x, const void* bias, const void* weight, float eps, int M, int K,
                           cudaStream_t s) {
    rmsnorm_kernel<<<M, kNormThreads, 0, s>>>(static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(x),
                                              static_cast<const __nv_bfloat16*>(bias),
                                              static_cast<const __nv_bfloat16*>(weight), eps, K);
    return cudaGetLastError();
}

cudaError_t launch_swiglu(const void* gate, const void* up, long long row_stride_in, int M, int I,
                          void* out, long long row_stride_out, cudaStream_t s, bool interleaved) {
    const long long vecs = (long long)M * ((I + 7) >> 3);
    swiglu_kernel<<<grid_for(vecs, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gate),
                                                    static_cast<const __nv_bfloat16*>(up),
                                                    static_cast<__nv_bfloat16*>(out), row_stride_in, row_stride_out, M, I,
                                                    interleaved ? 1 : 0);
    return cudaGetLastError();
}

}  // namespace nvfp4
