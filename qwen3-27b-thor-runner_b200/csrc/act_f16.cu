// Activation pre-pass of the tcgen05 kernels: BF16 -> FP16 with an exact per-token power-of-two
// scale (largest magnitude of the token -> [2^14, 2^15)), so BF16's wider exponent range costs
// nothing; the GEMM epilogue multiplies by the inverse factor in FP32.  The tensor core takes
// both operands in one 16-bit format, and the hardware E2M1 conversion produces FP16 weights.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "nvfp4_internal.h"
#include "ptx.cuh"

namespace nvfp4 {
namespace {

// One CTA per token.
__global__ void __launch_bounds__(1024)
act_to_f16_kernel(const __nv_bfloat16* __restrict__ A, __half* __restrict__ out, float* __restrict__ unscale, int K) {
    __shared__ unsigned int s_max;
    const int m = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(A + (size_t)m * K);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)m * K);
    if (threadIdx.x == 0) s_max = 0u;
    ptx::griddep_launch_dependents();      // the GEMM behind this kernel may set itself up and start streaming weights
    ptx::griddep_wait();                   // A is the output of the kernel before this one
    __syncthreads();
    unsigned int amax = 0;
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
        const uint4 x = __ldg(src + i);
        const uint32_t v[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) amax = max(amax, max(v[q] & 0x7FFFu, (v[q] >> 16) & 0x7FFFu));
    }
    amax = __reduce_max_sync(0xffffffffu, amax);
    if ((threadIdx.x & 31) == 0 && amax) atomicMax(&s_max, amax);
    __syncthreads();
    int se = 268 - (int)(s_max >> 7);      // scale = 2^(141 - biased exponent): largest -> exponent 14
    se = se < 1 ? 1 : (se > 254 ? 254 : se);
    const float sc = __uint_as_float((uint32_t)se << 23);
    if (threadIdx.x == 0) unscale[m] = __uint_as_float((uint32_t)(254 - se) << 23);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
        const uint4 x = __ldg(src + i);
        const uint32_t v[4] = {x.x, x.y, x.z, x.w};
        uint32_t y[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            y[q] = ptx::pack_f16x2(__uint_as_float(v[q] << 16) * sc, __uint_as_float(v[q] & 0xFFFF0000u) * sc);
        dst[i] = make_uint4(y[0], y[1], y[2], y[3]);
    }
}

}  // namespace

cudaError_t launch_act_to_f16(const void* A, int M, int K, void* out_f16, float* unscale, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(M <= 32 ? 1024 : 256);     // few tokens: latency matters, use the whole SM
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, act_to_f16_kernel, static_cast<const __nv_bfloat16*>(A), static_cast<__half*>(out_f16),
                              unscale, K);
}

}  // namespace nvfp4
