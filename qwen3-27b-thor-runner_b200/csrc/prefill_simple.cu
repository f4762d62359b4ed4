// Debug-only BF16 GEMM on CUDA cores: C[M,N] = A[M,K] * Wdq[N,K]^T (+ residual),
// FP32 accumulation, one rounding.  Wdq is a BF16 matrix already produced by the
// dequant kernel in the handle workspace -- the same two-step structure as the
// reference's M>8 path (src/engine/dense_gemm_fp4_sm110.cu:558-583), with this
// plain tiled kernel where the reference calls a library GEMM.  It exists so that
// the tensor-core kernel has an independent device-side cross-check; it is only
// reached through nvfp4_set_option("prefill_impl", 1).
#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"

namespace nvfp4 {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_bf16_simple_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                        const __nv_bfloat16* residual, __nv_bfloat16* C, int M, int N, int K) {
    __shared__ float sA[BK][BM + 1];
    __shared__ float sW[BK][BN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            sA[c][r] = (m < M && k < K) ? __bfloat162float(A[(size_t)m * K + k]) : 0.0f;
            sW[c][r] = (n < N && k < K) ? __bfloat162float(W[(size_t)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = sA[k][ty * 4 + i]; w[i] = sW[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * w[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (residual) v += __bfloat162float(residual[(size_t)m * N + n]);
            C[(size_t)m * N + n] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace

cudaError_t launch_gemm_bf16_simple(const void* A, const void* Wdq, const void* residual, void* C,
                                    int M, int N, int K, cudaStream_t s) {
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_bf16_simple_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(A),
                                                static_cast<const __nv_bfloat16*>(Wdq),
                                                static_cast<const __nv_bfloat16*>(residual),
                                                static_cast<__nv_bfloat16*>(C), M, N, K);
    return cudaGetLastError();
}

}  // namespace nvfp4
