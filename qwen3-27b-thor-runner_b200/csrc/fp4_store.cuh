// Last step of the NVFP4 tensor-core GEMVs' epilogue (decode_fp4.cu, decode_fp4_stream.cu): a thread holds
// the finished FP32 sums of one weight row for every token and stores them.
#pragma once
#include <cuda_bf16.h>

#include "nvfp4_format.cuh"

namespace nvfp4 {

struct Fp4Out {
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    float inv_gs;
    int M, N;
    int out_f32;        // unrounded FP32 sums, no residual
    int swiglu_out;     // weight rows interleaved in slabs of 16 (8 gate rows, their 8 up rows): C is [M, N/2] = bf16(silu(gate) * up)
};

// te: the thread's row within the 128-row tile (= its tensor-memory lane).  Called by whole warps.
template <int KTOK>
__device__ __forceinline__ void fp4_store_rows(const float (&v)[KTOK], const Fp4Out& o, int tile, int te) {
    const int n = tile * 128 + te;
    if (o.swiglu_out) {
        // A gate row and its up row sit 8 lanes apart in one warp.  The projection's outputs are rounded to BF16 as
        // the separate kernels would store them, then silu(gate) * up with one more rounding (the reference's
        // SwiGLU, src/engine/light_ops.cu:186-187).
        const int n_out = tile * 64 + (te >> 4) * 8 + (te & 7);
#pragma unroll
        for (int m = 0; m < KTOK; ++m) {
            if (m >= o.M) continue;
            const float x = __bfloat162float(__float2bfloat16_rn(v[m] * o.inv_gs));
            const float up = __shfl_down_sync(0xffffffffu, x, 8);
            if ((te & 8) == 0 && n < o.N) o.C[(size_t)m * (o.N / 2) + n_out] = __float2bfloat16_rn(silu(x) * up);
        }
        return;
    }
    if (n >= o.N) return;
#pragma unroll
    for (int m = 0; m < KTOK; ++m) {
        if (m >= o.M) continue;
        float x = v[m] * o.inv_gs;
        const size_t at = (size_t)m * o.N + n;
        if (o.out_f32) { reinterpret_cast<float*>(o.C)[at] = x; continue; }
        if (o.residual) x += __bfloat162float(o.residual[at]);
        o.C[at] = __float2bfloat16_rn(x);
    }
}

}  // namespace nvfp4
