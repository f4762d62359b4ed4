// Last step of the NVFP4 tensor-core GEMVs' epilogue (decode_fp4.cu, decode_fp4_stream.cu): a thread holds
// the finished FP32 sums of one weight row for every token and stores them.
#pragma once
#include <cuda_bf16.h>

#include "nvfp4_format.cuh"
#include "ptx.cuh"

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

// Requests the pairs of CN CTAs x TN tokens together (CN x TN loads in flight, one trip to L2), asks again until
// all carry this launch's tag, then adds them to v in CTA order per token.  Bounded; false after the budget.
template <int KTOK, int CN, int TN>
__device__ __forceinline__ bool fp4_gather_block(float (&v)[KTOK], const unsigned char* pairs, size_t slot_bytes, int c0, int last,
                                                 int M, int te, unsigned int tag, long long t0, volatile int* abort_flag,
                                                 unsigned int* status, unsigned int code) {
#pragma unroll
    for (int mb = 0; mb < KTOK; mb += TN) {
        if (mb >= M) continue;
        while (true) {
            uint2 x[CN][TN];
#pragma unroll
            for (int ci = 0; ci < CN; ++ci)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    x[ci][j] = make_uint2(0u, tag);
                    if (mb + j < KTOK && mb + j < M && c0 + ci <= last)
                        x[ci][j] = ptx::ld_volatile_v2(pairs + (size_t)(c0 + ci) * slot_bytes + ((mb + j) * 128 + te) * 8);
                }
            bool ready = true;
#pragma unroll
            for (int ci = 0; ci < CN; ++ci)
#pragma unroll
                for (int j = 0; j < TN; ++j) ready &= (x[ci][j].y == tag);
            if (ready) {
#pragma unroll
                for (int ci = 0; ci < CN; ++ci)
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        if (mb + j < KTOK && mb + j < M && c0 + ci <= last) v[mb + j] += __uint_as_float(x[ci][j].x);
                break;
            }
            if (*abort_flag || clock64() - t0 > ptx::kWaitBudgetClocks) {
                *abort_flag = 1;
                atomicCAS(status, 0u, code);
                return false;
            }
        }
    }
    return true;
}

// Adds to v the FP32 partial sums the CTAs first .. last published for this row tile as {value, launch tag}
// pairs ([CTA][token][128 rows] x 8 bytes, slot_bytes per CTA), in CTA order per token (a fixed summation
// order).  Sixteen loads travel together: one contributor's tokens sixteen at a time, or, when the tile is
// split over more CTAs, four contributors x four tokens -- a tile split over five CTAs costs the owner one or
// two round trips, not one per contributor and token group (3 us on the deep down projection at 16 tokens).
template <int KTOK>
__device__ __forceinline__ bool fp4_gather_pairs(float (&v)[KTOK], const unsigned char* pairs, size_t slot_bytes, int first, int last,
                                                 int M, int te, unsigned int tag, volatile int* abort_flag, unsigned int* status,
                                                 unsigned int code) {
    const long long t0 = clock64();
    if (last == first) return fp4_gather_block<KTOK, 1, 16>(v, pairs, slot_bytes, first, last, M, te, tag, t0, abort_flag, status, code);
    for (int c0 = first; c0 <= last; c0 += 4)
        if (!fp4_gather_block<KTOK, 4, 4>(v, pairs, slot_bytes, c0, last, M, te, tag, t0, abort_flag, status, code)) return false;
    return true;
}

}  // namespace nvfp4
