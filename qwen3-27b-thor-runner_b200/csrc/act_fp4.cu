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
// (A block far below its token's largest reaches the smallest scale, 2^-9, before its last term: its
// remainder is then at most 2^-11, which is 2^-20 of the token's largest element.)
// All scales are powers of two, so every product and every remainder is exact in FP32.  The term
// rows become columns of the MMA's B operand (tokens x T, padded to a multiple of 16); the GEMV's
// epilogue adds the T columns of a token.
//
// The fusions nvfp4_linear_ex applies to the activations (SwiGLU of a gate/up pair, RMSNorm, a row stride,
// a K padded beyond the tensor) happen here, on the way in.
//
// Outputs: codes [NCp, K/2] (row c = token * 5 + term; two codes per byte, low nibble = even k), the
// block scales in the order the GEMV moves them into tensor memory (see sfb_offset), and 1 / c per token.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fp4_quant.cuh"
#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "ptx.cuh"

namespace nvfp4 {
namespace {

using namespace fp4q;

constexpr int kSliceBlocks = 64;        // 16-element blocks (1024 k) per CTA
constexpr int kPreThreads = 4 * kSliceBlocks;
constexpr int kMaxRowLoads = 4;         // 16-byte loads of the row per thread held in registers at once

// Where the activations come from (the fusions of nvfp4_linear_ex that act on them):
//   kPlain   A itself;
//   kSwiglu  bf16(silu(A) * up): A is the gate half, `up` the up half of a gate/up projection's output
//            (the reference's SwiGLU with its single rounding, src/engine/light_ops.cu:186-187);
//   kNorm    bf16((A / rms(A)) * (1 + w)): the reference's RMSNorm with the centred weight
//            (rmsnorm_kernel, src/engine/light_ops.cu:65-106), the bits the separate kernel would store.
// Columns from k_valid on count as zero and are never read (a K padded beyond the tensor).
enum { kPlain = 0, kSwiglu = 1, kNorm = 2 };

struct ActParams {
    const __nv_bfloat16* A;
    const __nv_bfloat16* up;       // kSwiglu
    const __nv_bfloat16* norm_w;   // kNorm: [K]
    long long a_stride;            // elements between rows of A (and of up)
    int K, k_valid, groups;
    float eps;
    uint8_t* codes;
    uint8_t* sfb;
    float* unscale;
};

__device__ __forceinline__ uint32_t absmax_bf16x8(uint4 x) {
    const uint32_t v[4] = {x.x, x.y, x.z, x.w};
    uint32_t m = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) m = max(m, max(v[q] & 0x7FFFu, (v[q] >> 16) & 0x7FFFu));
    return m;
}

// grid: (K slices, tokens).  Every CTA walks the token's whole row once (cheap, and it saves a grid-wide
// step) for its largest magnitude -- and, for the RMSNorm, its sum of squares, added in a fixed order --
// then expands its own slice: four threads per 16-element block, four elements each (the terms are a
// dependent chain per element, so more threads, not longer ones).  All loads are issued before the first
// use, so the kernel pays one trip to L2.
// Columns beyond tokens x terms are never written: whatever an earlier call left there only reaches
// accumulator columns the GEMV's epilogue does not read (stale codes and scales are finite).
template <int TERMS, int MODE>
__global__ void __launch_bounds__(kPreThreads)
act_to_fp4_kernel(const ActParams p) {
    __shared__ unsigned int s_max;
    __shared__ float s_part[kPreThreads / 32];
    const int m = blockIdx.y;
    const int K = p.K;
    const int blocks = K / 16;
    if (threadIdx.x == 0) s_max = 0u;
    ptx::griddep_launch_dependents();      // the GEMV behind this kernel may set itself up and start streaming weights
    ptx::griddep_wait();                   // A is the output of the kernel before this one
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(p.A + (size_t)m * p.a_stride);
    const uint4* src_up = MODE == kSwiglu ? reinterpret_cast<const uint4*>(p.up + (size_t)m * p.a_stride) : nullptr;
    const int b = blockIdx.x * kSliceBlocks + (threadIdx.x >> 2), part = threadIdx.x & 3;     // block, quarter of it
    const bool live = b < blocks;                          // whole quads are live or not: the shuffles below stay converged
    const bool own_valid = live && b * 16 + part * 4 < p.k_valid;      // k_valid is a multiple of 8: a quarter is valid or not
    uint2 own = make_uint2(0u, 0u), own2 = make_uint2(0u, 0u);
    if (own_valid) {
        own = __ldg(reinterpret_cast<const uint2*>(src + 2 * b) + part);
        if (MODE == kSwiglu) own2 = __ldg(reinterpret_cast<const uint2*>(src_up + 2 * b) + part);
        if (MODE == kNorm) own2 = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint4*>(p.norm_w) + 2 * b) + part);
    }
    unsigned int amax = 0;
    float ss = 0.0f, mt = 0.0f;
    const int chunks = p.k_valid / 8;
    for (int i0 = threadIdx.x; i0 < chunks; i0 += kPreThreads * kMaxRowLoads) {
        uint4 x[kMaxRowLoads], y[kMaxRowLoads];
#pragma unroll
        for (int j = 0; j < kMaxRowLoads; ++j) {
            const int i = i0 + j * kPreThreads;
            x[j] = y[j] = make_uint4(0u, 0u, 0u, 0u);
            if (i < chunks) {
                x[j] = __ldg(src + i);
                if (MODE == kSwiglu) y[j] = __ldg(src_up + i);
                if (MODE == kNorm) y[j] = __ldg(reinterpret_cast<const uint4*>(p.norm_w) + i);
            }
        }
#pragma unroll
        for (int j = 0; j < kMaxRowLoads; ++j) {
            if (MODE == kPlain) amax = max(amax, absmax_bf16x8(x[j]));
            if (MODE == kSwiglu) amax = max(amax, absmax_bf16x8(swiglu_bf16x8(x[j], y[j])));
            if (MODE == kNorm) {
                const uint32_t xv[4] = {x[j].x, x[j].y, x[j].z, x[j].w}, wv[4] = {y[j].x, y[j].y, y[j].z, y[j].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float x0 = __uint_as_float(xv[q] << 16), x1 = __uint_as_float(xv[q] & 0xFFFF0000u);
                    const float w0 = 1.0f + __uint_as_float(wv[q] << 16), w1 = 1.0f + __uint_as_float(wv[q] & 0xFFFF0000u);
                    ss = fmaf(x0, x0, ss);
                    ss = fmaf(x1, x1, ss);
                    mt = fmaxf(mt, fmaxf(fabsf(x0 * w0), fabsf(x1 * w1)));
                }
            }
        }
    }
    float inv_rms = 0.0f;
    if (MODE == kNorm) {
        // the sum of squares in a fixed order: lanes by butterfly, warps one after the other
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
        }
        if ((threadIdx.x & 31) == 0) {
            s_part[threadIdx.x >> 5] = ss;
            atomicMax(&s_max, __float_as_uint(mt));       // non-negative floats order like their bits
        }
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kPreThreads / 32; ++w) tot += s_part[w];
        inv_rms = 1.0f / sqrtf(tot / (float)K + p.eps);
        // the bound of the normalised row, as BF16 magnitude bits rounded up
        const float bound = __uint_as_float(s_max) * inv_rms;
        // an infinity or a NaN anywhere in the row (in x, in its sum of squares) marks the token as non-finite
        amax = (bound < 3.0e38f && tot < 3.0e38f) ? (__float_as_uint(bound) + 0xFFFFu) >> 16 : 0x7F80u;
    } else {
        amax = __reduce_max_sync(0xffffffffu, amax);
        if ((threadIdx.x & 31) == 0 && amax) atomicMax(&s_max, amax);
        __syncthreads();
        amax = s_max;
    }
    const int se = token_scale_exponent(amax);
    const float c = __uint_as_float((uint32_t)se << 23);
    if (blockIdx.x == 0 && threadIdx.x == 0) p.unscale[m] = token_unscale(amax, se);
    float r[4];
    r[0] = __uint_as_float(own.x << 16);
    r[1] = __uint_as_float(own.x & 0xFFFF0000u);
    r[2] = __uint_as_float(own.y << 16);
    r[3] = __uint_as_float(own.y & 0xFFFF0000u);
    if (MODE != kPlain) {
        const float o[4] = {__uint_as_float(own2.x << 16), __uint_as_float(own2.x & 0xFFFF0000u),
                            __uint_as_float(own2.y << 16), __uint_as_float(own2.y & 0xFFFF0000u)};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float y = MODE == kSwiglu ? silu(r[q]) * o[q] : r[q] * inv_rms * (1.0f + o[q]);
            r[q] = own_valid ? __bfloat162float(__float2bfloat16_rn(y)) : 0.0f;      // the one rounding of the separate kernel
        }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) r[q] *= c;
    float bmax = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
    if (live) {
        const int p0 = first_term_exponent(bmax);
#pragma unroll
        for (int t = 0; t < TERMS; ++t) {
            const int pw = term_exponent(p0, t);
            const uint32_t w = take_term(r, pw);
            const int col = m * TERMS + t;
            *reinterpret_cast<uint16_t*>(p.codes + (size_t)col * (K / 2) + (size_t)b * 8 + part * 2) = (uint16_t)w;
            if (part == 0) p.sfb[fp4::sfb_offset(b, col, p.groups)] = (uint8_t)ue4m3_pow2(pw);
        }
    }
}

template <int TERMS>
cudaError_t launch_mode(const cudaLaunchConfig_t& cfg, int mode, const ActParams& p) {
    if (mode == kSwiglu) return cudaLaunchKernelEx(&cfg, act_to_fp4_kernel<TERMS, kSwiglu>, p);
    if (mode == kNorm) return cudaLaunchKernelEx(&cfg, act_to_fp4_kernel<TERMS, kNorm>, p);
    return cudaLaunchKernelEx(&cfg, act_to_fp4_kernel<TERMS, kPlain>, p);
}

}  // namespace

bool act_to_fp4_supported(const LinearArgs& a) {
    if (a.swiglu_up && a.norm_w) return false;
    if (a.norm_w && a.k_valid && a.k_valid != a.K) return false;
    if (a.k_valid && (a.k_valid < 0 || a.k_valid > a.K || (a.k_valid & 7))) return false;
    if (a.a_stride && (a.a_stride & 7)) return false;                  // rows must stay 16-byte aligned
    if (reinterpret_cast<uintptr_t>(a.A) & 15u) return false;
    if (a.swiglu_up && (reinterpret_cast<uintptr_t>(a.swiglu_up) & 15u)) return false;
    if (a.norm_w && (reinterpret_cast<uintptr_t>(a.norm_w) & 15u)) return false;
    return true;
}

cudaError_t launch_act_to_fp4(const LinearArgs& a, int terms, int groups, void* codes, void* sfb, float* unscale, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((a.K / 16 + kSliceBlocks - 1) / kSliceBlocks, a.M);
    cfg.blockDim = dim3(kPreThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ActParams p{};
    p.A = static_cast<const __nv_bfloat16*>(a.A);
    p.up = static_cast<const __nv_bfloat16*>(a.swiglu_up);
    p.norm_w = static_cast<const __nv_bfloat16*>(a.norm_w);
    p.a_stride = a.a_stride ? a.a_stride : a.K;
    p.K = a.K;
    p.k_valid = a.k_valid ? a.k_valid : a.K;
    p.groups = groups;
    p.eps = a.norm_eps;
    p.codes = static_cast<uint8_t*>(codes);
    p.sfb = static_cast<uint8_t*>(sfb);
    p.unscale = unscale;
    const int mode = a.swiglu_up ? kSwiglu : (a.norm_w ? kNorm : kPlain);
    if (terms == 6) return launch_mode<6>(cfg, mode, p);
    if (terms == 5) return launch_mode<5>(cfg, mode, p);
    return cudaErrorInvalidValue;
}

}  // namespace nvfp4
