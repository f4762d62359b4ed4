/*
 * CPU oracle for the NVFP4 W4A16 linear layer.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a scalar C restatement of the reference engine's algorithm
 * (src/engine/dense_gemm_fp4_sm110.cu, src/engine/light_ops.cu,
 * src/engine/layer.cu).  It is the checker for the CUDA library and the timed
 * CPU baseline; nothing in the shipped library links or calls it.
 *
 * Parity status: the reference holds no golden vector, known-answer test or
 * fixture for this path (its test runner never includes the FP4 header).  The
 * oracle is pinned instead against outputs of the reference's own kernels,
 * compiled from the reference tree into oracle/_ref and run on a B200
 * (tests/golden/reference_b200.npz and the GPU parity tests).
 *
 * All tensors are host pointers.  BF16 values travel as uint16_t bit patterns.
 */
#ifndef NVFP4_ORACLE_H
#define NVFP4_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* E2M1 code (0..15) -> float.  Code 8 is +0.0f.
 * Follows src/engine/dense_gemm_fp4_sm110.cu:24-27. */
float nvfp4_oracle_e2m1(unsigned code);

/* Unsigned E4M3 scale byte -> float: bit 7 ignored, exp==0 -> man*2^-9,
 * else (1+man/8)*2^(exp-7), no NaN (0x7F -> 480).
 * Follows src/engine/dense_gemm_fp4_sm110.cu:30-41. */
float nvfp4_oracle_ue4m3(uint8_t v);

/* float -> BF16 bits, round to nearest even (what __float2bfloat16 does). */
uint16_t nvfp4_oracle_f2bf(float f);
float nvfp4_oracle_bf2f(uint16_t b);

/* float -> E4M3 byte, round to nearest even, subnormals kept, saturating at
 * 448.  Input generation only (the reference never encodes). */
uint8_t nvfp4_oracle_f2e4m3(float f);

/* out[n,k] = bf16( lut[nib] * (ue4m3(scale[n,k/16]) * (1.0f/gs)) ), low nibble
 * = even k.  Follows src/engine/dense_gemm_fp4_sm110.cu:444-467 and :554. */
void nvfp4_oracle_dequant_bf16(const uint8_t* packed, const uint8_t* scale,
                               float global_scale, int N, int K, uint16_t* out);

/* Accumulation semantics of the linear layer. */
enum {
    NVFP4_ORACLE_AUTO = 0,  /* M<=8 -> GEMV semantics, else GEMM semantics (reference :494) */
    NVFP4_ORACLE_GEMV = 1,  /* FP32 group dot x FP32 group scale, lane-strided, xor tree (:96-141, :192-240) */
    NVFP4_ORACLE_GEMM = 2   /* BF16-rounded dequantised weights, FP32 accumulate (:558-583) */
};

/* C[m,n] = bf16( sum_k A[m,k]*W[n,k] (+ residual[m,n]) ), FP32 accumulate, one
 * rounding.  residual may be NULL and may alias C.  rows [n0,n1) only. */
void nvfp4_oracle_linear_rows(const uint16_t* A, int M, const uint8_t* packed,
                              const uint8_t* scale, float global_scale, int N, int K,
                              const uint16_t* residual, uint16_t* C, int mode,
                              int n0, int n1);

void nvfp4_oracle_linear(const uint16_t* A, int M, const uint8_t* packed,
                         const uint8_t* scale, float global_scale, int N, int K,
                         const uint16_t* residual, uint16_t* C, int mode);

/* Same, rows partitioned over `threads` host threads (pthreads). */
void nvfp4_oracle_linear_mt(const uint16_t* A, int M, const uint8_t* packed,
                            const uint8_t* scale, float global_scale, int N, int K,
                            const uint16_t* residual, uint16_t* C, int mode, int threads);

/* out = bf16( silu(gate) * up ), silu(x) = x / (1 + expf(-x)), FP32.
 * Follows src/engine/light_ops.cu:168-199. */
void nvfp4_oracle_swiglu(const uint16_t* gate, const uint16_t* up, size_t n, uint16_t* out);

/* merged is [T, 2*I]: gate = cols [0,I), up = cols [I,2I).  out is [T, I].
 * Follows src/engine/light_ops.cu:1542-1577. */
void nvfp4_oracle_swiglu_merged(const uint16_t* merged, int T, int I, uint16_t* out);

/* C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ) for a BF16 weight: exact BF16 products added in
 * FP32 in k order, residual added in FP32 before the only rounding.  The semantics of the
 * reference's dense GEMV family (invoke_dense_gemv / _add, src/engine/dense_gemm.h:64-95) up to
 * the FP32 summation order. */
void nvfp4_oracle_dense_linear(const uint16_t* A, int M, const uint16_t* W, int N, int K,
                               const uint16_t* residual, uint16_t* C);
/* One token through the reference's BF16 GEMV kernels in their own summation order (lane-strided
 * 8-element chunks, pairwise products, xor-shuffle tree; src/engine/dense_gemm_sm110.cu:544-604,
 * 682-735, 811-1033, 1140-1216).  Pinned bit for bit against those kernels' outputs. */
void nvfp4_oracle_dense_gemv_ref(const uint16_t* A, const uint16_t* W, int N, int K, const uint16_t* residual,
                                 uint16_t* C);


/* RMSNorm with the centred weight, one row per token:
 *   out = bf16( (x * rsqrt(mean(x^2) + eps)) * (1 + w) ), FP32 throughout.
 * Follows rmsnorm_kernel, src/engine/light_ops.cu:65-106, including its summation order (256
 * threads, thread t sums elements t, t+256, ... with fused multiply-adds, then the shuffle-down
 * trees of blockReduceSum, :30-57).  The device's rsqrtf is an approximation; 1/sqrtf stands
 * in for it here, so outputs may differ from the device's in the last BF16 bit of a few elements.
 * K % 256 == 0.  bias != NULL: x = residual + bias first (FP32), and bf16(x) is written back to
 * `residual_out` (fused_add_rmsnorm_kernel, :270-318; the norm uses the unrounded sum). */
void nvfp4_oracle_rmsnorm(const uint16_t* x, const uint16_t* bias, const uint16_t* weight, float eps,
                          int M, int K, uint16_t* out, uint16_t* residual_out);

/* The MLP sequence of src/engine/layer.cu:62-110 with merged gate/up:
 * gate_up linear -> BF16 -> SwiGLU -> BF16 -> down linear (+residual) -> BF16.
 * gate_up weight is [2I, H] (gate rows then up rows), down weight is [H, I]. */
void nvfp4_oracle_mlp(const uint16_t* X, int M, int H, int I,
                      const uint8_t* gu_packed, const uint8_t* gu_scale, float gu_gs,
                      const uint8_t* dn_packed, const uint8_t* dn_scale, float dn_gs,
                      const uint16_t* residual, uint16_t* out, int mode, int threads);

/* Partition-aware tensor-parallel MLP: P ranks, gate/up column-split (rank r
 * owns gate rows and up rows [r*I/P,(r+1)*I/P)), down row-split over K.
 * partial_bf16 != 0: every rank's down partial is rounded to BF16, partials
 * are summed in FP32 in rank order (+ residual), one final rounding.
 * partial_bf16 == 0: partials stay FP32. */
void nvfp4_oracle_tp_mlp(const uint16_t* X, int M, int H, int I, int P,
                         const uint8_t* gu_packed, const uint8_t* gu_scale, float gu_gs,
                         const uint8_t* dn_packed, const uint8_t* dn_scale, float dn_gs,
                         const uint16_t* residual, uint16_t* out, int mode,
                         int partial_bf16, int threads);

/* sqrt(sum (a-b)^2) / sqrt(sum b^2) over BF16 vectors (double accumulation). */
double nvfp4_oracle_rel_frobenius(const uint16_t* a, const uint16_t* b, size_t n);

#ifdef __cplusplus
}
#endif
#endif
