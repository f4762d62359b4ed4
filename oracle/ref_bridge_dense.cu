// C-callable bridge onto the reference engine's BF16 GEMV entry points.
// TEST INFRASTRUCTURE ONLY.  This file holds no reference code: it includes the reference's
// header from the reference tree at build time and forwards plain-C arguments to
// qwen_thor::ops::invoke_dense_gemv / invoke_dense_gemv_add (src/engine/dense_gemm.h:64-95).
// It is linked with the reference's unmodified dense_gemm_sm110.cu into
// oracle/_ref/libref_dense.so; that translation unit also instantiates a CUTLASS GEMM, so the
// build needs a CUTLASS header tree (the reference does not vendor one; the recipe takes the
// tree that ships inside the flashinfer Python package when it is installed).
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include "dense_gemm.h"

extern "C" {

void ref_dense_gemv(const void* A, const void* W, void* C, int N, int K, cudaStream_t s) {
    qwen_thor::ops::invoke_dense_gemv((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, N, K, s);
}

void ref_dense_gemv_add(const void* A, const void* W, void* C, const void* residual, int N, int K, cudaStream_t s) {
    qwen_thor::ops::invoke_dense_gemv_add((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C,
                                          (const __nv_bfloat16*)residual, N, K, s);
}

}  // extern "C"
