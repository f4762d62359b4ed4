// Source-level drop-in for the reference engine's FP4 operator header.
//
// A translation unit of the reference that includes its own "dense_gemm_fp4.h" and calls
// qwen_thor::ops::invoke_fp4_* (declared at src/engine/dense_gemm_fp4.h:25-72, called from
// src/engine/layer.cu:67-104, :198-215, :406-408, :524-540, :613-615) compiles unchanged against
// this header instead and links libnvfp4_b200.so: same namespace, names, argument order and
// default stream argument, void returns.  The weight descriptor is the reference's own
// qwen_thor::core::QuantizedWeight (src/engine/layer.h:197-204); it is only forward-declared here
// and reinterpreted as the layout-identical C struct nvfp4_quantized_weight, so the reference's
// layer.h keeps defining it.  Errors do not throw (the reference's functions cannot fail
// either): the status of the last call is kept for nvfp4_last_status().
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/nvfp4_b200.h"

namespace qwen_thor {
namespace core { struct QuantizedWeight; }
namespace ops {

namespace nvfp4_detail {
inline const nvfp4_quantized_weight* qw(const core::QuantizedWeight& w) {
    return reinterpret_cast<const nvfp4_quantized_weight*>(&w);
}
}  // namespace nvfp4_detail

inline void invoke_fp4_gemv(const __nv_bfloat16* A, const core::QuantizedWeight& W, __nv_bfloat16* C,
                            cudaStream_t stream = nullptr) {
    nvfp4_invoke_fp4_gemv(A, nvfp4_detail::qw(W), C, stream);
}

inline void invoke_fp4_gemv_add(const __nv_bfloat16* A, const core::QuantizedWeight& W, __nv_bfloat16* C,
                                const __nv_bfloat16* residual, cudaStream_t stream = nullptr) {
    nvfp4_invoke_fp4_gemv_add(A, nvfp4_detail::qw(W), C, residual, stream);
}

inline void invoke_fp4_dual_gemv(const __nv_bfloat16* A, const core::QuantizedWeight& W1,
                                 const core::QuantizedWeight& W2, __nv_bfloat16* C1, __nv_bfloat16* C2,
                                 cudaStream_t stream = nullptr) {
    nvfp4_invoke_fp4_dual_gemv(A, nvfp4_detail::qw(W1), nvfp4_detail::qw(W2), C1, C2, stream);
}

inline void invoke_fp4_gemm(const __nv_bfloat16* A, const core::QuantizedWeight& W, __nv_bfloat16* C, int M,
                            cudaStream_t stream = nullptr) {
    nvfp4_invoke_fp4_gemm(A, nvfp4_detail::qw(W), C, M, stream);
}

inline void invoke_fp4_gemm_add(const __nv_bfloat16* A, const core::QuantizedWeight& W, __nv_bfloat16* D,
                                const __nv_bfloat16* residual, int M, cudaStream_t stream = nullptr) {
    nvfp4_invoke_fp4_gemm_add(A, nvfp4_detail::qw(W), D, residual, M, stream);
}

inline void init_fp4_cublaslt() { nvfp4_init_fp4_cublaslt(); }
inline void cleanup_fp4_cublaslt() { nvfp4_cleanup_fp4_cublaslt(); }

}  // namespace ops
}  // namespace qwen_thor
