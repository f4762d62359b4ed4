// Test driver: the reference engine's decode/prefill MLP sequence (run_mlp, src/engine/layer.cu:62-110)
// written against the reference's own operator names and compiled against the shim header instead
// of the reference's dense_gemm_fp4.h:
//     invoke_fp4_gemm(x, gate_up)  ->  SwiGLU on the merged tensor  ->  invoke_fp4_gemm_add(act, down, hidden, hidden)
// and, for one token, the GEMV forms invoke_fp4_gemv / invoke_fp4_gemv_add.  Inputs come from a
// file written by the Python test, the output goes back to a file; the test compares it with the
// CPU oracle.  With -DNVFP4_TEST_REF_LAYER_H the weight descriptor is the reference's own struct
// from its layer.h; otherwise a layout-identical stand-in (the reference tree is not always there).
//
// File layout (little endian): int32 M, H, I; float gs_gu, gs_dn; then X [M,H] bf16, R [M,H] bf16,
// gate_up packed [2I, H/2], gate_up scale [2I, H/16], down packed [H, I/2], down scale [H, I/16].
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#ifdef NVFP4_TEST_REF_LAYER_H
#include "layer.h"
#else
namespace qwen_thor { namespace core {
struct QuantizedWeight {
    uint8_t* packed = nullptr;
    uint8_t* scale = nullptr;
    float global_scale = 1.0f;
    float input_scale = 1.0f;
    int N = 0, K = 0;
};
}}
#endif
#include "nvfp4_qwen_thor_shim.hpp"

static_assert(sizeof(qwen_thor::core::QuantizedWeight) == sizeof(nvfp4_quantized_weight), "descriptor layout");

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 10; } } while (0)

template <class T>
static T* to_device(const std::vector<uint8_t>& blob, size_t& off, size_t bytes) {
    void* d = nullptr;
    if (cudaMalloc(&d, bytes) != cudaSuccess) return nullptr;
    if (cudaMemcpy(d, blob.data() + off, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    off += bytes;
    return static_cast<T*>(d);
}

int main(int argc, char** argv) {
    if (argc != 3) return 2;
    std::FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 3;
    std::fseek(f, 0, SEEK_END);
    const long size = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> blob((size_t)size);
    if (std::fread(blob.data(), 1, blob.size(), f) != blob.size()) return 3;
    std::fclose(f);
    const int32_t* hdr = reinterpret_cast<const int32_t*>(blob.data());
    const int M = hdr[0], H = hdr[1], I = hdr[2];
    const float gs_gu = reinterpret_cast<const float*>(blob.data())[3], gs_dn = reinterpret_cast<const float*>(blob.data())[4];
    size_t off = 20;
    const size_t xb = (size_t)M * H * 2;
    __nv_bfloat16* x = to_device<__nv_bfloat16>(blob, off, xb);
    __nv_bfloat16* hidden = to_device<__nv_bfloat16>(blob, off, xb);          // the residual stream, updated in place
    qwen_thor::core::QuantizedWeight gate_up, down;
    gate_up.packed = to_device<uint8_t>(blob, off, (size_t)2 * I * H / 2);
    gate_up.scale = to_device<uint8_t>(blob, off, (size_t)2 * I * H / 16);
    gate_up.global_scale = gs_gu; gate_up.N = 2 * I; gate_up.K = H;
    down.packed = to_device<uint8_t>(blob, off, (size_t)H * I / 2);
    down.scale = to_device<uint8_t>(blob, off, (size_t)H * I / 16);
    down.global_scale = gs_dn; down.N = H; down.K = I;
    if (!x || !hidden || !gate_up.packed || !gate_up.scale || !down.packed || !down.scale || off != blob.size()) return 4;
    __nv_bfloat16 *gu = nullptr, *act = nullptr;
    CK(cudaMalloc(&gu, (size_t)M * 2 * I * 2));
    CK(cudaMalloc(&act, (size_t)M * I * 2));
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    nvfp4_handle* h = nullptr;                                               // for the SwiGLU between the two projections
    if (nvfp4_create(0, 0, &h) != NVFP4_OK) return 5;

    using namespace qwen_thor::ops;
    init_fp4_cublaslt();
    if (M == 1) {
        invoke_fp4_gemv(x, gate_up, gu, stream);
        if (nvfp4_last_status()) return 6;
        if (nvfp4_swiglu(h, gu, nullptr, 1, I, act, stream)) return 7;
        invoke_fp4_gemv_add(act, down, hidden, hidden, stream);
    } else {
        invoke_fp4_gemm(x, gate_up, gu, M, stream);
        if (nvfp4_last_status()) return 6;
        if (nvfp4_swiglu(h, gu, nullptr, M, I, act, stream)) return 7;
        invoke_fp4_gemm_add(act, down, hidden, hidden, M, stream);
    }
    if (nvfp4_last_status()) return 8;
    CK(cudaStreamSynchronize(stream));
    std::vector<uint8_t> out(xb);
    CK(cudaMemcpy(out.data(), hidden, xb, cudaMemcpyDeviceToHost));
    cleanup_fp4_cublaslt();
    nvfp4_destroy(h);
    f = std::fopen(argv[2], "wb");
    if (!f || std::fwrite(out.data(), 1, out.size(), f) != out.size()) return 9;
    std::fclose(f);
    return 0;
}
