// Host side of the C ABI: handle lifecycle, argument validation, kernel selection
// and the reference-shaped entry points.  No call here allocates, frees or
// synchronises after nvfp4_create (two excepted, both by contract: nvfp4_linear_host, the
// host-buffer convenience path, and nvfp4_scan_scales, a load-time check that returns a count).
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "nvfp4_internal.h"

using namespace nvfp4;

struct nvfp4_handle {
    nvfp4_device_info dev{};
    char* workspace = nullptr;
    size_t workspace_bytes = 0;
    int decode_impl = 0;
    int prefill_impl = 0;
    int decode_max_m = 16;
    int wide_gemv = 1;                           // 9..16 tokens: one launch of the wide GEMV kernel
    int skinny_min_m = 9, skinny_max_m = 64;     // token counts routed to the weights-in-TMEM kernel
    int fp4_native = 1;                          // the NVFP4 tensor-core GEMV (weights untouched, activations as NVFP4 terms) ...
    int fp4_min_m = 1;                           // ... from this token count on (up to 16)
    int fp4_stream_min_m = 10;                   // from this token count on its activations travel through the ring (decode_fp4_stream.cu)
    int gemm_weight_rounding = 0;                // above 8 tokens: the reference's BF16-rounded weights (its GEMM branch)
    unsigned long long launches = 0;
    int host_direct_out = 1;                     // nvfp4_linear_host: kernels store into a pinned, device-mapped C_host themselves
    const void* host_out_seen = nullptr;         // the last C_host looked up, and its device address (null: not pinned)
    void* host_out_dev = nullptr;
    // scale tensors in which nvfp4_scan_scales found a byte 0x7F / 0xFF: the tensor core reads those as NaN, so
    // these weights stay on the kernels that decode the scale themselves
    std::vector<const void*> nan_scales;
    bool has_nan_scales(const void* scale) const {
        if (nan_scales.empty()) return false;
        return std::find(nan_scales.begin(), nan_scales.end(), scale) != nan_scales.end();
    }
};

#include <atomic>

namespace nvfp4 {
unsigned int next_launch_tag() {
    static std::atomic<unsigned int> counter{0u};
    unsigned int t = counter.fetch_add(1u, std::memory_order_relaxed) + 1u;
    if (t == 0u) t = counter.fetch_add(1u, std::memory_order_relaxed) + 1u;
    return t;
}
}  // namespace nvfp4

namespace {

// status word + the split-tile partial pairs of the GEMV kernels: the wide one from 16 KB, the 8-token one from 6 MB
// (1.2 MB), the tensor-core one from 7.25 MB (2.5 MB), and from 10 MB the NVFP4 form of that kernel's activations
constexpr size_t kDecodeScratchBytes = 12u << 20;
constexpr size_t kFp4PairsOffset = 29u << 18, kFp4ActOffset = 10u << 20, kFp4ActBytes = 2u << 20;
static_assert(kFp4PairsOffset + nvfp4::fp4::kPairBytes <= kFp4ActOffset, "scratch layout");

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_scale(float gs) {
    if (!(gs > 0.0f) || !std::isfinite(gs)) return NVFP4_E_SCALE;
    return NVFP4_OK;
}

int validate_linear(const nvfp4_handle* h, const void* A, int M, const uint8_t* packed, const uint8_t* scale,
                    float gs, int N, int K, const void* residual, const void* C, int c_cols = 0) {
    if (!h || !A || !packed || !scale || !C) return NVFP4_E_NULL;
    if (M < 0 || N <= 0 || K <= 0 || (K & 15) != 0) return NVFP4_E_SHAPE;
    if ((long long)N * K / 2 > (1LL << 40)) return NVFP4_E_SHAPE;
    if (int e = check_scale(gs)) return e;
    if (!aligned16(A) || !aligned16(C) || (residual && !aligned16(residual))) return NVFP4_E_ALIGN;
    if ((reinterpret_cast<uintptr_t>(packed) & 7u) != 0) return NVFP4_E_ALIGN;
    // A must not overlap the output (the reference has the same unstated rule:
    // every block re-reads A while others already store C).
    const char* a0 = static_cast<const char*>(A);
    const char* a1 = a0 + (size_t)M * K * 2;
    const char* c0 = static_cast<const char*>(C);
    const char* c1 = c0 + (size_t)M * (c_cols ? c_cols : N) * 2;
    if (M > 0 && a0 < c1 && c0 < a1) return NVFP4_E_ALIAS;
    return NVFP4_OK;
}

int cuda_status(cudaError_t e) { return e == cudaSuccess ? NVFP4_OK : (int)e; }

// options only the mma.sync GEMV kernels implement (the tensor-core GEMV takes plain calls, with or without FP32 output)
// One linear call on device buffers.
// `ws_bytes`: how much of the workspace the kernels may use (the host-buffer path keeps its staging behind it).
int run_linear(nvfp4_handle* h, const LinearArgs& a, cudaStream_t s, size_t ws_bytes = 0) {
    if (a.M == 0) return NVFP4_OK;
    if (ws_bytes == 0) ws_bytes = h->workspace_bytes;
    const bool fast_path_wanted = a.M <= h->decode_max_m ? h->decode_impl != 1 : h->prefill_impl != 1;
    const bool wide_ok = fast_path_wanted && h->wide_gemv && decode_wide_supported(a) &&
                         kDecodeScratchBytes + prefill_umma_scratch_bytes(17, a.N, a.K) <= ws_bytes &&
                         decode_wide_scratch_bytes(h->dev.sm_count) <= h->dev.gemv_pairs_offset;
    // options only the GEMV kernels implement (the SwiGLU epilogue and the group reduction exist in the wide one too)
    const bool other_options = a.out_f32 || a.swiglu_up || a.a_stride || a.k_valid || a.norm_w;
    if (h->gemm_weight_rounding && a.M > 8 && !a.out_f32 && !a.px && !a.swiglu_up && !a.a_stride && !a.k_valid && !a.norm_w &&
        !a.swiglu_out) {
        // The reference's own arithmetic above 8 tokens, for a caller who wants ITS bits rather than exact weights.
        if (h->prefill_impl == 1 || !prefill_umma_supported(a)) return NVFP4_E_LIMIT;
        if (kDecodeScratchBytes + prefill_umma_scratch_bytes(a.M, a.N, a.K) > ws_bytes) return NVFP4_E_WORKSPACE;
        LinearArgs r = a;
        r.round_weights = true;
        int nl = 0;
        cudaError_t e = launch_prefill_umma(r, h->dev, h->workspace, ws_bytes, kDecodeScratchBytes, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    if (a.out_f32 && a.M > 16) {
        // unrounded FP32 sums beyond the GEMV kernels: the 128-token-tile tcgen05 kernel's FP32 epilogue
        if (a.swiglu_up || a.a_stride || a.k_valid || a.norm_w || a.px || a.swiglu_out) return NVFP4_E_LIMIT;
        if (h->prefill_impl == 1 || !prefill_umma_supported(a)) return NVFP4_E_LIMIT;
        if (kDecodeScratchBytes + prefill_umma_scratch_bytes(a.M, a.N, a.K) > ws_bytes) return NVFP4_E_WORKSPACE;
        int nl = 0;
        cudaError_t e = launch_prefill_umma(a, h->dev, h->workspace, ws_bytes, kDecodeScratchBytes, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    if (a.swiglu_out && !other_options && !a.px && a.M > 16) {
        // beyond the GEMV kernels only the 128-token-tile tcgen05 kernel has the SwiGLU epilogue
        if (h->prefill_impl == 1 || !prefill_umma_supported(a)) return NVFP4_E_LIMIT;
        if (kDecodeScratchBytes + prefill_umma_scratch_bytes(a.M, a.N, a.K) > ws_bytes) return NVFP4_E_WORKSPACE;
        int nl = 0;
        cudaError_t e = launch_prefill_umma(a, h->dev, h->workspace, ws_bytes, kDecodeScratchBytes, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    const bool fp4_wanted = a.M <= h->decode_max_m &&
                            (h->decode_impl == 3 || (h->decode_impl == 0 && h->fp4_native && a.M >= h->fp4_min_m));
    if (fp4_wanted && !a.px && decode_fp4_scratch_bytes(a.K) <= kFp4ActBytes && kDecodeScratchBytes <= ws_bytes &&
        !h->has_nan_scales(a.scale)) {
        // up to 9 tokens with the activations resident beside the ring, else streamed through it
        // Resident activations win on few tokens and wherever a CTA's share of the weights is short (qkv, o: 0.7-1.0 us
        // per call); from seven tokens on with a long share (gate_up, down) the streamed form's larger ring of weights
        // wins (gate_up at 8 tokens 23.4 against 25.2 us).  At four to six tokens the streamed form is 0.4 us ahead
        // call by call but 2 us per layer behind in a 64-layer sequence of distinct weights, so it is not taken there.
        // A threshold set by the caller is taken as it is.
        bool want_stream = a.M >= h->fp4_stream_min_m;
        if (h->fp4_stream_min_m == 10 && a.M >= 7 && !a.packed2) {
            const long long units = (long long)((a.N + 127) / 128) * (a.K / 256);
            const long long ctas = units < h->dev.sm_count ? units : h->dev.sm_count;
            if (ctas > 0 && (units + ctas - 1) / ctas >= 12) want_stream = true;
        }
        if (want_stream && !decode_fp4_stream_supported(a, h->dev)) want_stream = false;
        const bool res = !want_stream && decode_fp4_supported(a, h->dev);
        if (res || decode_fp4_stream_supported(a, h->dev)) {
            int nl = 0;
            cudaError_t e = res ? launch_decode_fp4(a, h->dev, h->workspace, kFp4PairsOffset, h->workspace + kFp4ActOffset, &nl, s)
                                : launch_decode_fp4_stream(a, h->dev, h->workspace, kFp4PairsOffset, h->workspace + kFp4ActOffset, &nl, s);
            h->launches += (unsigned long long)nl;
            return cuda_status(e);
        }
    }
    if (other_options || ((a.swiglu_out || a.px) && !wide_ok)) {
        if (a.M > 16 || !decode_mma_supported(a) || !decode_mma_fits(a, h->dev)) return NVFP4_E_LIMIT;
        int nl = 0;
        cudaError_t e = launch_decode_mma(a, h->dev, h->workspace, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    if (wide_ok) {
        // the FP16 activation copy and the per-token factors sit where the prefill kernel keeps its own
        char* base = h->workspace + kDecodeScratchBytes + prefill_umma_reserved_bytes();
        float* unscale = reinterpret_cast<float*>(base + ((size_t)a.M * a.K * 2 + 255) / 256 * 256);
        int nl = 0;
        cudaError_t e = launch_decode_wide(a, h->dev, h->workspace, base, unscale, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    if (fast_path_wanted && a.M >= h->skinny_min_m && a.M <= h->skinny_max_m && skinny_umma_supported(a) &&
        kDecodeScratchBytes + prefill_umma_reserved_bytes() <= ws_bytes) {
        int nl = 0;
        cudaError_t e = launch_skinny_umma(a, h->dev, h->workspace, ws_bytes, kDecodeScratchBytes, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    if (a.M <= h->decode_max_m) {
        int impl = h->decode_impl;
        const bool fast_ok = decode_mma_supported(a) && decode_mma_fits(a, h->dev);
        if (impl == 0 || impl == 3) impl = fast_ok ? 2 : 1;
        if (impl == 2) {
            if (!fast_ok) return NVFP4_E_SHAPE;
            size_t need = decode_mma_scratch_bytes(a, h->dev);
            if (need > ws_bytes) return NVFP4_E_WORKSPACE;
            int nl = 0;
            cudaError_t e = launch_decode_mma(a, h->dev, h->workspace, &nl, s);
            h->launches += (unsigned long long)nl;
            return cuda_status(e);
        }
        // Scalar path: at most 16 tokens per launch.
        for (int m0 = 0; m0 < a.M; m0 += 16) {
            LinearArgs b = a;
            b.M = (a.M - m0 < 16) ? a.M - m0 : 16;
            b.A = static_cast<const char*>(a.A) + (size_t)m0 * a.K * 2;
            b.C = static_cast<char*>(a.C) + (size_t)m0 * a.N * 2;
            if (a.residual) b.residual = static_cast<const char*>(a.residual) + (size_t)m0 * a.N * 2;
            cudaError_t e = launch_decode_simple(b, s);
            h->launches += 1;
            if (e != cudaSuccess) return (int)e;
        }
        return NVFP4_OK;
    }
    int impl = h->prefill_impl;
    if (impl == 0) impl = prefill_umma_supported(a) ? 2 : 1;
    if (impl == 2) {
        if (!prefill_umma_supported(a)) return NVFP4_E_SHAPE;
        if (kDecodeScratchBytes + prefill_umma_scratch_bytes(a.M, a.N, a.K) > ws_bytes) return NVFP4_E_WORKSPACE;
        int nl = 0;
        cudaError_t e = launch_prefill_umma(a, h->dev, h->workspace, ws_bytes, kDecodeScratchBytes, &nl, s);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    // Debug path: dequantise the whole weight into the workspace, then a CUDA-core GEMM.
    // The matrix goes behind the status word, flags and partial tiles of the fast kernels.
    const size_t skip = kDecodeScratchBytes + prefill_umma_reserved_bytes();
    const size_t need = (size_t)a.N * a.K * 2;
    if (skip + need > ws_bytes) return NVFP4_E_WORKSPACE;
    cudaError_t e = launch_dequant_bf16(a.packed, a.scale, a.inv_gs, a.N, a.K, h->workspace + skip, s);
    h->launches += 1;
    if (e != cudaSuccess) return (int)e;
    e = launch_gemm_bf16_simple(a.A, h->workspace + skip, a.residual, a.C, a.M, a.N, a.K, s);
    h->launches += 1;
    return cuda_status(e);
}

}  // namespace

extern "C" {

const char* nvfp4_status_string(int status) {
    switch (status) {
        case NVFP4_OK: return "ok";
        case NVFP4_E_NULL: return "null pointer argument";
        case NVFP4_E_SHAPE: return "unsupported shape (need M>=0, N>0, K>0, K % 16 == 0)";
        case NVFP4_E_ALIGN: return "misaligned pointer (A, C, residual: 16 bytes; packed: 8 bytes)";
        case NVFP4_E_WORKSPACE: return "handle workspace too small for this call";
        case NVFP4_E_ALIAS: return "A overlaps the output";
        case NVFP4_E_SCALE: return "global_scale must be finite and > 0";
        case NVFP4_E_DEVICE: return "no usable CUDA device (compute capability 10.x required)";
        case NVFP4_E_OPTION: return "unknown option or value";
        case NVFP4_E_TP: return "tensor-parallel set-up error";
        case NVFP4_E_LIMIT:
            return "beyond the fixed maximum of the allocation-free GEMV (need M <= 16, K % 256 == 0, activations of 8 "
                   "tokens fitting in shared memory)";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

int nvfp4_workspace_bytes(int max_M, int max_N, int max_K, size_t* bytes) {
    if (!bytes) return NVFP4_E_NULL;
    if (max_M < 0 || max_N <= 0 || max_K <= 0) return NVFP4_E_SHAPE;
    // GEMV scratch + host-convenience staging (A, residual, C) + prefill scratch.
    size_t staging = ((size_t)max_M * max_K * 2 + 255) / 256 * 256 + 2 * (((size_t)max_M * max_N * 2 + 255) / 256 * 256);
    *bytes = kDecodeScratchBytes + staging + prefill_umma_scratch_bytes(max_M, max_N, max_K);
    return NVFP4_OK;
}

int nvfp4_create(int device, size_t workspace_bytes, nvfp4_handle** out) {
    if (!out) return NVFP4_E_NULL;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        (void)cudaGetLastError();
        return NVFP4_E_DEVICE;
    }
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return NVFP4_E_DEVICE;
    if (prop.major != 10) return NVFP4_E_DEVICE;   // the kernels are built for sm_100a only
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return (int)e;
    nvfp4_handle* h = new nvfp4_handle();
    h->dev.device = device;
    h->dev.sm_count = prop.multiProcessorCount;
    h->dev.cc_major = prop.major;
    h->dev.cc_minor = prop.minor;
    h->dev.smem_optin = prop.sharedMemPerBlockOptin;
    if (workspace_bytes < kDecodeScratchBytes) workspace_bytes = kDecodeScratchBytes;
    workspace_bytes &= ~(size_t)255;     // everything carved out of the workspace, from either end, stays 256-byte aligned
    e = cudaMalloc(&h->workspace, workspace_bytes);
    if (e == cudaSuccess) e = cudaMemset(h->workspace, 0, workspace_bytes);
    if (e == cudaSuccess) e = configure_kernels(h->dev);
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        if (h->workspace) cudaFree(h->workspace);
        delete h;
        return (int)e;
    }
    h->workspace_bytes = workspace_bytes;
    h->dev.maps = new TensorMapCache();
    *out = h;
    return NVFP4_OK;
}

int nvfp4_destroy(nvfp4_handle* h) {
    if (!h) return NVFP4_E_NULL;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(h->dev.device);
    cudaError_t e = cudaFree(h->workspace);
    cudaSetDevice(prev);
    delete h->dev.maps;
    delete h;
    return cuda_status(e);
}

int nvfp4_set_option(nvfp4_handle* h, const char* name, int value) {
    if (!h || !name) return NVFP4_E_NULL;
    if (!std::strcmp(name, "decode_impl")) {
        if (value < 0 || value > 3) return NVFP4_E_OPTION;
        h->decode_impl = value;
    } else if (!std::strcmp(name, "prefill_impl")) {
        if (value < 0 || value > 2) return NVFP4_E_OPTION;
        h->prefill_impl = value;
    } else if (!std::strcmp(name, "decode_max_m")) {
        if (value < 0 || value > 16) return NVFP4_E_OPTION;
        h->decode_max_m = value;
    } else if (!std::strcmp(name, "wide_gemv")) {
        if (value < 0 || value > 1) return NVFP4_E_OPTION;
        h->wide_gemv = value;
    } else if (!std::strcmp(name, "fp4_native")) {
        if (value < 0 || value > 1) return NVFP4_E_OPTION;
        h->fp4_native = value;
    } else if (!std::strcmp(name, "fp4_min_m")) {
        if (value < 1 || value > 16) return NVFP4_E_OPTION;
        h->fp4_min_m = value;
    } else if (!std::strcmp(name, "host_direct_out")) {
        if (value < 0 || value > 1) return NVFP4_E_OPTION;
        h->host_direct_out = value;
    } else if (!std::strcmp(name, "fp4_stream_min_m")) {
        if (value < 1 || value > 17) return NVFP4_E_OPTION;
        h->fp4_stream_min_m = value;
    } else if (!std::strcmp(name, "gemm_weight_rounding")) {
        if (value < 0 || value > 1) return NVFP4_E_OPTION;
        h->gemm_weight_rounding = value;
    } else if (!std::strcmp(name, "fp4_own_quant")) {
        if (value < 0 || value > 1) return NVFP4_E_OPTION;
        h->dev.fp4_own_quant = value;
    } else if (!std::strcmp(name, "skinny_min_m")) {
        if (value < 1 || value > 129) return NVFP4_E_OPTION;
        h->skinny_min_m = value;
    } else if (!std::strcmp(name, "skinny_max_m")) {
        if (value < 0 || value > 128) return NVFP4_E_OPTION;
        h->skinny_max_m = value;
    } else if (!std::strcmp(name, "skinny_split_cost")) {
        if (value < 0 || value > 1000) return NVFP4_E_OPTION;
        h->dev.skinny_split_cost = value;
    } else if (!std::strcmp(name, "prefill_stream_k")) {
        if (value < 0 || value > 1) return NVFP4_E_OPTION;
        h->dev.prefill_stream_k = value;
    } else {
        return NVFP4_E_OPTION;
    }
    return NVFP4_OK;
}

int nvfp4_get_option(nvfp4_handle* h, const char* name, int* value) {
    if (!h || !name || !value) return NVFP4_E_NULL;
    if (!std::strcmp(name, "decode_impl")) *value = h->decode_impl;
    else if (!std::strcmp(name, "prefill_impl")) *value = h->prefill_impl;
    else if (!std::strcmp(name, "decode_max_m")) *value = h->decode_max_m;
    else if (!std::strcmp(name, "prefill_stream_k")) *value = h->dev.prefill_stream_k;
    else if (!std::strcmp(name, "wide_gemv")) *value = h->wide_gemv;
    else if (!std::strcmp(name, "fp4_native")) *value = h->fp4_native;
    else if (!std::strcmp(name, "fp4_min_m")) *value = h->fp4_min_m;
    else if (!std::strcmp(name, "fp4_own_quant")) *value = h->dev.fp4_own_quant;
    else if (!std::strcmp(name, "gemm_weight_rounding")) *value = h->gemm_weight_rounding;
    else if (!std::strcmp(name, "fp4_stream_min_m")) *value = h->fp4_stream_min_m;
    else if (!std::strcmp(name, "host_direct_out")) *value = h->host_direct_out;
    else if (!std::strcmp(name, "skinny_min_m")) *value = h->skinny_min_m;
    else if (!std::strcmp(name, "skinny_max_m")) *value = h->skinny_max_m;
    else if (!std::strcmp(name, "skinny_split_cost")) *value = h->dev.skinny_split_cost;
    else if (!std::strcmp(name, "sm_count")) *value = h->dev.sm_count;
    else return NVFP4_E_OPTION;
    return NVFP4_OK;
}

int nvfp4_device_status(nvfp4_handle* h, unsigned int* status) {
    if (!h || !status) return NVFP4_E_NULL;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(h->dev.device);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(status, h->workspace, sizeof(unsigned int), cudaMemcpyDeviceToHost);
    cudaSetDevice(prev);
    return cuda_status(e);
}

int nvfp4_launch_count(nvfp4_handle* h, unsigned long long* count) {
    if (!h || !count) return NVFP4_E_NULL;
    *count = h->launches;
    return NVFP4_OK;
}

int nvfp4_linear(nvfp4_handle* h, const void* A, int M, const uint8_t* packed, const uint8_t* scale,
                 float global_scale, int N, int K, const void* residual, void* C, nvfp4_stream_t stream) {
    if (int e = validate_linear(h, A, M, packed, scale, global_scale, N, K, residual, C)) return e;
    LinearArgs a{A, packed, scale, 1.0f / global_scale, residual, C, M, N, K};
    return run_linear(h, a, stream);
}

int nvfp4_linear_f32(nvfp4_handle* h, const void* A, int M, const uint8_t* packed, const uint8_t* scale,
                     float global_scale, int N, int K, void* C_f32, nvfp4_stream_t stream) {
    if (int e = validate_linear(h, A, M, packed, scale, global_scale, N, K, nullptr, C_f32)) return e;
    if (M == 0) return NVFP4_OK;
    {   // the output is twice as large as the BF16 one validate_linear assumed
        const char* a0 = static_cast<const char*>(A);
        const char* c0 = static_cast<const char*>(C_f32);
        if (a0 < c0 + (size_t)M * N * 4 && c0 < a0 + (size_t)M * K * 2) return NVFP4_E_ALIAS;
    }
    LinearArgs a{A, packed, scale, 1.0f / global_scale, nullptr, C_f32, M, N, K};
    a.out_f32 = true;
    return run_linear(h, a, stream);
}

int nvfp4_linear_reduce_peers(nvfp4_handle* h, const void* A, int M, const uint8_t* packed, const uint8_t* scale,
                              float global_scale, int N, int K, const void* residual, void* C,
                              const nvfp4_peer_exchange* px, nvfp4_stream_t stream) {
    if (int e = validate_linear(h, A, M, packed, scale, global_scale, N, K, residual, C)) return e;
    if (!px) return NVFP4_E_NULL;
    if (px->world < 1 || px->world > 8 || px->rank < 0 || px->rank >= px->world) return NVFP4_E_TP;
    for (int q = 0; q < px->world; ++q)
        if (!px->peer[q] || (reinterpret_cast<uintptr_t>(px->peer[q]) & 15u)) return NVFP4_E_NULL;
    if (M == 0) return NVFP4_OK;
    if ((long long)M * N > px->slot_pairs) return NVFP4_E_LIMIT;
    LinearArgs a{A, packed, scale, 1.0f / global_scale, residual, C, M, N, K};
    a.px = px;
    return run_linear(h, a, stream);
}

// Validation of a descriptor and its translation into the kernels' argument record.
static int desc_to_args(nvfp4_handle* h, const nvfp4_linear_desc* d, LinearArgs* out) {
    if (!d) return NVFP4_E_NULL;
    if (int e = validate_linear(h, d->A, d->M, d->packed, d->scale, d->global_scale, d->N, d->K, d->residual, d->C,
                                d->swiglu_epilogue ? d->N / 2 : 0))
        return e;
    const long long stride = d->a_row_stride ? d->a_row_stride : d->K;
    const int k_valid = d->k_valid ? d->k_valid : d->K;
    if (stride < k_valid || (stride & 7) || k_valid < 1 || k_valid > d->K || (k_valid & 7)) return NVFP4_E_SHAPE;
    if (d->swiglu_up && !aligned16(d->swiglu_up)) return NVFP4_E_ALIGN;
    if (d->M > 0) {
        // What the kernel reads of A (and of the up half) spans (M-1) strides plus the valid columns; every CTA
        // re-reads it while others already store C, so neither may overlap the output, nor may the norm weight.
        const char* c0 = static_cast<const char*>(d->C);
        const char* c1 = c0 + (size_t)d->M * (d->swiglu_epilogue ? d->N / 2 : d->N) * 2;
        const size_t span = ((size_t)(d->M - 1) * (size_t)stride + (size_t)k_valid) * 2;
        auto overlaps = [&](const void* p, size_t bytes) {
            const char* p0 = static_cast<const char*>(p);
            return p && p0 < c1 && c0 < p0 + bytes;
        };
        if (overlaps(d->A, span) || overlaps(d->swiglu_up, span) || overlaps(d->norm_weight, (size_t)d->K * 2))
            return NVFP4_E_ALIAS;
    }
    if (d->norm_weight) {
        if (!aligned16(d->norm_weight)) return NVFP4_E_ALIGN;
        if (d->swiglu_up || k_valid != d->K || !(d->norm_eps >= 0.0f)) return NVFP4_E_SHAPE;   // the norm runs over all K columns of A itself
    }
    if (d->swiglu_epilogue) {
        if ((d->N & 15) != 0 || d->residual || d->px) return NVFP4_E_SHAPE;   // whole 16-row slabs; the output is the activation of the next linear
    }
    if (d->px) {
        if (d->px->world < 1 || d->px->world > 8 || d->px->rank < 0 || d->px->rank >= d->px->world) return NVFP4_E_TP;
        for (int q = 0; q < d->px->world; ++q)
            if (!d->px->peer[q] || (reinterpret_cast<uintptr_t>(d->px->peer[q]) & 15u)) return NVFP4_E_NULL;
        if ((long long)d->M * d->N > d->px->slot_pairs) return NVFP4_E_LIMIT;
    }
    LinearArgs a{d->A, d->packed, d->scale, 1.0f / d->global_scale, d->residual, d->C, d->M, d->N, d->K};
    a.px = d->px;
    a.swiglu_up = d->swiglu_up;
    a.a_stride = d->a_row_stride;
    a.k_valid = d->k_valid;
    a.norm_w = d->norm_weight;
    a.norm_eps = d->norm_eps;
    a.swiglu_out = d->swiglu_epilogue != 0;
    if (!a.px && !a.swiglu_up && stride == d->K && k_valid == d->K) { a.a_stride = 0; a.k_valid = 0; }   // the plain call
    *out = a;
    return NVFP4_OK;
}

int nvfp4_linear_ex(nvfp4_handle* h, const nvfp4_linear_desc* d, nvfp4_stream_t stream) {
    LinearArgs a{};
    if (int e = desc_to_args(h, d, &a)) return e;
    if (d->M == 0) return NVFP4_OK;
    return run_linear(h, a, stream);
}

struct nvfp4_chain {
    nvfp4_handle* h = nullptr;
    nvfp4::DecodeChain* c = nullptr;
    std::vector<nvfp4_peer_exchange> px;     // copies of the descriptors' exchanges (the kernel parameters keep only the pointers inside)
    int n = 0;
};

int nvfp4_chain_create(nvfp4_handle* h, const nvfp4_linear_desc* descs, int n, nvfp4_chain** out) {
    if (!h || !descs || !out) return NVFP4_E_NULL;
    *out = nullptr;
    if (n < 1 || n > 4096) return NVFP4_E_SHAPE;
    std::vector<LinearArgs> args((size_t)n);
    for (int l = 0; l < n; ++l) {
        if (int e = desc_to_args(h, &descs[l], &args[l])) return e;
        if (descs[l].M < 1 || descs[l].M > 8) return NVFP4_E_LIMIT;
    }
    if (decode_mma_scratch_bytes(args[0], h->dev) > h->workspace_bytes) return NVFP4_E_WORKSPACE;
    int prev = 0;
    cudaGetDevice(&prev);
    if (cudaSetDevice(h->dev.device) != cudaSuccess) return NVFP4_E_DEVICE;
    nvfp4_chain* c = new nvfp4_chain();
    c->h = h;
    c->n = n;
    const int st = create_decode_chain(args.data(), n, h->dev, h->workspace, &c->c);
    cudaSetDevice(prev);
    if (st != NVFP4_OK) { delete c; return st; }
    *out = c;
    return NVFP4_OK;
}

int nvfp4_chain_run(nvfp4_chain* c, nvfp4_stream_t stream) {
    if (!c || !c->c) return NVFP4_E_NULL;
    cudaError_t e = launch_decode_chain(c->c, stream);
    c->h->launches += 1;
    return cuda_status(e);
}

int nvfp4_chain_destroy(nvfp4_chain* c) {
    if (!c) return NVFP4_E_NULL;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->h->dev.device);
    destroy_decode_chain(c->c);
    cudaSetDevice(prev);
    delete c;
    return NVFP4_OK;
}

int nvfp4_linear_dual(nvfp4_handle* h, const void* A, int M, const uint8_t* packed1, const uint8_t* scale1,
                      float gs1, const uint8_t* packed2, const uint8_t* scale2, float gs2, int N, int K,
                      void* C1, void* C2, nvfp4_stream_t stream) {
    if (int e = validate_linear(h, A, M, packed1, scale1, gs1, N, K, nullptr, C1)) return e;
    if (int e = validate_linear(h, A, M, packed2, scale2, gs2, N, K, nullptr, C2)) return e;
    LinearArgs a{A, packed1, scale1, 1.0f / gs1, nullptr, C1, M, N, K};
    {
        // One launch of the NVFP4 tensor-core GEMV over both weights (one activation pre-pass), as the reference's
        // dual kernel is one launch (src/engine/dense_gemm_fp4_sm110.cu:264-351).
        LinearArgs d = a;
        d.packed2 = packed2; d.scale2 = scale2; d.inv_gs2 = 1.0f / gs2; d.C2 = C2;
        const bool fp4_wanted = M <= h->decode_max_m && (h->decode_impl == 3 || (h->decode_impl == 0 && h->fp4_native && M >= h->fp4_min_m));
        if (fp4_wanted && decode_fp4_scratch_bytes(K) <= kFp4ActBytes && kDecodeScratchBytes <= h->workspace_bytes &&
            !h->has_nan_scales(scale1) && !h->has_nan_scales(scale2) && decode_fp4_supported(d, h->dev)) {
            int nl = 0;
            cudaError_t e = launch_decode_fp4(d, h->dev, h->workspace, kFp4PairsOffset, h->workspace + kFp4ActOffset, &nl, stream);
            h->launches += (unsigned long long)nl;
            return cuda_status(e);
        }
    }
    // Otherwise two back-to-back launches on one stream: A (tens of KB) stays in L2 between them.
    if (int e = run_linear(h, a, stream)) return e;
    LinearArgs b{A, packed2, scale2, 1.0f / gs2, nullptr, C2, M, N, K};
    return run_linear(h, b, stream);
}

int nvfp4_dequant_bf16(nvfp4_handle* h, const uint8_t* packed, const uint8_t* scale, float global_scale,
                       int N, int K, void* out, nvfp4_stream_t stream) {
    if (!h || !packed || !scale || !out) return NVFP4_E_NULL;
    if (N <= 0 || K <= 0 || (K & 15) != 0) return NVFP4_E_SHAPE;
    if (int e = check_scale(global_scale)) return e;
    if (!aligned16(out) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return NVFP4_E_ALIGN;
    cudaError_t e = launch_dequant_bf16(packed, scale, 1.0f / global_scale, N, K, out, stream);
    h->launches += 1;
    return cuda_status(e);
}

int nvfp4_scan_scales(nvfp4_handle* h, const uint8_t* scale, int N, int K, long long* count, nvfp4_stream_t stream) {
    if (!h || !scale) return NVFP4_E_NULL;
    if (N <= 0 || K <= 0 || (K & 15) != 0) return NVFP4_E_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long* d_count = nullptr;
    unsigned long long n = 0;
    cudaError_t e = cudaMalloc(&d_count, sizeof(n));
    if (e != cudaSuccess) return (int)e;
    e = cudaMemsetAsync(d_count, 0, sizeof(n), s);
    if (e == cudaSuccess) e = launch_count_nan_scales(scale, (long long)N * (K >> 4), d_count, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&n, d_count, sizeof(n), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(d_count);
    if (e != cudaSuccess) return (int)e;
    h->launches += 1;
    auto it = std::find(h->nan_scales.begin(), h->nan_scales.end(), static_cast<const void*>(scale));
    if (n != 0 && it == h->nan_scales.end()) h->nan_scales.push_back(scale);
    if (n == 0 && it != h->nan_scales.end()) h->nan_scales.erase(it);        // the tensor was rewritten since
    if (count) *count = (long long)n;
    return NVFP4_OK;
}

int nvfp4_swiglu_strided(nvfp4_handle* h, const void* gate, const void* up, int M, int I, long long in_stride,
                         void* out, long long out_stride, nvfp4_stream_t stream) {
    if (!h || !gate || !up || !out) return NVFP4_E_NULL;
    if (M < 0 || I <= 0 || in_stride < I || out_stride < I) return NVFP4_E_SHAPE;
    if (M == 0) return NVFP4_OK;
    // The vector path needs 16-byte aligned row starts.
    if (I >= 8 && (!aligned16(gate) || !aligned16(up) || !aligned16(out) || (I & 7) || (in_stride & 7) || (out_stride & 7)))
        return NVFP4_E_ALIGN;
    cudaError_t e = launch_swiglu(gate, up, in_stride, M, I, out, out_stride, stream);
    h->launches += 1;
    return cuda_status(e);
}

int nvfp4_swiglu_interleaved(nvfp4_handle* h, const void* gate_up, int M, int I, long long in_stride, void* out,
                             long long out_stride, nvfp4_stream_t stream) {
    if (!h || !gate_up || !out) return NVFP4_E_NULL;
    if (M < 0 || I <= 0 || (I & 7) != 0 || in_stride < 2LL * I || out_stride < I) return NVFP4_E_SHAPE;
    if (!aligned16(gate_up) || !aligned16(out) || (in_stride & 7) || (out_stride & 7)) return NVFP4_E_ALIGN;
    if (M == 0) return NVFP4_OK;
    cudaError_t e = launch_swiglu(gate_up, static_cast<const char*>(gate_up) + 16, in_stride, M, I, out, out_stride, stream, true);
    h->launches += 1;
    return cuda_status(e);
}

int nvfp4_swiglu(nvfp4_handle* h, const void* gate, const void* up, int M, int I, void* out,
                 nvfp4_stream_t stream) {
    if (!h || !gate || !out) return NVFP4_E_NULL;
    if (I <= 0) return NVFP4_E_SHAPE;
    const bool merged = (up == nullptr);
    if (merged) up = static_cast<const char*>(gate) + (size_t)I * 2;
    return nvfp4_swiglu_strided(h, gate, up, M, I, merged ? 2LL * I : (long long)I, out, I, stream);
}

int nvfp4_linear_bf16(nvfp4_handle* h, const void* A, int M, const void* W, int N, int K, const void* residual, void* C,
                      nvfp4_stream_t stream) {
    if (!h || !A || !W || !C) return NVFP4_E_NULL;
    if (M < 0 || N <= 0 || K <= 0 || (K & 7) != 0) return NVFP4_E_SHAPE;
    if (!aligned16(A) || !aligned16(W) || !aligned16(C) || (residual && !aligned16(residual))) return NVFP4_E_ALIGN;
    const char* a0 = static_cast<const char*>(A);
    const char* c0 = static_cast<const char*>(C);
    if (M > 0 && a0 < c0 + (size_t)M * N * 2 && c0 < a0 + (size_t)M * K * 2) return NVFP4_E_ALIAS;
    if (M == 0) return NVFP4_OK;
    DenseArgs a{A, W, residual, C, M, N, K};
    if (dense_gemv_supported(a, h->dev)) {
        int nl = 0;
        cudaError_t e = launch_dense_gemv(a, h->dev, h->workspace, &nl, stream);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    if (M > 16 && dense_umma_supported(a) && kDecodeScratchBytes + dense_umma_scratch_bytes() <= h->workspace_bytes) {
        int nl = 0;
        cudaError_t e = launch_dense_umma(a, h->dev, h->workspace, h->workspace_bytes, kDecodeScratchBytes, &nl, stream);
        h->launches += (unsigned long long)nl;
        return cuda_status(e);
    }
    // shapes neither kernel takes (K % 256, N % 8): the plain CUDA-core GEMM
    cudaError_t e = launch_gemm_bf16_simple(A, W, residual, C, M, N, K, stream);
    h->launches += 1;
    return cuda_status(e);
}

int nvfp4_rmsnorm(nvfp4_handle* h, const void* x, const void* weight, float eps, int M, int K, void* out,
                  nvfp4_stream_t stream) {
    if (!h || !x || !weight || !out) return NVFP4_E_NULL;
    if (M < 0 || K <= 0 || (K & 7) != 0) return NVFP4_E_SHAPE;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(out)) return NVFP4_E_ALIGN;
    if (M == 0) return NVFP4_OK;
    cudaError_t e = launch_rmsnorm(out, const_cast<void*>(x), nullptr, weight, eps, M, K, stream);
    h->launches += 1;
    return cuda_status(e);
}

int nvfp4_add_rmsnorm(nvfp4_handle* h, void* residual, const void* bias, const void* weight, float eps, int M, int K,
                      void* norm_out, nvfp4_stream_t stream) {
    if (!h || !residual || !bias || !weight || !norm_out) return NVFP4_E_NULL;
    if (M < 0 || K <= 0 || (K & 7) != 0) return NVFP4_E_SHAPE;
    if (!aligned16(residual) || !aligned16(bias) || !aligned16(weight) || !aligned16(norm_out)) return NVFP4_E_ALIGN;
    if (M == 0) return NVFP4_OK;
    cudaError_t e = launch_rmsnorm(norm_out, residual, bias, weight, eps, M, K, stream);
    h->launches += 1;
    return cuda_status(e);
}

int nvfp4_linear_host(nvfp4_handle* h, const void* A_host, int M, const uint8_t* packed, const uint8_t* scale,
                      float global_scale, int N, int K, const void* residual_host, void* C_host,
                      nvfp4_stream_t stream) {
    if (!h || !A_host || !C_host || !packed || !scale) return NVFP4_E_NULL;
    if (M < 0 || N <= 0 || K <= 0 || (K & 15) != 0) return NVFP4_E_SHAPE;
    if (int e = check_scale(global_scale)) return e;
    const size_t a_bytes = ((size_t)M * K * 2 + 255) / 256 * 256;
    const size_t c_bytes = ((size_t)M * N * 2 + 255) / 256 * 256;
    const size_t tail = a_bytes + c_bytes;   // staging lives at the END of the workspace
    if (h->workspace_bytes < kDecodeScratchBytes + tail) return NVFP4_E_WORKSPACE;
    char* dA = h->workspace + h->workspace_bytes - tail;
    char* dC = dA + a_bytes;
    cudaError_t e = cudaMemcpyAsync(dA, A_host, (size_t)M * K * 2, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    const void* dR = nullptr;
    if (residual_host) {   // the residual is staged straight into the output buffer (C may alias residual)
        e = cudaMemcpyAsync(dC, residual_host, (size_t)M * N * 2, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return (int)e;
        dR = dC;
    }
    if (!aligned16(dA) || !aligned16(dC)) return NVFP4_E_ALIGN;
    // Without a residual the kernels may write a pinned, device-mapped C_host themselves (coalesced stores over PCIe
    // that overlap the kernel's tail) and the copy back, with its own start-up latency, is not needed.
    void* out = dC;
    if (h->host_direct_out && !residual_host && aligned16(C_host) && (size_t)M * N * 2 <= (2u << 20)) {
        if (C_host != h->host_out_seen) {
            cudaPointerAttributes at{};
            h->host_out_seen = C_host;
            h->host_out_dev = nullptr;
            if (cudaPointerGetAttributes(&at, C_host) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer)
                h->host_out_dev = at.devicePointer;
            else
                cudaGetLastError();
        }
        if (h->host_out_dev) out = h->host_out_dev;
    }
    // The kernels see the workspace without the staging area, so their scratch never reaches it.
    LinearArgs a{dA, packed, scale, 1.0f / global_scale, dR, out, M, N, K};
    int st = run_linear(h, a, stream, h->workspace_bytes - tail);
    if (st) return st;
    if (out == dC) {
        e = cudaMemcpyAsync(C_host, dC, (size_t)M * N * 2, cudaMemcpyDeviceToHost, stream);
        if (e != cudaSuccess) return (int)e;
    }
    return cuda_status(cudaStreamSynchronize(stream));
}

// ---- reference-shaped entry points on a per-device default handle ---------------------

namespace {
std::mutex g_mu;
nvfp4_handle* g_default[64] = {};
size_t g_default_ws = 64u << 20;
thread_local int g_last_status = 0;

nvfp4_handle* default_handle() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_default[dev]) {
        nvfp4_handle* h = nullptr;
        g_last_status = nvfp4_create(dev, g_default_ws, &h);
        g_default[dev] = h;
    }
    return g_default[dev];
}

void linear_on_default(const void* A, const nvfp4_quantized_weight* W, void* C, const void* residual, int M,
                       nvfp4_stream_t s) {
    if (!W) { g_last_status = NVFP4_E_NULL; return; }
    nvfp4_handle* h = default_handle();
    if (!h) { if (!g_last_status) g_last_status = NVFP4_E_DEVICE; return; }
    g_last_status = nvfp4_linear(h, A, M, W->packed, W->scale, W->global_scale, W->N, W->K, residual, C, s);
}
}  // namespace

int nvfp4_default_handle_workspace(size_t bytes) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_default_ws = bytes;
    return NVFP4_OK;
}

void nvfp4_init_fp4_cublaslt(void) { (void)default_handle(); }

void nvfp4_cleanup_fp4_cublaslt(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& h : g_default) {
        if (h) { nvfp4_destroy(h); h = nullptr; }
    }
}

int nvfp4_last_status(void) { return g_last_status; }

void nvfp4_invoke_fp4_gemv(const void* A, const nvfp4_quantized_weight* W, void* C, nvfp4_stream_t s) {
    linear_on_default(A, W, C, nullptr, 1, s);
}
void nvfp4_invoke_fp4_gemv_add(const void* A, const nvfp4_quantized_weight* W, void* C, const void* residual,
                               nvfp4_stream_t s) {
    linear_on_default(A, W, C, residual, 1, s);
}
void nvfp4_invoke_fp4_dual_gemv(const void* A, const nvfp4_quantized_weight* W1, const nvfp4_quantized_weight* W2,
                                void* C1, void* C2, nvfp4_stream_t s) {
    if (!W1 || !W2) { g_last_status = NVFP4_E_NULL; return; }
    nvfp4_handle* h = default_handle();
    if (!h) { if (!g_last_status) g_last_status = NVFP4_E_DEVICE; return; }
    // The reference takes N and K from W1 for both weights (dense_gemm_fp4_sm110.cu:405-406).
    g_last_status = nvfp4_linear_dual(h, A, 1, W1->packed, W1->scale, W1->global_scale, W2->packed, W2->scale,
                                      W2->global_scale, W1->N, W1->K, C1, C2, s);
}
void nvfp4_invoke_fp4_gemm(const void* A, const nvfp4_quantized_weight* W, void* C, int M, nvfp4_stream_t s) {
    linear_on_default(A, W, C, nullptr, M, s);
}
void nvfp4_invoke_fp4_gemm_add(const void* A, const nvfp4_quantized_weight* W, void* D, const void* residual,
                               int M, nvfp4_stream_t s) {
    linear_on_default(A, W, D, residual, M, s);
}

}  // extern "C"
