// Internal declarations shared by the host-side dispatcher and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/nvfp4_b200.h"

namespace nvfp4 {

// Arguments of one linear call after validation.  All pointers are device pointers.
struct LinearArgs {
    const void* A;          // [M,K] bf16
    const uint8_t* packed;  // [N,K/2]
    const uint8_t* scale;   // [N,K/16]
    float inv_gs;           // 1.0f / global_scale, computed on the host in FP32
    const void* residual;   // [M,N] bf16 or nullptr
    void* C;                // [M,N] bf16 (fp32 when out_f32)
    int M, N, K;
    bool out_f32 = false;   // unrounded FP32 sums, no residual: partial results a caller reduces itself
    const nvfp4_peer_exchange* px = nullptr;   // push the sums to the peers and reduce over the group in the same kernel
    const void* swiglu_up = nullptr;   // A is the gate half, this the up half: activations = bf16(silu(gate) * up)
    long long a_stride = 0;            // elements between rows of A / swiglu_up (0 = K)
    int k_valid = 0;                   // activation columns >= k_valid are zero (0 = K)
    bool swiglu_out = false;           // weight rows interleaved (8 gate, 8 up per 16): C is [M, N/2] = bf16(silu(gate) * up)
    const void* norm_w = nullptr;      // [K] BF16: activations = rmsnorm(A) with the centred weight (1 + w)
    float norm_eps = 0.0f;
    // The reference's arithmetic above 8 tokens (fp4_dequant_kernel + BF16 GEMM, src/engine/dense_gemm_fp4_sm110.cu:444-467,
    // 558-583): weights rounded to BF16 AFTER the global scale, bf16(lut * (scale * 1/gs)).  The tcgen05 GEMM only.
    bool round_weights = false;
    // A second weight of the same shape on the same activations, its own output (the reference's dual GEMV,
    // src/engine/dense_gemm_fp4_sm110.cu:264-351): one launch of the NVFP4 tensor-core GEMV takes both.
    const uint8_t* packed2 = nullptr;
    const uint8_t* scale2 = nullptr;
    float inv_gs2 = 0.0f;
    void* C2 = nullptr;
};

// Encoded tensor maps of recently used tensors, keyed by everything that goes into the encoding: a decode
// step calls the same few weights over and over, and cuTensorMapEncodeTiled costs the host more than a
// microsecond per map.  Direct-mapped, owned by the handle (one host thread at a time).
struct TensorMapCache {
    struct Entry {
        const void* base = nullptr;
        uint64_t cols = 0, rows = 0;
        uint32_t box_cols = 0, box_rows = 0;
        int dtype = 0, esize = 0, swizzle = 0;
        CUtensorMap map;
    };
    static constexpr int kEntries = 128;
    Entry e[kEntries];
};

struct nvfp4_device_info {
    int device;
    int sm_count;
    int cc_major, cc_minor;
    size_t smem_optin;
    int prefill_stream_k = 1;    // split the tiles left after whole waves by k over all CTAs
    int skinny_split_cost = 12;  // stage-times charged to splitting row tiles by k in the few-token kernel
    int fp4_own_quant = 1;       // one or two tokens: the tensor-core GEMV expands its activations itself, no pre-pass launch
    size_t gemv_pairs_offset = 6u << 20;   // where the 8-token GEMV's {value, epoch} partial pairs start in its scratch
    TensorMapCache* maps = nullptr;        // null: encode every time
};

// The tag of one GEMV launch on the split-tile pairs in its scratch: a process-wide counter, never 0
// (what a cleared slot holds), safe to call from any host thread.  It is only the second line of
// defence -- the owner of a row tile clears every pair it has read, so a captured launch that is
// replayed with the same tag still never meets an old pair; a changing tag additionally keeps a
// pair that a timed-out launch left behind from being accepted by a later eager launch.
unsigned int next_launch_tag();

// --- decode_simple.cu: scalar CUDA-core GEMV, any K % 16 == 0, M <= 16 per launch.
cudaError_t launch_decode_simple(const LinearArgs& a, cudaStream_t s);

// --- dequant_swiglu.cu
cudaError_t launch_dequant_bf16(const uint8_t* packed, const uint8_t* scale, float inv_gs, int N, int K,
                                void* out, cudaStream_t s);
// adds to *count (zeroed by the caller) the block-scale bytes that are 0x7F or 0xFF
cudaError_t launch_count_nan_scales(const uint8_t* scale, long long bytes, unsigned long long* count, cudaStream_t s);
cudaError_t launch_swiglu(const void* gate, const void* up, long long row_stride_in, int M, int I,
                          void* out, long long row_stride_out, cudaStream_t s, bool interleaved = false);
// out = rmsnorm(x (+ bias)) with the centred weight; with a bias, x is updated in place.  One CTA per token.
cudaError_t launch_rmsnorm(void* out, void* x, const void* bias, const void* weight, float eps, int M, int K,
                           cudaStream_t s);

// --- prefill_simple.cu: C = A * Wdq^T with Wdq bf16 [N,K] already dequantised (debug path).
cudaError_t launch_gemm_bf16_simple(const void* A, const void* Wdq, const void* residual, void* C,
                                    int M, int N, int K, cudaStream_t s);

// --- dense_gemv.cu: BF16 weights [N,K], up to 16 tokens (8 per launch), the NVFP4 GEMV's skeleton without dequantisation.
struct DenseArgs {
    const void* A;          // [M,K] BF16
    const void* W;          // [N,K] BF16 row-major
    const void* residual;   // [M,N] BF16 or null
    void* C;                // [M,N] BF16
    int M, N, K;
};
bool dense_gemv_supported(const DenseArgs& a, const nvfp4_device_info& dev);
cudaError_t configure_dense_gemv();
cudaError_t launch_dense_gemv(const DenseArgs& a, nvfp4_device_info& dev, void* scratch, int* launches, cudaStream_t s);
// --- prefill_umma.cu, BF16 weights: the tcgen05 GEMM without the dequantisation (K % 256 == 0, N % 8 == 0).
bool dense_umma_supported(const DenseArgs& a);
size_t dense_umma_scratch_bytes();
cudaError_t launch_dense_umma(const DenseArgs& a, nvfp4_device_info& dev, void* scratch, size_t scratch_bytes, size_t offset,
                              int* launches, cudaStream_t s);

// --- decode_mma.cu: TMA-fed shared-memory ring + register dequant + warp MMA GEMV (M <= 16).
bool decode_mma_supported(const LinearArgs& a);
bool decode_mma_fits(const LinearArgs& a, const nvfp4_device_info& dev);   // activations fit in shared memory
size_t decode_mma_scratch_bytes(const LinearArgs& a, const nvfp4_device_info& dev);
cudaError_t launch_decode_mma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, int* launches,
                              cudaStream_t s);
cudaError_t configure_decode_mma();
// A chain: n linears of up to 8 tokens each, run in order by one persistent launch (the producer streams the
// next linear's weights while the consumers pass a grid-wide barrier and stage the next activations).
struct DecodeChain;
int create_decode_chain(const LinearArgs* linears, int n, const nvfp4_device_info& dev, void* scratch, DecodeChain** out);
cudaError_t launch_decode_chain(DecodeChain* c, cudaStream_t s);
void destroy_decode_chain(DecodeChain* c);

// Opt a kernel in to `bytes` of dynamic shared memory and pin its carve-out to the largest one.  Left to
// itself the driver picks the smallest carve-out that holds one CTA; a launch that lands just under a
// carve-out step (196 KB, say) then leaves no room for the small kernels launched next to it with
// programmatic stream serialization (activation pre-passes, norms), and those and the next GEMV's
// CTAs wait for each other's SMs: 4 us on a 10 us call, measured.
template <class Kernel>
inline cudaError_t configure_large_smem(Kernel kernel, int bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

// --- act_fp4.cu / decode_fp4.cu: the GEMV on the NVFP4 tensor-core path (tcgen05.mma kind::mxf4nvf4).
namespace fp4 {
constexpr int kMaxTokens = 16;
constexpr int kMaxTerms = 6;
constexpr size_t kPairBytes = 5u << 19;     // 2.5 MB of split-tile pair slots in the handle's scratch
// NVFP4 term rows per token (act_fp4.cu): five, and a sixth where it fits the MMA columns five need anyway
// (tokens x terms padded to a multiple of 16): 1, 2, 4, 5, 7, 8, 10 and 13 tokens.
__host__ __device__ constexpr int terms_for(int tokens) {
    return ((tokens * 5 + 15) / 16 * 16) / tokens >= 6 ? 6 : 5;
}
// Where the block scale of column c (token * terms + term), 16-element block b along K, sits in the
// scale buffer: [256-k chunk][column group c / 32][lane c % 32][64-k MMA of the chunk][block of the MMA],
// i.e. per chunk and column group one 16-byte word per tensor-memory lane, which the GEMV loads with one
// 128-bit access and spreads over the four tensor-memory columns the four MMAs of the chunk read.
__host__ __device__ inline size_t sfb_offset(int b, int c, int groups) {
    const int kc = b >> 4, s = (b >> 2) & 3, kb = b & 3;
    return ((size_t)kc * groups + (size_t)(c >> 5)) * 512 + (size_t)(c & 31) * 16 + (size_t)s * 4 + kb;
}
// The activation scratch the pre-pass fills and the GEMV kernels read: codes [kMaxCols, K/2], block scales
// [K/256][3 groups][512 bytes] (a kernel with fewer column groups uses a prefix), 16 per-token factors.
constexpr int kMaxCols = 96;
inline size_t act_sfb_offset(int K) { return ((size_t)kMaxCols * (K / 2) + 255) / 256 * 256; }
inline size_t act_unscale_offset(int K) { return act_sfb_offset(K) + ((size_t)(K / 256) * 1536 + 255) / 256 * 256; }
inline size_t act_scratch_bytes(int K) { return act_unscale_offset(K) + 256; }
}  // namespace fp4
// The pre-pass takes the activation-side options of `a` (swiglu_up, norm_w, a_stride, k_valid).
bool act_to_fp4_supported(const LinearArgs& a);
cudaError_t launch_act_to_fp4(const LinearArgs& a, int terms, int groups, void* codes, void* sfb, float* unscale, cudaStream_t s);
bool decode_fp4_supported(const LinearArgs& a, const nvfp4_device_info& dev);
size_t decode_fp4_scratch_bytes(int K);       // codes + scale atoms + per-token factors of the activation pre-pass
cudaError_t configure_decode_fp4();
// scratch: the handle workspace (status word at 0, launch counter at 64, pairs at pairs_offset); act: decode_fp4_scratch_bytes.
cudaError_t launch_decode_fp4(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t pairs_offset, void* act,
                              int* launches, cudaStream_t s);
// decode_fp4_stream.cu: the same GEMV for 10 to 16 tokens (and any shape whose activations do not fit beside the
// ring): the activations travel through the ring with the weights.  Same scratch, same arguments.
bool decode_fp4_stream_supported(const LinearArgs& a, const nvfp4_device_info& dev);
cudaError_t configure_decode_fp4_stream();
cudaError_t launch_decode_fp4_stream(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t pairs_offset, void* act,
                                     int* launches, cudaStream_t s);

// --- act_f16.cu: BF16 activations -> FP16 copy with an exact per-token power-of-two scale; unscale[m] = 1/scale.
cudaError_t launch_act_to_f16(const void* A, int M, int K, void* out_f16, float* unscale, cudaStream_t s);

// --- prefill_umma.cu: fused dequant + tcgen05 BF16 GEMM with TMEM accumulators.
bool prefill_umma_supported(const LinearArgs& a);
size_t prefill_umma_reserved_bytes();   // flags + partial tiles at the start of the kernel's scratch
size_t prefill_umma_scratch_bytes(int max_M, int max_N, int max_K);
// scratch[0] is the handle's status word; the FP16 activation copy lives at scratch + offset.
cudaError_t launch_prefill_umma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch,
                                size_t scratch_bytes, size_t offset, int* launches, cudaStream_t s);

// Sets the per-kernel attributes (dynamic shared memory opt-in) once per device.
// --- decode_wide.cu: 9..16 tokens in one GEMV launch, activations streamed through the ring.
bool decode_wide_supported(const LinearArgs& a);
size_t decode_wide_scratch_bytes(int sm_count);
cudaError_t configure_decode_wide();
cudaError_t launch_decode_wide(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, void* act_f16, float* unscale,
                               int* launches, cudaStream_t s);

// --- skinny_umma.cu: 1 <= M <= 128, dequantised weights as the TMEM A operand of tcgen05.mma.
bool skinny_umma_supported(const LinearArgs& a);
cudaError_t configure_skinny_umma();
cudaError_t launch_skinny_umma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t scratch_bytes,
                               size_t offset, int* launches, cudaStream_t s);

cudaError_t configure_kernels(const nvfp4_device_info& dev);

}  // namespace nvfp4
