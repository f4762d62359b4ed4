/*
 * nvfp4_b200 — C ABI of the B200 (sm_100a) NVFP4 W4A16 linear layer.
 *
 * Drop-in boundary for the reference engine's FP4 operator set
 * (namespace qwen_thor::ops, src/engine/dense_gemm_fp4.h:25-72) and the weight
 * descriptor it takes (struct QuantizedWeight, src/engine/layer.h:197-204).
 *
 * Data format (identical to the reference's):
 *   packed  uint8 [N, K/2]   two E2M1 codes per byte, low nibble = even k
 *   scale   uint8 [N, K/16]  unsigned E4M3, one per 16 consecutive k of a row
 *   global_scale  float      W[n,k] = e2m1(code) * ue4m3(scale) / global_scale
 *   activations / outputs    BF16, row-major [M, K] / [M, N]
 * All data pointers are DEVICE pointers owned by the caller.  Every call is
 * asynchronous on the given stream, allocates nothing and never synchronises.
 * There is no CPU fallback: without a CUDA device every call fails.
 *
 * Status codes: 0 = OK; < 0 = argument / shape error (NVFP4_E_*); > 0 = a
 * cudaError_t raised by a launch.
 */
#ifndef NVFP4_B200_H
#define NVFP4_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* nvfp4_stream_t; /* == cudaStream_t */
typedef struct nvfp4_handle nvfp4_handle;

enum {
    NVFP4_OK = 0,
    NVFP4_E_NULL = -1,       /* a required pointer is NULL */
    NVFP4_E_SHAPE = -2,      /* M,N,K out of range, K % 16 != 0, ... */
    NVFP4_E_ALIGN = -3,      /* a pointer or row pitch breaks the alignment rule */
    NVFP4_E_WORKSPACE = -4,  /* handle workspace too small for this call */
    NVFP4_E_ALIAS = -5,      /* A aliases the output */
    NVFP4_E_SCALE = -6,      /* global_scale is 0, negative, inf or NaN */
    NVFP4_E_DEVICE = -7,     /* no CUDA device / wrong device / not sm_100 */
    NVFP4_E_OPTION = -8,     /* unknown option or value */
    NVFP4_E_TP = -9,         /* tensor-parallel set-up error */
    NVFP4_E_LIMIT = -10      /* beyond the fixed maximum of the allocation-free entry point */
};

/* Layout-identical to qwen_thor::core::QuantizedWeight (src/engine/layer.h:197-204):
 * ptr@0, ptr@8, float@16, float@20, int@24, int@28, sizeof 32.  input_scale is
 * carried but unused in W4A16 (src/engine/dense_gemm_fp4.h:21). */
typedef struct nvfp4_quantized_weight {
    uint8_t* packed;
    uint8_t* scale;
    float global_scale;
    float input_scale;
    int N;
    int K;
} nvfp4_quantized_weight;

/* ---- lifecycle ---------------------------------------------------------
 * Replaces the reference's process-global state (lazy dequant scratch and
 * cuBLAS handles, src/engine/dense_gemm_fp4_sm110.cu:428,470-486) and its
 * init_fp4_cublaslt()/cleanup_fp4_cublaslt() hooks (:430-441): one handle per
 * device, workspace sized once at creation. */
int nvfp4_create(int device, size_t workspace_bytes, nvfp4_handle** out);
int nvfp4_destroy(nvfp4_handle* h);
/* Workspace needed so that every call with M<=max_M, N<=max_N, K<=max_K succeeds. */
int nvfp4_workspace_bytes(int max_M, int max_N, int max_K, size_t* bytes);
const char* nvfp4_status_string(int status);

/* Kernel-selection knobs for tests and benchmarks.
 *   "decode_impl":  0 = auto, 1 = scalar CUDA-core GEMV, 2 = TMA ring + mma.sync GEMV,
 *                   3 = the NVFP4 tensor-core GEMV wherever it applies (1..9 tokens, K % 256 == 0,
 *                   plain [M, K] activations), the auto choice elsewhere
 *   "fp4_native":   1 (default) = in auto mode "fp4_min_m" (default 1) .. 9 tokens take the NVFP4
 *                   tensor-core GEMV: tcgen05.mma kind::mxf4nvf4 on the packed weights as they lie
 *                   in HBM, the BF16 activations expanded into six NVFP4 terms per token (five for
 *                   3, 6 and 9 tokens); their sum reproduces a token to 1e-5 (8e-5) of each 16-element
 *                   block's largest value, whose own BF16 rounding step is 4e-3.  A scale byte 0x7F / 0xFF is NaN to the
 *                   tensor core, as it is in FP8 E4M3; every other kernel, like the reference's
 *                   table-free decoder (dense_gemm_fp4_sm110.cu:30-41), reads it as 480.  No finite
 *                   FP8 E4M3 value encodes to it; nvfp4_scan_scales finds such a weight at load time
 *                   and keeps it off this kernel.  0 = off
 *   "gemm_weight_rounding": 0 (default) = every kernel multiplies the exact block-scaled weights and applies
 *                   1 / global_scale once, in FP32 (the reference's arithmetic up to 8 tokens,
 *                   dense_gemm_fp4_sm110.cu:96-141).  1 = above 8 tokens the weights are rounded to BF16
 *                   after the global scale, bf16(e2m1 * (ue4m3 * 1/gs)), operation for operation what the
 *                   reference's GEMM branch does (:444-467, 558-583); with a global scale that is not a
 *                   power of two the two forms lie 2.7e-3 apart.  Plain calls with N % 8 == 0 and
 *                   K % 256 == 0 only (NVFP4_E_LIMIT otherwise); slower (the tcgen05 GEMM with a longer
 *                   dequantisation)
 *   "fp4_stream_min_m": token count from which that kernel's activations travel through the shared-memory
 *                   ring with the weights instead of staying resident beside it (they must from 10 on:
 *                   48 MMA columns are the resident form's limit).  10 (default) = chosen per call below
 *                   10: streamed from seven tokens on where a CTA's share of the weights is long
 *   "fp4_own_quant": 1 (default) = for one or two tokens (no SwiGLU or RMSNorm in front) that kernel
 *                   expands the activations itself and no pre-pass kernel is launched; 0 = always
 *                   the pre-pass
 *   "prefill_impl": 0 = auto, 1 = dequant-to-workspace + CUDA-core GEMM (debug),
 *                   2 = fused dequant + tcgen05 GEMM
 *   "decode_max_m": largest M routed to the GEMV path (default 16)
 *   "wide_gemv": 1 (default) = 9..16 tokens take one launch of the wide GEMV kernel (two
 *                   8-token MMA tiles, activations streamed with the weights); 0 = off
 *   "skinny_min_m", "skinny_max_m": token counts (default 9..64) routed to the few-token
 *                   kernel that keeps the dequantised weights in tensor memory; min 129 or
 *                   max 0 turns it off.  "skinny_split_cost": stage-times charged to
 *                   splitting row tiles along K when that kernel plans its work.
 *   "prefill_stream_k": 1 (default) = output tiles left over after whole waves of tiles are
 *                   split along K over all SMs; 0 = whole tiles only                */
int nvfp4_set_option(nvfp4_handle* h, const char* name, int value);
int nvfp4_get_option(nvfp4_handle* h, const char* name, int* value);

/* ---- the linear layer ---------------------------------------------------
 * C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual[M,N]) ), FP32 accumulation,
 * residual added in FP32 before the single rounding; residual may be NULL and
 * may alias C.  One entry point for the reference's four:
 *   invoke_fp4_gemv      (dense_gemm_fp4_sm110.cu:360-375)  M=1, residual NULL
 *   invoke_fp4_gemv_add  (:377-393)                          M=1
 *   invoke_fp4_gemm      (:539-584)                          residual NULL
 *   invoke_fp4_gemm_add  (:586-632)
 * Requirements: K % 16 == 0; A, C, residual 16-byte aligned; packed 16-byte
 * aligned; K % 32 == 0 for the fast paths (other K take the scalar path). */
int nvfp4_linear(nvfp4_handle* h, const void* A_bf16, int M,
                 const uint8_t* packed, const uint8_t* scale_ue4m3, float global_scale,
                 int N, int K, const void* residual_bf16_or_null, void* C_bf16,
                 nvfp4_stream_t stream);

/* The GEMV for callers that must not allocate device memory (no counterpart in the reference:
 * there the scratch is a lazily grown global buffer).  Same arguments and result as nvfp4_linear
 * without a handle: the cross-CTA scratch of the GEMV kernel sits in a fixed ~1.3 MB array inside
 * the library's device image (held by every GPU that loads the library, until the process exits),
 * so the call performs no cudaMalloc / cudaFree of any kind.  It serves hosts whose device memory
 * is fully planned before they start calling -- e.g. an engine that gives all remaining HBM to its
 * KV-cache pool at start-up, where a later allocation by this library could fail or break the
 * engine's budget.
 * Limits (else NVFP4_E_LIMIT): M <= 16, K % 256 == 0, packed and scale 16-byte aligned, and the
 * FP16 copy of <= 8 tokens' activations must fit in shared memory beside the weight ring; the
 * grid is capped at 160 CTAs, the size the array was laid out for.
 * The first call on each device looks up the array's device address and sets the kernel's
 * shared-memory attribute (host-side work that later calls skip).  All calls share the
 * one array: it keeps the previous call's partial sums, which is harmless because every partial
 * carries the sequence number of its launch, taken from a counter in the array itself, and is
 * rewritten before it is read; but two calls that overlap on the GPU
 * (different streams) race on it -- issue them on one stream.  The device of `stream` must be the
 * current device.  nvfp4_noalloc_status reads back whether a device-side wait ever ran out. */
int nvfp4_linear_decode_noalloc(const void* A_bf16, int M, const uint8_t* packed, const uint8_t* scale_ue4m3,
                                float global_scale, int N, int K, const void* residual_bf16_or_null,
                                void* C_bf16, nvfp4_stream_t stream);

/* The device-side status word of the allocation-free GEMV on the current device (no counterpart in
 * the reference).  A bounded wait of nvfp4_linear_decode_noalloc that ran out leaves its code in the
 * fixed array (the first failure wins, codes as for nvfp4_device_status) and part of C unwritten;
 * the entry point itself cannot see that, it only enqueues.  This call synchronises the device,
 * copies the four bytes back and, with reset != 0, clears them.  It allocates nothing. */
int nvfp4_noalloc_status(unsigned int* status, int reset);

/* C_f32[M,N] = A * W^T as unrounded FP32 (no residual, no BF16 rounding): a partial result for
 * callers that sum several of them before rounding once, e.g. the K-split down projection of
 * the tensor-parallel MLP.  No reference counterpart (the reference is single-GPU and always
 * rounds, src/engine/dense_gemm_fp4_sm110.cu:137-140).  K % 256 == 0; more than 16 tokens also need
 * N % 8 == 0 (the tcgen05 GEMM's FP32 epilogue); otherwise NVFP4_E_LIMIT. */
int nvfp4_linear_f32(nvfp4_handle* h, const void* A_bf16, int M, const uint8_t* packed, const uint8_t* scale_ue4m3,
                     float global_scale, int N, int K, void* C_f32, nvfp4_stream_t stream);

/* The K-split linear of a tensor-parallel group in ONE kernel: this rank's partial sums
 * A * W^T (W = this rank's K columns) are pushed, unrounded, into the exchange buffers of all
 * ranks of the group over peer memory (plain NVLink stores of {value, epoch} pairs), and the
 * same kernel then adds the partials of all ranks in rank order in FP32, adds the residual and
 * rounds once: C[M,N] is the full sum, identical on every rank.  `px` names the buffers:
 * peer[q] is rank q's buffer as mapped into this process (peer[rank] is this rank's own; layout
 * in csrc/exchange_layout.h, allocated zero-filled with room for 16 * N pairs per slot by
 * libnvfp4_b200_tp).  Every rank of the group must make the same call (same M, N) in the same
 * order; a peer whose data does not arrive within about a second sets the buffer's status word
 * and leaves that part of C unwritten.  No reference counterpart (the reference is single-GPU).
 * M <= 16, K % 256 == 0, world <= 8, otherwise NVFP4_E_LIMIT. */
typedef struct nvfp4_peer_exchange {
    void* peer[8];
    int rank, world;
    int slot_pairs;      /* pairs per slot of the buffers: at least M * N */
} nvfp4_peer_exchange;
int nvfp4_linear_reduce_peers(nvfp4_handle* h, const void* A_bf16, int M, const uint8_t* packed,
                              const uint8_t* scale_ue4m3, float global_scale, int N, int K,
                              const void* residual_bf16_or_null, void* C_bf16, const nvfp4_peer_exchange* px,
                              nvfp4_stream_t stream);

/* The linear layer with its optional fusions, for M <= 16 and K % 256 == 0 (NVFP4_E_LIMIT
 * otherwise; a descriptor that uses none of the options is the plain nvfp4_linear for any M):
 *   swiglu_up     the activations are bf16(silu(A) * swiglu_up) (the reference's SwiGLU with its
 *                 single rounding, src/engine/light_ops.cu:186-187), formed while the kernel
 *                 stages them: A is the gate half, swiglu_up the up half of the gate/up output,
 *                 so the [M, I] SwiGLU tensor of run_mlp (src/engine/layer.cu:87-99) is never written;
 *   a_row_stride  elements between token rows of A and swiglu_up (2I for the merged gate/up layout);
 *   k_valid       activation columns >= k_valid count as zero (a weight shard whose K was padded);
 *   px            sum over a tensor-parallel group inside the kernel (see nvfp4_linear_reduce_peers);
 *   norm_weight   [K] BF16: the activations are rmsnorm(A) with the centred weight,
 *                 bf16((A * rsqrt(mean(A^2) + norm_eps)) * (1 + norm_weight)) per token row, formed
 *                 while the kernel stages them: the bits nvfp4_rmsnorm would store, up to the FP32
 *                 summation order of mean(A^2), without the kernel or the round trip (the
 *                 reference fuses the norm into its BF16 GEMV only, src/engine/layer.cu:217-222; its
 *                 FP4 path runs invoke_rmsnorm first, :190-193).  Not together with swiglu_up or
 *                 k_valid.  Every CTA normalises for itself, so this pays for a few tokens only.
 *   swiglu_epilogue  non-zero: the weight is a merged gate/up tensor whose rows were interleaved in
 *                 slabs of 16 (rows 16s..16s+7 = gate rows 8s..8s+7, rows 16s+8..16s+15 = their up rows:
 *                 nvfp4_interleave_gate_up in nvfp4_checkpoint.h does it at load time); C is then
 *                 [M, N/2] = bf16(silu(gate) * up) with gate and up rounded to BF16 first, i.e. the bits
 *                 of nvfp4_linear followed by nvfp4_swiglu, without the [M, N] round trip and the second
 *                 kernel.  N % 16 == 0, no residual, no px.  More than 16 tokens: N % 32 == 0, no other
 *                 option (the tcgen05 GEMM's epilogue; NVFP4_E_LIMIT otherwise).
 * Zero / NULL fields mean "not used".  No reference counterpart for the fused forms. */
typedef struct nvfp4_linear_desc {
    const void* A;
    const void* swiglu_up;
    long long a_row_stride;
    int k_valid;
    int M;
    const uint8_t* packed;
    const uint8_t* scale;
    float global_scale;
    int N, K;
    const void* residual;
    void* C;
    const nvfp4_peer_exchange* px;
    const void* norm_weight;
    float norm_eps;
    int swiglu_epilogue;
} nvfp4_linear_desc;
int nvfp4_linear_ex(nvfp4_handle* h, const nvfp4_linear_desc* desc, nvfp4_stream_t stream);

/* A chain: a fixed sequence of linears, each with up to 8 tokens and K % 256 == 0 and any of the options of
 * nvfp4_linear_desc, executed in order by ONE launch of the GEMV kernel.  Linear i+1 may read what linear i
 * wrote (the activations, the residual stream): between two linears all CTAs meet at a grid-wide barrier
 * in device memory.  Meanwhile the kernel's loader keeps streaming the next linear's weights into its
 * shared-memory ring -- weights depend on nothing -- and the per-launch cost is paid once.  (Measured on a
 * B200 this saves launches, not time: separate launches with programmatic dependent launch overlap what the
 * barrier serialises, and a 64-layer token step takes 3.97 ms as a chain against 3.63 ms.)  The reference runs
 * one kernel per projection (src/engine/layer.cu:62-110, 190-217, 404-409): a decode layer's sequence
 * o-projection + residual -> RMSNorm -> gate_up -> SwiGLU -> down + residual, or all layers of a token
 * step, is one chain here.
 * The descriptors are read at creation: pointers, shapes and options are frozen into the chain (buffers
 * are fixed, their contents change from run to run, as in a captured decode step).  A run adds one launch;
 * it may be captured in a CUDA graph and replayed (the barrier and the split-tile tags count in device
 * memory, nothing comes from the host).  All CTAs of the launch must be resident at the same time: the
 * grid is one CTA per SM, so nothing else may occupy whole SMs of the device for the duration; a barrier
 * that is not met within about a second sets the handle's status word (0x9xx) and the launch winds down.
 * NVFP4_E_LIMIT: a linear the 8-token kernel does not take, or activations that leave no room for the ring.
 * No reference counterpart. */
typedef struct nvfp4_chain nvfp4_chain;
int nvfp4_chain_create(nvfp4_handle* h, const nvfp4_linear_desc* descs, int n, nvfp4_chain** out);
int nvfp4_chain_run(nvfp4_chain* chain, nvfp4_stream_t stream);
int nvfp4_chain_destroy(nvfp4_chain* chain);

/* Two linears sharing A: C1 = A*W1^T, C2 = A*W2^T, both [N,K].
 * Replaces invoke_fp4_dual_gemv (:395-416), generalised to any M. */
int nvfp4_linear_dual(nvfp4_handle* h, const void* A_bf16, int M,
                      const uint8_t* packed1, const uint8_t* scale1, float global_scale1,
                      const uint8_t* packed2, const uint8_t* scale2, float global_scale2,
                      int N, int K, void* C1_bf16, void* C2_bf16, nvfp4_stream_t stream);

/* Load-time check of a weight's block scales [N, K/16] (device memory): *count (may be NULL) = how many
 * of the bytes are 0x7F or 0xFF, which the reference's decoder (dense_gemm_fp4_sm110.cu:30-41) reads as
 * 480 and the tensor core's FP8 E4M3 as NaN.  If there are any, the handle remembers the pointer and
 * every later call on that scale tensor takes the kernels that decode the scale as the reference does,
 * so its results match the reference on such a weight too; a later scan that finds none forgets it.
 * Synchronises the stream and allocates 8 bytes for the duration of the call: not for capture, not
 * for the decode loop.  No counterpart in the reference, whose one decoder needs none. */
int nvfp4_scan_scales(nvfp4_handle* h, const uint8_t* scale_ue4m3, int N, int K, long long* count,
                      nvfp4_stream_t stream);

/* out[n,k] = bf16( e2m1 * (ue4m3 * (1.0f/global_scale)) ), bit-exact to
 * fp4_dequant_kernel (:444-467). */
int nvfp4_dequant_bf16(nvfp4_handle* h, const uint8_t* packed, const uint8_t* scale_ue4m3,
                       float global_scale, int N, int K, void* out_bf16, nvfp4_stream_t stream);

/* out[M,I] = bf16( silu(gate) * up ).  up != NULL: gate and up are [M,I]
 * (invoke_swiglu, src/engine/light_ops.cu:172-208).  up == NULL: gate points at
 * a merged [M,2I] tensor, gate = cols [0,I), up = cols [I,2I)
 * (invoke_swiglu_merged, src/engine/light_ops.cu:1542-1587). */
int nvfp4_swiglu(nvfp4_handle* h, const void* gate_bf16, const void* up_bf16_or_null,
                 int M, int I, void* out_bf16, nvfp4_stream_t stream);

/* C[M,N] = A[M,K] * W^T (+ residual) for a weight that stayed BF16 in the checkpoint (lm_head, the
 * linear-attention projections): W is [N,K] row-major BF16, the reference's "[K,N] column major".
 * Replaces invoke_dense_gemv / invoke_dense_gemv_add / invoke_dense_gemm(_add)
 * (src/engine/dense_gemm.h:44-115).  Up to 16 tokens (K % 128 == 0) run the HBM-bound GEMV kernel
 * (TMA ring + mma.sync BF16, FP32 accumulation, residual added before the only rounding); more tokens
 * (K % 256 == 0, N % 8 == 0) run the tcgen05 GEMM of the quantised path with the weight blocks loaded
 * straight into the operand buffers; other shapes fall back to a plain CUDA-core GEMM: correct,
 * not fast.  residual may alias C. */
int nvfp4_linear_bf16(nvfp4_handle* h, const void* A_bf16, int M, const void* W_bf16, int N, int K,
                      const void* residual_bf16_or_null, void* C_bf16, nvfp4_stream_t stream);

/* out[M,K] = bf16( (x * rsqrt(mean(x^2) + eps)) * (1 + weight) ) per token row, FP32 inside
 * (invoke_rmsnorm, src/engine/light_ops.cu:65-112; the centred weight of the reference's model).
 * K % 8 == 0; out may alias x. */
int nvfp4_rmsnorm(nvfp4_handle* h, const void* x_bf16, const void* weight_bf16, float eps, int M, int K,
                  void* out_bf16, nvfp4_stream_t stream);
/* residual += bias (rounded once to BF16, in place), norm_out = rmsnorm of the unrounded sum
 * (invoke_fused_add_rmsnorm, src/engine/light_ops.cu:270-328: the step in front of the MLP,
 * src/engine/layer.cu:47-50). */
int nvfp4_add_rmsnorm(nvfp4_handle* h, void* residual_bf16, const void* bias_bf16, const void* weight_bf16, float eps,
                      int M, int K, void* norm_out_bf16, nvfp4_stream_t stream);

/* Same with explicit row strides (in elements): gate and up rows are in_stride apart, output
 * rows out_stride apart.  Used where the SwiGLU output feeds a K-padded weight shard. */
int nvfp4_swiglu_strided(nvfp4_handle* h, const void* gate_bf16, const void* up_bf16, int M, int I,
                         long long in_stride, void* out_bf16, long long out_stride, nvfp4_stream_t stream);
/* The same on the output of a linear whose gate/up weight rows were interleaved in slabs of 16
 * (nvfp4_interleave_gate_up): gate_up rows hold 8 gate values, their 8 up values, 8 gate values, ...;
 * out[M,I].  I % 8 == 0; row strides in elements. */
int nvfp4_swiglu_interleaved(nvfp4_handle* h, const void* gate_up_bf16, int M, int I, long long in_stride,
                             void* out_bf16, long long out_stride, nvfp4_stream_t stream);

/* ---- reference-shaped entry points --------------------------------------
 * Same argument meaning as the reference functions of the same name (void
 * return, no validation surfaced); they run on a lazily created per-device
 * default handle and stash the status for nvfp4_last_status().  The C++ shim
 * nvfp4_qwen_thor_shim.hpp maps qwen_thor::ops::invoke_fp4_* onto these. */
void nvfp4_invoke_fp4_gemv(const void* A, const nvfp4_quantized_weight* W, void* C,
                           nvfp4_stream_t stream);
void nvfp4_invoke_fp4_gemv_add(const void* A, const nvfp4_quantized_weight* W, void* C,
                               const void* residual, nvfp4_stream_t stream);
void nvfp4_invoke_fp4_dual_gemv(const void* A, const nvfp4_quantized_weight* W1,
                                const nvfp4_quantized_weight* W2, void* C1, void* C2,
                                nvfp4_stream_t stream);
void nvfp4_invoke_fp4_gemm(const void* A, const nvfp4_quantized_weight* W, void* C, int M,
                           nvfp4_stream_t stream);
void nvfp4_invoke_fp4_gemm_add(const void* A, const nvfp4_quantized_weight* W, void* D,
                               const void* residual, int M, nvfp4_stream_t stream);
void nvfp4_init_fp4_cublaslt(void);    /* init_fp4_cublaslt (:430-434): creates the default handle */
void nvfp4_cleanup_fp4_cublaslt(void); /* cleanup_fp4_cublaslt (:436-441): destroys it */
int nvfp4_last_status(void);
/* Workspace of the default handle; call before its first use (default 64 MiB). */
int nvfp4_default_handle_workspace(size_t bytes);

/* A handle serves one host thread and one stream at a time: its workspace holds the kernels'
 * cross-CTA scratch, and calls that overlap on the GPU would race on it. */

/* ---- host-memory convenience (the end-to-end path of the benchmark) ------
 * Same as nvfp4_linear but A, residual and C are HOST pointers (pinned for
 * best speed); copies A (and residual) to the device, runs the layer on the
 * handle's staging buffers, copies C back and synchronises the stream.
 * Weights stay device-resident, as in the reference engine.  Staging space
 * comes out of the handle workspace.  Without a residual, a pinned (device-mapped) C_host of up
 * to 2 MB is written by the kernels themselves, with no copy back (5 us per call less); option
 * "host_direct_out" = 0 always stages. */
int nvfp4_linear_host(nvfp4_handle* h, const void* A_host, int M,
                      const uint8_t* packed_dev, const uint8_t* scale_dev, float global_scale,
                      int N, int K, const void* residual_host_or_null, void* C_host,
                      nvfp4_stream_t stream);

/* Reads the sticky device-side status word of the handle (synchronises the device).
 * 0 = no kernel of this handle ever gave up a bounded wait; otherwise the code of the first
 * wait that ran out (0x1xx producer ring slot, 0x2xx consumer ring slot, 0x300 cross-CTA
 * partial flag, 0x4xx tensor-core pipeline). */
int nvfp4_device_status(nvfp4_handle* h, unsigned int* status);

/* Number of kernels this library has launched on the handle since creation. */
int nvfp4_launch_count(nvfp4_handle* h, unsigned long long* count);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H */
