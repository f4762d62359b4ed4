// Decode dequant-GEMV for M <= 16: a persistent, HBM-bound kernel.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W = e2m1(code) * ue4m3(scale) / global_scale
//
// Structure (one CTA per SM, 1 producer warp + 16 consumer warps in two groups of 8):
//   * The weight matrix is cut into half-units of 128 rows x 256 k (16 KB of packed codes + 2 KB
//     of block scales).  The half-units, ordered row-tile-major, are split evenly over the CTAs
//     ("stream-K"): every CTA streams the same number of bytes (+-1 half-unit) whatever N, K are.
//   * The producer warp feeds a multi-stage shared-memory ring with TMA tile copies (packed codes
//     with the 128-byte swizzle, scales), completing on the stage's mbarrier.  A stage carries two
//     consecutive half-units (36 KB): large enough that one issuing thread keeps HBM busy.  No
//     cluster multicast anywhere.
//   * Consumer group h works on half-unit h of every stage (two groups in a 17-warp CTA, one in a
//     9-warp CTA, see GROUPS); each of a group's 8 warps owns 16 of the 128
//     rows.  Codes are expanded in registers: cvt.rn.f16x2.e2m1x2 turns one packed byte into two
//     exact FP16 values, one f16x2 multiply applies the block scale, formed without a table: the
//     unsigned E4M3 byte shifted left by 7 IS the scale / 2^8 as an FP16 bit pattern (subnormal
//     codes included).  Every product lut*scale/2^8 is exact in FP16 (2 + 4 significant bits, all
//     within [2^-18, 11.25]); the 2^8 returns in the FP32 epilogue.  The dot products run on the
//     tensor cores (mma.sync m16n8k16, weights as the 16-row operand, the <= 8 tokens as the
//     8-column operand) with FP32 accumulators --
//     CUDA cores alone cannot convert AND multiply-accumulate 0.56 B/element at HBM speed.
//   * Activations: the CTA's whole k range stays resident in shared memory as FP16, converted
//     once by the consumer warps with an exact per-token power-of-two scale (largest magnitude ->
//     [2^14, 2^15)), so BF16's wider exponent range costs nothing; the scale is undone in FP32.
//     More than 8 tokens, or activations too large for shared memory, run as several launches.
//   * A row tile whose K range is split over several CTAs is finished by the CTA that holds its
//     first half-unit: the others store their FP32 partials to the handle's scratch as 8-byte
//     {value, launch epoch} pairs (one transaction each, so a pair is its own arrival flag: no
//     fence, no flag write, one L2 round trip for the reader); the owner adds them in a fixed
//     order (deterministic), clears the slots it has read (so a replayed launch, which carries
//     the same tag, never meets the previous replay's pairs), applies 2^8/global_scale and the
//     residual in FP32 and rounds once to BF16.  Its wait on the pairs is bounded.
//
// Arithmetic: group products are summed in FP32 by the MMA, block scales are applied exactly
// before the sum (they are exact), 1/global_scale once at the end.  This is the reference's
// GEMV arithmetic (src/engine/dense_gemm_fp4_sm110.cu:96-141, :192-240) up to FP32 summation
// order.
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>
#include <vector>

#include "exchange_layout.h"
#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "gemv_common.cuh"
#include "ptx.cuh"
#include "umma.cuh"

namespace nvfp4 {
namespace {

using namespace gemv;


// GROUPS consumer groups per CTA; group h takes half-unit h of every stage, so a stage carries
// GROUPS half-units.  GROUPS = 2: one 17-warp CTA per SM (what the library uses).  GROUPS = 1:
// 9-warp CTAs, two per SM when the activations are small (measured slower).
constexpr int kMaxTokens = 8;                     // tokens per launch (one 8-column MMA tile)
constexpr uint32_t kTxBytes = kPackedBytes + kScaleBytes;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 227 * 1024;           // one CTA per SM
constexpr int kSmemBudgetHalf = 113 * 1024;       // two CTAs per SM

struct DecodeParams {
    const __nv_bfloat16* A;         // activations, or the gate half when A_up is set
    const __nv_bfloat16* A_up;      // null, or the up half: the activations are bf16(silu(gate) * up), formed while staging
    long long a_stride;             // elements between token rows of A (and A_up)
    int k_valid;                    // columns >= k_valid are zero (a K padded beyond the tensor)
    const __nv_bfloat16* norm_w;    // null, or [K]: the activations are rmsnorm(A) with the centred weight, formed while staging
    float norm_eps;
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    unsigned char* scratch;
    unsigned char* pairs;  // split-tile partials as {FP32 value, epoch} pairs: [CTA][8 tokens][128 rows] x 8 bytes
    float inv_gs;        // 1 / global_scale
    int M, N, K;         // M <= 8 tokens in this launch
    int units, kchunks;  // total half-units, half-units per row tile
    int stages;          // ring depth (each stage holds up to two half-units)
    int act_slots;       // activation slots (k-chunks of 256) held in shared memory
    int act_all;         // 1 = slot index is the k-chunk, 0 = position in the CTA's span
    int swiglu_out;      // rows interleaved in slabs of 16 (8 gate rows, their 8 up rows): C is [M, N/2] = bf16(silu(gate) * up)
    int out_f32;         // C is FP32 [M,N]: store the scaled sum unrounded (partial results for a later reduction)
    unsigned int epoch;
    // Tensor-parallel K split: world > 0 = push the sums to the ranks' exchange buffers and reduce
    // over the group at the end of this kernel (C then receives the full sum + residual).
    unsigned char* xpeer[xchg::kMaxWorld];
    int xrank, xworld, xslot_pairs;
};
static_assert(sizeof(DecodeParams) % 8 == 0, "DecodeParams is copied in 8-byte pieces");

// A chain: several linears run by ONE launch of the kernel, in order (see nvfp4_chain_run).  The
// per-linear parameters and tensor maps sit in device memory; p0 of the kernel carries what all
// linears share (ring depth, the size of the activation area).
struct ChainArgs {
    const DecodeParams* params;      // [n]
    const CUtensorMap* maps;         // [2 n]: packed codes, block scales
    unsigned long long* counter;     // arrivals of all launches of this chain: + gridDim.x per linear
    int n;
    int act_bytes;                   // resident-activation area: the largest of the linears
};

// Inside a chain a linear reads what an earlier linear of the same launch wrote from another SM: those
// loads go to L2 (this SM's L1 may still hold the buffer's lines from an earlier read); a single linear
// keeps the read-only path.
template <bool CHAIN>
__device__ __forceinline__ uint4 ld_act(const uint4* p) { return CHAIN ? __ldcg(p) : __ldg(p); }
template <bool CHAIN>
__device__ __forceinline__ float ld_res(const __nv_bfloat16* p) {
    if (CHAIN) return __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short*>(p)) << 16);
    return __bfloat162float(*p);
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// CHAIN = false: one linear, parameters in the kernel's own parameter space (nvfp4_linear and its
// variants).  CHAIN = true: ch.n linears one after the other in the same launch.  The producer lane
// walks straight on into the next linear's weights (they depend on nothing), so HBM keeps streaming
// into the ring while the consumer warps finish a linear, meet the other CTAs at a grid-wide barrier
// (the next linear reads what this one wrote) and stage the next activations.  The barrier is a
// 64-bit arrival counter in device memory: every CTA adds one per linear, so a launch adds
// gridDim.x * n in all and the counter's value modulo that is where the current launch began --
// nothing comes from the host, a captured launch can be replayed.  The same launch number tags the
// split-tile pairs, which live in a region of the chain's own.  All CTAs must be resident at once
// (the grid is one CTA per SM); every wait is bounded.
template <int GROUPS, bool CHAIN>
__global__ void __launch_bounds__((kGroupWarps * GROUPS + 1) * 32, 3 - GROUPS)
decode_mma_kernel(const __grid_constant__ CUtensorMap tm_packed0, const __grid_constant__ CUtensorMap tm_scale0,
                  const __grid_constant__ DecodeParams p0, const __grid_constant__ ChainArgs ch) {
    constexpr int kConsumerWarps = kGroupWarps * GROUPS;
    constexpr int kConsumerThreads = kConsumerWarps * 32;
    constexpr int kThreads = kConsumerThreads + 32;   // + producer warp
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by an offset on the shared-memory array itself: the pointer keeps its
    // address space, so every access below is a shared-memory instruction with a 32-bit address
    // (rounding a generic 64-bit pointer instead turns them into generic loads and stores).
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int stages = p0.stages;
    unsigned char* s_packed = smem;                                       // stages x GROUPS x 16 KB, 1024-aligned
    unsigned char* s_scale = s_packed + stages * GROUPS * kPackedBytes;   // stages x GROUPS x 2 KB
    unsigned char* s_act = s_scale + stages * GROUPS * kScaleBytes;       // slots x M x 512 B of FP16
    float* s_out = reinterpret_cast<float*>(s_act + (CHAIN ? ch.act_bytes : p0.act_slots * p0.M * kActRowBytes));   // 2 FP32 exchange tiles
    float* s_tokscale = s_out + 2 * kMaxTokens * kOutLd;                  // [0..7] scale, [8..15] 1/scale per token
    unsigned int* s_amax = reinterpret_cast<unsigned int*>(s_tokscale + 16);   // [0..7] largest |activation| bits per token
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_amax + 16);
    uint64_t* empty_bar = full_bar + kMaxStages;
    volatile int* s_abort = reinterpret_cast<volatile int*>(empty_bar + kMaxStages);
    unsigned long long* s_chain_base = reinterpret_cast<unsigned long long*>(const_cast<int*>(s_abort) + 4);   // [0] counter at launch start
    DecodeParams* s_params = reinterpret_cast<DecodeParams*>(s_chain_base + 2);   // CHAIN: the current linear's parameters (16-byte aligned)

    unsigned int* status = reinterpret_cast<unsigned int*>(p0.scratch);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int n_linears = CHAIN ? ch.n : 1;
    // This CTA's half-units [u_begin, u_end) of the first (or only) linear: worked out before the waits below.
    // A chain's grid may exceed a linear's half-units: the first Ge CTAs share them, the others idle through it.
    int Ge = CHAIN && p0.units < G ? p0.units : G;
    int u_begin = cta < Ge ? (int)((long long)cta * p0.units / Ge) : 0;
    int u_end = cta < Ge ? (int)((long long)(cta + 1) * p0.units / Ge) : 0;
    int kc_begin = (int)(u_begin % p0.kchunks);

    // The producer lane sets the ring up itself and starts streaming weights at once; the
    // consumers meet it at named barrier 2 (they need the initialised mbarriers, it needs nothing
    // from them), so the first stages are in flight while the activations are still being staged.
    if (warp == kConsumerWarps) {
        if (lane == 0) {
            for (int s = 0; s < stages; ++s) {
                ptx::mbar_init(&full_bar[s], 1);                  // the producer's expect_tx arrive
                ptx::mbar_init(&empty_bar[s], kConsumerWarps);    // every consumer warp releases every stage
            }
            *s_abort = 0;
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::named_barrier_arrive(2, kThreads);
    }
    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer warp
        if (lane == 0) {
            const uint64_t pol_stream = ptx::policy_evict_first();
            int stage = 0;
            uint32_t ph = 0;
          for (int l = 0; l < n_linears; ++l) {
            const CUtensorMap& tm_packed = CHAIN ? ch.maps[2 * l] : tm_packed0;
            const CUtensorMap& tm_scale = CHAIN ? ch.maps[2 * l + 1] : tm_scale0;
            const DecodeParams& p = CHAIN ? ch.params[l] : p0;
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
            const int p_units = p.units, p_kchunks = p.kchunks;
            if (CHAIN && l > 0) {
                Ge = p_units < G ? p_units : G;
                u_begin = cta < Ge ? (int)((long long)cta * p_units / Ge) : 0;
                u_end = cta < Ge ? (int)((long long)(cta + 1) * p_units / Ge) : 0;
                kc_begin = (int)(u_begin % p_kchunks);
            }
            int hu = u_begin;
            int tile = (int)(u_begin / p_kchunks);
            int kc = kc_begin;                                // k-chunk of hu inside its row tile
            while (hu < u_end) {
                const int tile_end = hu - kc + p_kchunks;
                const int seg_end = tile_end < u_end ? tile_end : u_end;
                const int row0 = tile * kRT;
                while (hu < seg_end) {
                    const int cnt = (seg_end - hu) >= GROUPS ? GROUPS : 1;
                    ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, 0x100u + (unsigned)stage);
                    const int k0 = kc * kKC;
                    ptx::mbar_arrive_expect_tx(&full_bar[stage], kTxBytes * cnt);
                    for (int h = 0; h < cnt; ++h) {
                        ptx::tma_load_2d(s_packed + (stage * GROUPS + h) * kPackedBytes, &tm_packed, &full_bar[stage],
                                         (k0 + h * kKC) >> 1, row0, pol_stream);
                        ptx::tma_load_2d(s_scale + (stage * GROUPS + h) * kScaleBytes, &tm_scale, &full_bar[stage],
                                         (k0 + h * kKC) >> 4, row0, pol_stream);
                    }
                    hu += cnt;
                    kc += cnt;
                    if (++stage == stages) { stage = 0; ph ^= 1u; }
                }
                if (kc >= p_kchunks) { kc = 0; ++tile; }
            }
          }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int grp = warp / kGroupWarps, gw = warp % kGroupWarps;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = gw * 16 + g;                                // tile rows r0 and r0 + 8
    // Shared-memory offsets that do not change from stage to stage.
    const int off_w0 = r0 * 128 + (((2 * t) ^ g) << 4);       // row r0, logical 16-byte chunk 2t   (swizzle: chunk ^ (row & 7))
    const int off_w1 = r0 * 128 + (((2 * t + 1) ^ g) << 4);   // row r0, chunk 2t+1
    const int off_s = r0 * 16 + 4 * t;                         // 4 scale bytes: blocks 4t..4t+3 of the row

    // Programmatic dependent launch: the next kernel of the stream may start its own weight
    // streaming while this grid drains; whatever depends on the previous grid (activations,
    // residual, the outputs and the cross-CTA scratch) is only touched after griddep_wait().
    ptx::griddep_launch_dependents();
    if (!CHAIN && tid < 16) s_amax[tid] = 0u;
    ptx::named_barrier_sync(2, kThreads);            // mbarriers initialised (the producer only arrives)
    if (!CHAIN) ptx::named_barrier_sync(1, kConsumerThreads);

    // Resident activations.  Chunk id = (slot * M + token) * 32 + c names 8 consecutive k of one
    // token; every thread takes ids tid, tid + 512, ... four at a time so that the loads overlap.
    // Pass A finds, per token, the largest magnitude over the k range this CTA works on; the
    // per-token power-of-two scale maps it to [2^14, 2^15), so the FP16 copy loses nothing that
    // matters (an element keeps all 8 significant bits unless it is below 2^-28 of the largest)
    // and never overflows.  Pass B converts and stores in natural k order.  The scale is undone in
    // FP32 in the epilogue.
    ptx::griddep_wait();
    int stage = 0;
    uint32_t ph = 0;
    unsigned long long chain_base = 0;       // CHAIN: the arrival counter's value where this launch began
    if (CHAIN) {
        // No CTA passes the first barrier before this one has arrived there, so at most gridDim.x - 1
        // arrivals of this launch are in the value read here: rounding down to a multiple of a launch's
        // total gives the launch's starting point, the same in every CTA.
        if (tid == 0) {
            const unsigned long long v = ld_acquire_gpu_u64(ch.counter);
            const unsigned long long per_launch = (unsigned long long)G * (unsigned long long)n_linears;
            s_chain_base[0] = v - v % per_launch;
        }
    }
  for (int l = 0; l < n_linears; ++l) {
    if (CHAIN) {
        // this linear's parameters into shared memory; the previous linear is behind a CTA-wide barrier
        if (tid < (int)(sizeof(DecodeParams) / 8))
            reinterpret_cast<uint2*>(s_params)[tid] = __ldg(reinterpret_cast<const uint2*>(ch.params + l) + tid);
        if (tid < 16) s_amax[tid] = 0u;
        ptx::named_barrier_sync(1, kConsumerThreads);
        chain_base = s_chain_base[0];
        if (l > 0) {
            // Grid-wide barrier: every CTA has stored its share of the previous linear's outputs (it arrives
            // behind a CTA barrier and a fence), and this linear may read them.  Thread 0 polls, the others
            // wait for it at the CTA barrier.  Bounded: a CTA that is not resident would otherwise hang us.
            if (tid == 0) {
                const unsigned long long target = chain_base + (unsigned long long)G * (unsigned long long)l;
                const long long t0 = clock64();
                while (ld_acquire_gpu_u64(ch.counter) < target) {
                    if (*s_abort || clock64() - t0 > ptx::kWaitBudgetClocks) {
                        *s_abort = 1;
                        atomicCAS(status, 0u, 0x900u + (unsigned)(l & 0xFF));
                        break;
                    }
                }
            }
            ptx::named_barrier_sync(1, kConsumerThreads);
        }
    }
    const DecodeParams& p = CHAIN ? *s_params : p0;
    unsigned char* pairs = p.pairs;
    // CHAIN: (number of linears all launches of this chain have run before this one) * 2 + 1: odd, never 0, new for every linear of every launch
    const unsigned int epoch = CHAIN ? (unsigned int)((chain_base / (unsigned long long)G) + (unsigned long long)l) * 2u + 1u : p.epoch;
    const int tok = g < p.M ? g : 0;                           // token feeding MMA column g (columns >= M are never stored)
    if (CHAIN && l > 0) {
        Ge = p.units < G ? p.units : G;
        u_begin = cta < Ge ? (int)((long long)cta * p.units / Ge) : 0;
        u_end = cta < Ge ? (int)((long long)(cta + 1) * p.units / Ge) : 0;
        kc_begin = (int)(u_begin % p.kchunks);
    }
    // Group reduction: this launch's epoch and slot set (the counter was advanced by the previous
    // launch -- or the previous linear of this chain -- that used the buffer, which has completed by now).
    unsigned int xepoch = 0, xset = 0;
    if (p.xworld > 0) {
        xepoch = *reinterpret_cast<volatile unsigned int*>(p.xpeer[p.xrank] + xchg::kEpochOff) + 1u;
        xset = xepoch & 1u;
    }
    if (p.norm_w) {
        // RMSNorm on the fly (rmsnorm_kernel, src/engine/light_ops.cu:65-106): every CTA reads the
        // whole rows once for the sum of squares and for the largest |x (1 + w)| -- that times
        // 1/rms bounds the normalised row, which is what the FP16 scale needs.  A warp's 32 lanes
        // hold 32 consecutive chunks of one token; warp w adds its share of token t into
        // s_part[w][t] in loop order, so the sum has a fixed order.
        float* s_part = s_out;                                // [kConsumerWarps][8], free until the first epilogue
        if (tid < kConsumerWarps * 8) s_part[tid] = 0.0f;
        ptx::named_barrier_sync(1, kConsumerThreads);
        const int row_chunks = p.K >> 3;                      // a multiple of 32
        const int total = p.M * row_chunks;
        for (int base = tid; base < total; base += 4 * kConsumerThreads) {
            uint4 x[4], w[4];
            int tk[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int id = base + u * kConsumerThreads;
                x[u] = w[u] = make_uint4(0u, 0u, 0u, 0u);
                tk[u] = -1;
                if (id < total) {
                    tk[u] = id / row_chunks;
                    const int c = id - tk[u] * row_chunks;
                    x[u] = ld_act<CHAIN>(reinterpret_cast<const uint4*>(p.A + (size_t)tk[u] * p.a_stride) + c);
                    w[u] = __ldg(reinterpret_cast<const uint4*>(p.norm_w) + c);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (tk[u] < 0) continue;                      // uniform across the warp
                const uint32_t xv[4] = {x[u].x, x[u].y, x[u].z, x[u].w}, wv[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
                float ss = 0.0f, mt = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float x0 = __uint_as_float(xv[i] << 16), x1 = __uint_as_float(xv[i] & 0xFFFF0000u);
                    const float w0 = 1.0f + __uint_as_float(wv[i] << 16), w1 = 1.0f + __uint_as_float(wv[i] & 0xFFFF0000u);
                    ss = fmaf(x0, x0, ss);
                    ss = fmaf(x1, x1, ss);
                    mt = fmaxf(mt, fmaxf(fabsf(x0 * w0), fabsf(x1 * w1)));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
                }
                if (lane == 0) {
                    s_part[warp * 8 + tk[u]] += ss;
                    atomicMax(&s_amax[tk[u]], __float_as_uint(mt));
                }
            }
        }
        ptx::named_barrier_sync(1, kConsumerThreads);
        if (tid < p.M) {
            float ss = 0.0f;
            for (int w = 0; w < kConsumerWarps; ++w) ss += s_part[w * 8 + tid];
            const float inv = 1.0f / sqrtf(ss / (float)p.K + p.norm_eps);
            s_amax[8 + tid] = __float_as_uint(inv);
            // the bound of the normalised row, in the BF16 bit pattern the scale selection below reads
            float b = __uint_as_float(s_amax[tid]) * inv;
            b = b < 3.0e38f ? b : 3.0e38f;                    // also catches a NaN row: the scale stays finite
            s_amax[tid] = __float_as_uint(b) >> 16;
        }
        // the staging passes below end with barriers of their own before s_amax[8..] is read
    }
    {
        const int per_slot = p.M * 32;
        const int total = p.act_slots * per_slot;
        const int kc0 = p.act_all ? 0 : kc_begin;
        auto chunk_src = [&](int id, int& j, int& tk, int& c) -> const uint4* {
            j = id / per_slot;
            const int r = id - j * per_slot;
            tk = r >> 5;
            c = r & 31;
            int kc = kc0 + j;
            if (kc >= p.kchunks) kc -= p.kchunks;
            const int k = kc * kKC + c * 8;
            return k < p.k_valid ? reinterpret_cast<const uint4*>(p.A + (size_t)tk * p.a_stride + k) : nullptr;
        };
        // Pass A: one trip to global memory, eight chunks in flight per thread; the raw BF16 chunk
        // goes to its final (swizzled) place, the magnitudes feed the per-token maximum.
        for (int base = tid; base < total; base += 8 * kConsumerThreads) {
            uint4 x[8];
            int tk[8], dst[8];      // dst: byte offset of the chunk; -1 = no chunk, <= -2 = a zero chunk (encodes -2 - offset)
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                x[u] = make_uint4(0u, 0u, 0u, 0u);
                tk[u] = 0;
                dst[u] = -1;
                const int id = base + u * kConsumerThreads;
                if (id < total) {
                    int j, c;
                    const uint4* src = chunk_src(id, j, tk[u], c);
                    if (src) x[u] = ld_act<CHAIN>(src);
                    dst[u] = src ? (j * p.M + tk[u]) * kActRowBytes + act_chunk_offset(c) : -2 - ((j * p.M + tk[u]) * kActRowBytes + act_chunk_offset(c));
                }
            }
            if (p.A_up) {
                // SwiGLU on the fly: the up half sits (A_up - A) elements behind the gate half; four
                // chunks at a time keep the registers in bounds.
                const long long up_off = (p.A_up - p.A) / 8;
#pragma unroll
                for (int h4 = 0; h4 < 8; h4 += 4) {
                    uint4 y[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        y[u] = make_uint4(0u, 0u, 0u, 0u);
                        const int id = base + (h4 + u) * kConsumerThreads;
                        if (id < total && dst[h4 + u] >= 0) {
                            int j, tkk, c;
                            y[u] = ld_act<CHAIN>(chunk_src(id, j, tkk, c) + up_off);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (dst[h4 + u] >= 0) x[h4 + u] = swiglu_bf16x8(x[h4 + u], y[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (dst[u] == -1) continue;   // uniform across the warp: total is a multiple of 32
                if (dst[u] < 0) dst[u] = -2 - dst[u];           // a chunk beyond k_valid: stays zero
                const uint32_t v[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
                uint32_t m = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) m = max(m, max(v[i] & 0x7FFFu, (v[i] >> 16) & 0x7FFFu));
                // the 32 lanes of a warp hold the 32 chunks of one (slot, token) row
                m = __reduce_max_sync(0xffffffffu, m);
                if (lane == 0 && m && !p.norm_w) atomicMax(&s_amax[tk[u]], m);
                *reinterpret_cast<uint4*>(s_act + dst[u]) = x[u];
            }
        }
        ptx::named_barrier_sync(1, kConsumerThreads);
        if (tid < p.M) {
            const int e8 = (int)(s_amax[tid] >> 7);           // biased BF16 exponent of the largest element
            int se = 268 - e8;                                // scale = 2^(141 - e8): largest -> exponent 14
            se = se < 1 ? 1 : (se > 254 ? 254 : se);
            s_tokscale[tid] = __uint_as_float((uint32_t)se << 23);
            s_tokscale[8 + tid] = __uint_as_float((uint32_t)(254 - se) << 23);
        }
        ptx::named_barrier_sync(1, kConsumerThreads);
        // Pass B: BF16 -> scaled FP16 in place.  Chunk i of the data sits at row i/32 (row modulo M
        // = its token), position act_chunk_offset(i mod 32) inside the padded row.
        const int nchunks = total;                            // 16-byte data chunks in the resident area
        for (int i = tid; i < nchunks; i += kConsumerThreads) {
            const int row = i >> 5;
            const float sc = s_tokscale[row % p.M];
            uint4* ptr = reinterpret_cast<uint4*>(s_act + row * kActRowBytes + act_chunk_offset(i & 31));
            const uint4 x = *ptr;
            uint32_t v[4] = {x.x, x.y, x.z, x.w};
            if (p.norm_w) {
                // bf16( (x / rms) * (1 + w) ), the bits the separate RMSNorm kernel would have stored
                const int tkn = row % p.M;
                int kc = kc0 + row / p.M;
                if (kc >= p.kchunks) kc -= p.kchunks;
                const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(p.norm_w + kc * kKC) + (i & 31));
                const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
                const float inv = __uint_as_float(s_amax[8 + tkn]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float y0 = __uint_as_float(v[q] << 16) * inv * (1.0f + __uint_as_float(wv[q] << 16));
                    const float y1 = __uint_as_float(v[q] & 0xFFFF0000u) * inv * (1.0f + __uint_as_float(wv[q] & 0xFFFF0000u));
                    const __nv_bfloat162 yb = __floats2bfloat162_rn(y0, y1);
                    v[q] = *reinterpret_cast<const uint32_t*>(&yb);
                }
            }
            uint32_t y[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
                y[q] = ptx::pack_f16x2(__uint_as_float(v[q] << 16) * sc, __uint_as_float(v[q] & 0xFFFF0000u) * sc);
            *ptr = make_uint4(y[0], y[1], y[2], y[3]);
        }
        ptx::named_barrier_sync(1, kConsumerThreads);
    }

    int hu = u_begin;
    int tile = u_begin / p.kchunks;
    int kc = kc_begin;                                         // k-chunk of hu inside its row tile
    int seg_parity = 0;
    while (hu < u_end) {
        const int kc_first = kc;
        const int tile_end = hu - kc + p.kchunks;
        const int seg_end = tile_end < u_end ? tile_end : u_end;

        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

        // Segment bookkeeping known up front.
        const bool owner = (kc_first == 0);
        const bool complete = owner && (seg_end == tile_end);
        const int m0 = 2 * t, m1 = 2 * t + 1;
        const int rr[4] = {r0, r0, r0 + 8, r0 + 8};
        const int mm[4] = {m0, m1, m0, m1};
        int last = cta;                              // contributors are CTAs cta+1 .. last
        float pre[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        bool prefetched = complete;
        bool need_clear = false;
        if (grp == 0 && owner && !complete)
            while (last + 1 < Ge && (long long)(last + 1) * p.units / Ge < tile_end) ++last;
        // The contributors' pairs for this thread's (up to four) outputs, added in CTA order (a fixed
        // summation order).  Two contributors at a time: their eight loads are issued before any
        // is looked at, so they share one L2 round trip.  blocking: wait (bounded) for pairs that
        // do not carry this launch's epoch yet; otherwise give up at the first such pair.
        auto gather_pairs = [&](float (&sum)[4], bool blocking) -> bool {
            const long long t0 = clock64();
            for (int c0 = cta + 1; c0 <= last; c0 += 2) {
                const bool two = c0 + 1 <= last;
                const unsigned char* src = pairs + ((size_t)c0 * (kMaxTokens * kRT)) * 8;
                while (true) {
                    uint2 v[2][4];
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            v[j][i] = make_uint2(0u, epoch);
                            if (mm[i] < p.M && (j == 0 || two))
                                v[j][i] = ptx::ld_volatile_v2(src + ((size_t)j * (kMaxTokens * kRT) + mm[i] * kRT + rr[i]) * 8);
                        }
                    bool ready = true;
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) ready &= (v[j][i].y == epoch);
                    if (ready) {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) sum[i] += __uint_as_float(v[j][i].x);
                        break;
                    }
                    if (!blocking) return false;
                    if (*s_abort || clock64() - t0 > ptx::kWaitBudgetClocks) {
                        *s_abort = 1;
                        atomicCAS(status, 0u, 0x300u);
                        return false;
                    }
                }
            }
            return true;
        };
        // Once a gather has been ACCEPTED (by the whole warp, for the early look) the slots are handed back
        // cleared, at the end of the segment.  The tag comes from the host and a captured CUDA graph replays
        // it unchanged, so a pair left behind would look current to the next replay; a cleared slot cannot.
        // (Each pair has exactly one reader, this thread; the next launch's contributors write only after
        // griddepcontrol.wait, when these stores have landed.  Measured alternatives: a tag from a counter in
        // the scratch costs one atomic per CTA on one address, +0.5 us per launch like these stores; the
        // hardware's %gridid repeats from one replay of a graph to the next and cannot serve.)
        auto clear_pairs = [&]() {
            for (int c = cta + 1; c <= last; ++c) {
                unsigned char* src = pairs + ((size_t)c * (kMaxTokens * kRT)) * 8;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (mm[i] < p.M) ptx::st_volatile_v2(src + ((size_t)mm[i] * kRT + rr[i]) * 8, 0u, 0u);
            }
        };

        while (hu < seg_end) {
            const int cnt = (seg_end - hu) >= GROUPS ? GROUPS : 1;
            const int slot = p.act_all ? kc + grp : (int)(hu - u_begin) + grp;
            hu += cnt;
            kc += cnt;
            // Every warp waits on every stage in order (an mbarrier waiter may not skip a phase);
            // group 1 has nothing to do in a stage that carries a single half-unit.
            ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0x200u + (unsigned)stage);
            // Two stages before the end of an owner's segment: if the contributors have published
            // their partials by now (the usual case: a contributor's share is the first thing it
            // computes), fetch them behind the remaining math; otherwise wait for them at the end.
            // (Looking at the start of the segment instead put two L2 round trips in front of the
            // first stage of every owner: 1.8 us per launch on a B200.)
            if (grp == 0 && owner && !prefetched && seg_end - hu <= 2 * GROUPS) {
                float got[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (__all_sync(0xffffffffu, gather_pairs(got, false))) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) pre[i] = got[i];
                    prefetched = true;
                    need_clear = true;
                }
            }
            if (grp < cnt) {
                const unsigned char* wp = s_packed + (stage * GROUPS + grp) * kPackedBytes;
                const unsigned char* sp = s_scale + (stage * GROUPS + grp) * kScaleBytes + off_s;
                const unsigned char* ap = s_act + (slot * p.M + tok) * kActRowBytes + t * kActBlockBytes;
                const uint4 wa0 = *reinterpret_cast<const uint4*>(wp + off_w0);
                const uint4 wa1 = *reinterpret_cast<const uint4*>(wp + off_w1);
                const uint4 wb0 = *reinterpret_cast<const uint4*>(wp + off_w0 + 8 * 128);
                const uint4 wb1 = *reinterpret_cast<const uint4*>(wp + off_w1 + 8 * 128);
                const uint32_t qa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
                const uint32_t qb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
                // The four block scales of each row (blocks 4t..4t+3 of the half-unit) as f16x2
                // operands: scale / 2^8, formed from the byte without a table.
                uint32_t Sa[4], Sb[4];
                {
                    const uint32_t ba = mask_scale_bytes(*reinterpret_cast<const uint32_t*>(sp));
                    const uint32_t bb = mask_scale_bytes(*reinterpret_cast<const uint32_t*>(sp + 8 * 16));
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        Sa[b] = scale_byte_to_f16x2(ba, b);
                        Sb[b] = scale_byte_to_f16x2(bb, b);
                    }
                }
                float acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // second accumulator: halves the MMA dependency chain
#pragma unroll
                for (int uu = 0; uu < 8; ++uu) {
                    uint32_t da[4], db[4];
                    expand_u32(qa[uu], Sa[uu >> 1], da);
                    expand_u32(qb[uu], Sb[uu >> 1], db);
                    const uint4 x = *reinterpret_cast<const uint4*>(ap + uu * 16);
                    const uint32_t a_lo[4] = {da[0], db[0], da[1], db[1]};   // k 0..3 of this 8-group: rows g, g+8
                    const uint32_t a_hi[4] = {da[2], db[2], da[3], db[3]};   // k 4..7
                    ptx::mma_f16_16x8x16(acc, a_lo, x.x, x.y);
                    ptx::mma_f16_16x8x16(acc2, a_hi, x.z, x.w);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[stage]);
            if (++stage == stages) { stage = 0; ph ^= 1u; }
        }

        // ------------------------------------------------------------ segment epilogue
        // Rows belong to warp pairs (warp gw of either group), so every pair finishes its 16 rows
        // on its own: group 1 hands its sums over through shared memory (two buffers alternating
        // per segment, one 64-thread barrier per segment), group 0 finishes from registers --
        // thread (g,t) holds rows r0, r0+8 x tokens 2t, 2t+1.  The other warps keep streaming.
        float* xchg = s_out + (seg_parity ? kMaxTokens * kOutLd : 0);
        seg_parity ^= 1;
        if (GROUPS == 2) {
            if (grp == 1) {
                xchg[(2 * t) * kOutLd + r0] = acc[0];
                xchg[(2 * t + 1) * kOutLd + r0] = acc[1];
                xchg[(2 * t) * kOutLd + r0 + 8] = acc[2];
                xchg[(2 * t + 1) * kOutLd + r0 + 8] = acc[3];
            }
            ptx::named_barrier_sync(4 + gw, 64);
        }
        if (grp == 0) {
            const float us0 = s_tokscale[8 + m0], us1 = s_tokscale[8 + m1];
            if (GROUPS == 2) {
                acc[0] += xchg[m0 * kOutLd + r0];
                acc[1] += xchg[m1 * kOutLd + r0];
                acc[2] += xchg[m0 * kOutLd + r0 + 8];
                acc[3] += xchg[m1 * kOutLd + r0 + 8];
            }
            float v[4] = {acc[0] * us0, acc[1] * us1, acc[2] * us0, acc[3] * us1};
            if (!owner) {
                // the pair is its own flag: an aligned 8-byte store is one transaction
                unsigned char* slot = pairs + (size_t)cta * (kMaxTokens * kRT) * 8;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (mm[i] < p.M) ptx::st_volatile_v2(slot + (mm[i] * kRT + rr[i]) * 8, __float_as_uint(v[i]), epoch);
            } else {
                if (!prefetched) {
                    if (gather_pairs(pre, true)) need_clear = true;
                    __syncwarp();
                }
                const int row_base = tile * kRT;
                if (p.swiglu_out) {
                    // Thread (g,t) holds gate row 8 gw + g of this tile's 64 pairs (i = 0, 1) and its up row
                    // (i = 2, 3) for tokens 2t, 2t+1: the projection's outputs are rounded to BF16 as the
                    // separate kernels would store them, then silu(gate) * up, one more rounding.
                    const int n_out = tile * (kRT / 2) + gw * 8 + g;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        if (mm[i] >= p.M || row_base + rr[i] >= p.N) continue;
                        const float gate = __bfloat162float(__float2bfloat16_rn(((v[i] + pre[i]) * kBlockScaleUnfold) * p.inv_gs));
                        const float up = __bfloat162float(__float2bfloat16_rn(((v[i + 2] + pre[i + 2]) * kBlockScaleUnfold) * p.inv_gs));
                        p.C[(size_t)mm[i] * (p.N / 2) + n_out] = __float2bfloat16_rn(silu(gate) * up);
                    }
                } else
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = row_base + rr[i];
                    if (mm[i] >= p.M || n >= p.N) continue;
                    float x = ((v[i] + pre[i]) * kBlockScaleUnfold) * p.inv_gs;
                    const size_t o = (size_t)mm[i] * p.N + n;
                    if (p.out_f32) { reinterpret_cast<float*>(p.C)[o] = x; continue; }
                    if (p.xworld > 0) {   // the unrounded sum goes to slot [set][this rank] of every rank's buffer
                        const size_t pair = ((size_t)xset * p.xworld + p.xrank) * p.xslot_pairs + o;
                        for (int q = 0; q < p.xworld; ++q)
                            ptx::st_volatile_v2(p.xpeer[q] + xchg::kSlotsOff + pair * 8, __float_as_uint(x), xepoch);
                        continue;
                    }
                    if (p.residual) x += ld_res<CHAIN>(p.residual + o);
                    p.C[o] = __float2bfloat16_rn(x);
                }
            }
        }
        if (!CHAIN && need_clear) clear_pairs();      // a chain's tags come from the device and never repeat
        if (kc >= p.kchunks) { kc = 0; ++tile; }
    }

    // ---------------------------------------------------------------- reduction over the group
    // Every CTA takes 1/gridDim of the M x N outputs: it polls its own rank's buffer until the
    // pairs of all ranks carry this launch's epoch (bounded), adds them in rank order, adds the
    // residual and rounds once.  The pairs come from the tile owners on every rank, this GPU's
    // own CTAs included: all CTAs of the grid are resident (one per SM) and an owner's push waits
    // for nothing that happens after it, so these waits cannot form a cycle.
    if (p.xworld > 0) {
        unsigned char* mine = p.xpeer[p.xrank];
        const int E = p.M * p.N;
        const int e0 = (int)((long long)cta * E / G), e1 = (int)((long long)(cta + 1) * E / G);
        const long long t0 = clock64();
        bool failed = false;
        for (int e = e0 + tid; e < e1 && !failed; e += kConsumerThreads) {
            float sum = 0.0f;
            for (int q = 0; q < p.xworld && !failed; ++q) {
                const unsigned char* src = mine + xchg::kSlotsOff + (((size_t)xset * p.xworld + q) * p.xslot_pairs + e) * 8;
                uint2 v = ptx::ld_volatile_v2(src);
                while (v.y != xepoch) {
                    if (clock64() - t0 > xchg::kWaitClocks) {
                        atomicCAS(reinterpret_cast<unsigned int*>(mine + xchg::kStatusOff), 0u, 0x700u + (unsigned)q);
                        failed = true;
                        break;
                    }
                    v = ptx::ld_volatile_v2(src);
                }
                sum += __uint_as_float(v.x);
            }
            if (failed) break;
            if (p.residual) sum += ld_res<CHAIN>(p.residual + e);
            p.C[e] = __float2bfloat16_rn(sum);
        }
        // the last CTA to get here advances the launch counter for the next launch
        ptx::named_barrier_sync(1, kConsumerThreads);
        if (tid == 0) {
            __threadfence();
            unsigned int* done = reinterpret_cast<unsigned int*>(mine + xchg::kDoneOff);
            if (atomicAdd(done, 1u) == (unsigned)G - 1u) {
                *done = 0u;
                *reinterpret_cast<volatile unsigned int*>(mine + xchg::kEpochOff) = xepoch;
            }
        }
    }
    if (CHAIN) {
        // This CTA's share of linear l is stored: arrive at the grid-wide barrier (every linear, the last
        // one too: a launch always adds gridDim.x * n to the counter).  The CTA barrier orders every
        // thread's stores before thread 0's fence and arrival.
        ptx::named_barrier_sync(1, kConsumerThreads);
        if (tid == 0) {
            __threadfence();
            atomicAdd(ch.counter, 1ull);
        }
    }
  }   // linears
}

// ------------------------------------------------------------------------------------ host side

// Tensor maps of a weight's packed codes and block scales (uint8, 128 rows per box).
bool make_u8_map(TensorMapCache* cache, CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols,
                 uint32_t box_rows, CUtensorMapSwizzle sw) {
    return umma::make_map_cached(cache, m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, cols, rows, box_cols, box_rows, sw);
}

}  // namespace

bool decode_mma_supported(const LinearArgs& a) {
    if (a.M < 1 || a.M > 16) return false;
    if ((a.K % 256) != 0) return false;   // scale rows (K/16 bytes) must be 16-byte multiples for the tile copy
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u)) return false;
    return true;
}

size_t decode_mma_scratch_bytes(const LinearArgs&, const nvfp4_device_info& dev) {
    return dev.gemv_pairs_offset + (size_t)dev.sm_count * kMaxTokens * kRT * 8;
}

cudaError_t configure_decode_mma() {
    cudaError_t e = configure_large_smem(decode_mma_kernel<2, false>, kSmemBudget);
    if (e != cudaSuccess) return e;
    return configure_large_smem(decode_mma_kernel<2, true>, kSmemBudget);
}

namespace {

// Shared-memory plan of one launch of m <= 8 tokens: the ring gets what the resident
// activations leave, and needs at least three stages.
struct DecodePlan {
    DecodeParams p;
    int grid, smem, groups;
};

constexpr int kFixedSmem = 1024 + 2 * kMaxTokens * kOutLd * 4 + 128 + 2 * kMaxStages * 8 + 32 + 16 + (int)sizeof(DecodeParams) + 16;

// force_grid: a chain runs every linear on the same grid, also one with fewer half-units than CTAs.
bool plan_decode_groups(const LinearArgs& a, int m, int groups, int grid_cap, void* scratch, size_t pairs_offset,
                        DecodePlan* out, bool force_grid = false) {
    DecodeParams p{};
    p.A = static_cast<const __nv_bfloat16*>(a.A);
    p.A_up = static_cast<const __nv_bfloat16*>(a.swiglu_up);
    p.a_stride = a.a_stride ? a.a_stride : a.K;
    p.k_valid = a.k_valid ? a.k_valid : a.K;
    p.norm_w = static_cast<const __nv_bfloat16*>(a.norm_w);
    p.norm_eps = a.norm_eps;
    p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.C = static_cast<__nv_bfloat16*>(a.C);
    p.scratch = static_cast<unsigned char*>(scratch);
    p.pairs = p.scratch + pairs_offset;
    p.inv_gs = a.inv_gs;
    p.M = m; p.N = a.N; p.K = a.K;
    p.out_f32 = a.out_f32 ? 1 : 0;
    p.swiglu_out = a.swiglu_out ? 1 : 0;
    if (a.px) {
        for (int q = 0; q < a.px->world; ++q) p.xpeer[q] = static_cast<unsigned char*>(a.px->peer[q]);
        p.xrank = a.px->rank;
        p.xworld = a.px->world;
        p.xslot_pairs = a.px->slot_pairs;
    }
    p.kchunks = a.K / kKC;
    const long long tiles = (a.N + kRT - 1) / kRT;
    p.units = (int)(tiles * p.kchunks);
    int grid = grid_cap < kMaxGrid ? grid_cap : kMaxGrid;
    if (grid > p.units && !force_grid) grid = p.units;
    const int fixed = kFixedSmem;
    const int stage_w = groups * (kPackedBytes + kScaleBytes);
    const int budget = groups == 2 ? kSmemBudget : kSmemBudgetHalf;
    const int max_span = (p.units + grid - 1) / grid;
    p.act_all = p.kchunks <= max_span ? 1 : 0;
    p.act_slots = p.act_all ? p.kchunks : max_span;
    const long long act_res = (long long)p.act_slots * m * kActRowBytes;
    long long stages = (budget - fixed - act_res) / stage_w;
    if (stages < 3) return false;
    if (stages > kMaxStages) stages = kMaxStages;
    p.stages = (int)stages;
    out->p = p;
    out->grid = grid;
    out->groups = groups;
    out->smem = fixed + (int)stages * stage_w + (int)act_res;
    return true;
}

// One 17-warp CTA per SM.  (Two 9-warp CTAs per SM, GROUPS = 1, measured 1-2 us slower per launch
// on the MLP shapes: both CTAs of an SM start and end together, so nothing overlaps.)
bool plan_decode(const LinearArgs& a, int m, const nvfp4_device_info& dev, void* scratch, DecodePlan* out) {
    return plan_decode_groups(a, m, 2, dev.sm_count, scratch, dev.gemv_pairs_offset, out);
}

// Largest token count per launch (<= 8) whose activations fit beside the ring; 0 if none.
int decode_tokens_per_launch(const LinearArgs& a, const nvfp4_device_info& dev) {
    DecodePlan pl;
    for (int m = a.M < kMaxTokens ? a.M : kMaxTokens; m >= 1; --m)
        if (plan_decode(a, m, dev, nullptr, &pl)) return m;
    return 0;
}

}  // namespace

bool decode_mma_fits(const LinearArgs& a, const nvfp4_device_info& dev) { return decode_tokens_per_launch(a, dev) > 0; }

cudaError_t launch_decode_mma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, int* launches,
                              cudaStream_t s) {
    CUtensorMap tmp, tms;
    if (!make_u8_map(dev.maps, &tmp, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, kRT, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_u8_map(dev.maps, &tms, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, kRT, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    const int per = decode_tokens_per_launch(a, dev);
    if (per <= 0) return cudaErrorInvalidValue;
    int n = 0;
    // More than `per` tokens: one launch per group of tokens (each streams the weights again).
    for (int m0 = 0; m0 < a.M; m0 += per) {
        LinearArgs b = a;
        const int m = a.M - m0 < per ? a.M - m0 : per;
        b.A = static_cast<const char*>(a.A) + (size_t)m0 * (a.a_stride ? a.a_stride : a.K) * 2;
        if (a.swiglu_up) b.swiglu_up = static_cast<const char*>(a.swiglu_up) + (size_t)m0 * (a.a_stride ? a.a_stride : a.K) * 2;
        b.C = static_cast<char*>(a.C) + (size_t)m0 * (a.swiglu_out ? a.N / 2 : a.N) * (a.out_f32 ? 4 : 2);
        if (a.residual) b.residual = static_cast<const char*>(a.residual) + (size_t)m0 * a.N * 2;
        DecodePlan pl;
        if (!plan_decode(b, m, dev, scratch, &pl)) return cudaErrorInvalidValue;
        pl.p.epoch = next_launch_tag();
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(pl.grid);
        cfg.blockDim = dim3((2 * kGroupWarps + 1) * 32);
        cfg.dynamicSmemBytes = pl.smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, decode_mma_kernel<2, false>, tmp, tms, pl.p, ChainArgs{});
        ++n;
        if (e != cudaSuccess) { if (launches) *launches = n; return e; }
    }
    if (launches) *launches = n;
    return cudaSuccess;
}

}  // namespace nvfp4

// ----------------------------------------------------------------------------------------------
// Chains: a fixed sequence of linears (up to 8 tokens each) run by one launch of the kernel.
namespace nvfp4 {

struct DecodeChain {
    unsigned char* dev = nullptr;      // counter | parameters | tensor maps | split-tile pairs
    DecodeParams p0{};
    ChainArgs ch{};
    CUtensorMap map0, map1;            // stand-ins for the kernel's own map parameters (unused by a chain)
    int grid = 0, smem = 0, n = 0;
};

void destroy_decode_chain(DecodeChain* c) {
    if (!c) return;
    cudaFree(c->dev);
    delete c;
}

// status: NVFP4_OK, NVFP4_E_LIMIT (a linear the 8-token kernel does not take, or activations that leave
// no room for the ring), or a CUDA error code.
int create_decode_chain(const LinearArgs* linears, int n, const nvfp4_device_info& dev, void* scratch, DecodeChain** out) {
    *out = nullptr;
    if (n < 1 || n > 4096) return NVFP4_E_SHAPE;
    const int grid = dev.sm_count < kMaxGrid ? dev.sm_count : kMaxGrid;
    std::vector<DecodeParams> params((size_t)n);
    std::vector<CUtensorMap> maps((size_t)2 * n);
    long long act_max = 0;
    for (int l = 0; l < n; ++l) {
        const LinearArgs& a = linears[l];
        if (a.M < 1 || a.M > kMaxTokens || !decode_mma_supported(a)) return NVFP4_E_LIMIT;
        DecodePlan pl;
        if (!plan_decode_groups(a, a.M, 2, grid, scratch, 0, &pl, true)) return NVFP4_E_LIMIT;
        params[l] = pl.p;
        const long long act = (long long)pl.p.act_slots * a.M * kActRowBytes;
        act_max = act > act_max ? act : act_max;
        if (!make_u8_map(nullptr, &maps[2 * l], a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, kRT, CU_TENSOR_MAP_SWIZZLE_128B) ||
            !make_u8_map(nullptr, &maps[2 * l + 1], a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, kRT, CU_TENSOR_MAP_SWIZZLE_NONE))
            return (int)cudaErrorInvalidValue;
    }
    const int stage_w = 2 * (kPackedBytes + kScaleBytes);
    long long stages = (kSmemBudget - kFixedSmem - act_max) / stage_w;
    if (stages < 3) return NVFP4_E_LIMIT;
    if (stages > kMaxStages) stages = kMaxStages;
    const size_t off_params = 256;
    const size_t off_maps = (off_params + (size_t)n * sizeof(DecodeParams) + 127) / 128 * 128;
    const size_t off_pairs = (off_maps + (size_t)2 * n * sizeof(CUtensorMap) + 255) / 256 * 256;
    const size_t bytes = off_pairs + (size_t)grid * kMaxTokens * kRT * 8;
    DecodeChain* c = new DecodeChain();
    cudaError_t e = cudaMalloc((void**)&c->dev, bytes);
    if (e == cudaSuccess) e = cudaMemset(c->dev, 0, bytes);
    for (int l = 0; l < n; ++l) {
        params[l].stages = (int)stages;
        params[l].pairs = c->dev ? c->dev + off_pairs : nullptr;
        params[l].epoch = 0u;
    }
    if (e == cudaSuccess) e = cudaMemcpy(c->dev + off_params, params.data(), (size_t)n * sizeof(DecodeParams), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(c->dev + off_maps, maps.data(), (size_t)2 * n * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { destroy_decode_chain(c); return (int)e; }
    c->p0 = params[0];
    c->ch.params = reinterpret_cast<const DecodeParams*>(c->dev + off_params);
    c->ch.maps = reinterpret_cast<const CUtensorMap*>(c->dev + off_maps);
    c->ch.counter = reinterpret_cast<unsigned long long*>(c->dev);
    c->ch.n = n;
    c->ch.act_bytes = (int)act_max;
    c->map0 = maps[0];
    c->map1 = maps[1];
    c->grid = grid;
    c->n = n;
    c->smem = kFixedSmem + (int)stages * stage_w + (int)act_max;
    *out = c;
    return NVFP4_OK;
}

cudaError_t launch_decode_chain(DecodeChain* c, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(c->grid);
    cfg.blockDim = dim3((2 * kGroupWarps + 1) * 32);
    cfg.dynamicSmemBytes = c->smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_mma_kernel<2, true>, c->map0, c->map1, c->p0, c->ch);
}

}  // namespace nvfp4

// ----------------------------------------------------------------------------------------------
// Allocation-free GEMV entry point.
//
// Some hosts of this library must never call cudaMalloc once they are running: an inference
// engine that sizes its KV-cache pool to whatever device memory is left at start-up (the
// reference engine does) has nothing to give later, so an allocation made by a plug-in can
// fail or push the engine over its own budget; code running under a fixed memory plan is in
// the same position.  For them the GEMV is offered without a handle: the cross-CTA scratch
// (the partial tiles) that nvfp4_linear takes from the handle workspace lives in a
// fixed array in the library's device image instead.
//
// The array costs kNoAllocScratchBytes (about 1.3 MB) on every GPU that loads the library, for
// the life of the process.  Limits that follow from its fixed size and from the absence of a
// workspace: at most 160 CTAs (the grid is capped there), M <= 16, K % 256 == 0, and the
// activations of 8 tokens or fewer must fit in shared memory beside the weight ring; anything
// else is refused with NVFP4_E_LIMIT.
namespace nvfp4 {
namespace {

constexpr int kNoAllocMaxGrid = 160;
constexpr size_t kNoAllocScratchBytes = kPartialOffset + (size_t)kNoAllocMaxGrid * kMaxTokens * kRT * 8;

// File-scope device array: in HOST code this name is only a handle for the runtime, not an
// address a kernel can use.  noalloc_setup() asks the runtime for the real device address
// (cudaGetSymbolAddress) once per device and the kernel is always given that pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct NoAllocState {
    bool ready = false;
    void* scratch = nullptr;      // device address of g_noalloc_scratch on this device
    nvfp4_device_info dev{};
};
NoAllocState g_noalloc[64];
std::mutex g_noalloc_mu;

// Once per device, with that device current: device facts, the kernel's shared-memory opt-in
// and the device address of the scratch array.  Nothing here allocates.
int noalloc_setup(int device, NoAllocState** out) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocState& st = g_noalloc[device];
    if (!st.ready) {
        int sms = 0, major = 0;
        cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) return (int)e;
        if (major != 10) return NVFP4_E_DEVICE;
        e = configure_decode_mma();
        if (e != cudaSuccess) return (int)e;
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) return e != cudaSuccess ? (int)e : NVFP4_E_DEVICE;
        st.scratch = ptr;
        st.dev.device = device;
        st.dev.sm_count = sms < kNoAllocMaxGrid ? sms : kNoAllocMaxGrid;   // the grid never exceeds the scratch
        st.dev.cc_major = major;
        st.dev.gemv_pairs_offset = kPartialOffset;     // no other kernel shares this scratch
        st.ready = true;
    }
    *out = &st;
    return NVFP4_OK;
}

}  // namespace
}  // namespace nvfp4

extern "C" int nvfp4_linear_decode_noalloc(const void* A, int M, const uint8_t* packed, const uint8_t* scale,
                                           float global_scale, int N, int K, const void* residual, void* C,
                                           nvfp4_stream_t stream) {
    using namespace nvfp4;
    if (!A || !packed || !scale || !C) return NVFP4_E_NULL;
    if (M < 0 || N <= 0 || K <= 0 || (K & 15) != 0) return NVFP4_E_SHAPE;
    if (!(global_scale > 0.0f) || !(global_scale <= 3.0e38f)) return NVFP4_E_SCALE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (mis(A) || mis(C) || (residual && mis(residual)) || mis(packed) || mis(scale)) return NVFP4_E_ALIGN;
    const char* a0 = static_cast<const char*>(A);
    const char* c0 = static_cast<const char*>(C);
    if (M > 0 && a0 < c0 + (size_t)M * N * 2 && c0 < a0 + (size_t)M * K * 2) return NVFP4_E_ALIAS;
    if (M == 0) return NVFP4_OK;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return NVFP4_E_DEVICE;
    NoAllocState* st = nullptr;
    if (int e = noalloc_setup(device, &st)) return e;
    LinearArgs a{A, packed, scale, 1.0f / global_scale, residual, C, M, N, K};
    if (M > 16 || !decode_mma_supported(a) || !decode_mma_fits(a, st->dev)) return NVFP4_E_LIMIT;
    int launches = 0;
    cudaError_t e = launch_decode_mma(a, st->dev, st->scratch, &launches, stream);
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

// The status word of the fixed scratch on the current device: a bounded wait of the allocation-free
// GEMV that ran out leaves its code there (first failure wins) and part of C unwritten.  Reads
// four bytes with a blocking copy after synchronising the device; allocates nothing.
extern "C" int nvfp4_noalloc_status(unsigned int* status, int reset) {
    using namespace nvfp4;
    if (!status) return NVFP4_E_NULL;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return NVFP4_E_DEVICE;
    NoAllocState* st = nullptr;
    if (int e = noalloc_setup(device, &st)) return e;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(status, st->scratch, sizeof(unsigned int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && reset && *status != 0u) e = cudaMemset(st->scratch, 0, sizeof(unsigned int));
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}
