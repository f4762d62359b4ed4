// Dequant-free GEMV for up to 9 tokens on the NVFP4 tensor-core path (10 to 16 tokens: decode_fp4_stream.cu): the packed weights go from HBM
// to the tensor core untouched.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W = e2m1(code) * ue4m3(scale) / global_scale
//
// tcgen05.mma kind::mxf4nvf4 (block_scale, one unsigned E4M3 scale per 16 elements of K) takes both
// operands as packed E2M1 with block scales -- the weights' own HBM layout.  So, unlike the
// mma.sync GEMV (decode_mma.cu), whose 16 consumer warps spend their time converting codes and
// multiplying scales (and top out at the HBM rate with nothing to spare), this kernel has no
// per-weight instruction at all:
//   * warp 0 streams half-units (128 weight rows x 256 k: 16 KB of codes + 2 KB of scales) into a
//     shared-memory ring with plain tiled TMA (128-byte swizzle for the codes: the K-major operand
//     layout of the tensor core; no multicast); the half-units, row-tile-major, are split evenly
//     over the CTAs (stream-K);
//   * warps 4-7 move the 2 KB of block scales of each half-unit from shared into tensor memory
//     (tcgen05.st: row r of the MMA wants the four scales of a 64-k MMA in lane r % 32, column r / 32,
//     in every lane quarter), together with the activations' scales of the same k range; that is
//     the only touch the weights get.  (tcgen05.cp from re-ordered atoms does the same, but its four
//     copies per half-unit queue up in front of the MMAs in the tensor pipe: 5.7 TB/s measured);
//   * one thread of warp 1 issues four tcgen05.mma (128 rows x NCp columns x 64 k) per half-unit,
//     accumulating FP32 in tensor memory; tcgen05.commit recycles the ring stage;
//   * the activations are the B operand: a pre-pass (act_fp4.cu) expands every BF16 token into six
//     (five for 3, 6 and 9 tokens) NVFP4 term rows whose sum reproduces it to 1e-5 (8e-5) of each block's largest element; the CTA's k
//     range of the codes is loaded once by warp 2 and stays resident in shared memory, next to their
//     block scales (copied in by warps 8-11 before their first accumulator arrives).  For one or two
//     tokens without SwiGLU or RMSNorm in front, where a CTA's k range is short (up to 8 chunks), there
//     is no pre-pass at all: warps 4-11 expand the CTA's k range of the activations themselves,
//     straight into the operand layout in shared memory (CTAs repeat each other's work, but a
//     kernel boundary is gone);
//   * warps 8-11 read the accumulator (thread = weight row), add the term columns of each token,
//     undo the token scale, apply 1/global_scale and the residual in FP32 and round once.  A row
//     tile split over several CTAs is finished by the CTA holding its first half-unit: the others
//     publish FP32 partials as {value, launch tag} pairs (8-byte single transactions, the tag
//     from a counter in the scratch), the owner adds them in CTA order (deterministic).
// Every wait is bounded and reports through the status word; tensor memory is always freed.
//
// Arithmetic: the weight side is exact (the tensor core multiplies e2m1 x ue4m3 exactly and
// accumulates in FP32); the activation side carries the pre-pass's remainder.  Against the
// reference's GEMV (src/engine/dense_gemm_fp4_sm110.cu:96-141): same products up to that remainder,
// FP32 accumulation in another order, one rounding.  A scale byte 0x7F / 0xFF is NaN to the tensor
// core (as in FP8 E4M3, whose finite maximum is 0x7E = 448); the reference's table-free decoder reads
// it as 480.  No finite FP8 scale, hence no checkpoint, contains it.
#include <cuda.h>
#include <cuda_bf16.h>

#include "fp4_quant.cuh"
#include "fp4_mma.cuh"
#include "fp4_store.cuh"
#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "ptx.cuh"
#include "umma.cuh"

namespace nvfp4 {
namespace {

using namespace umma;
using namespace fp4mma;

constexpr int kMaxStages = 10;
constexpr int kThreads = 12 * 32;
constexpr int kEpiThreads = 4 * 32;
// Not all of an SM's 228 KB: the activation pre-pass of the NEXT call (launched with programmatic stream
// serialization while this kernel runs) must find room for its CTAs beside this kernel's, or the two
// calls serialize (5 us on a 10 us call, measured, when 544 bytes were left).
constexpr int kSmemBudget = 225 * 1024;
constexpr int kAccStride = 64;                     // tensor-memory columns per accumulator (NCp <= 48)
constexpr int kSfCol = 2 * kAccStride;             // per half-unit of the ring 32 columns: 16 of the weights' scales, 16 of the activations'
constexpr int kMaxRingHalfUnits = (512 - kSfCol) / 32;   // 12
constexpr int kTokens = 9;                         // most tokens of this kernel: 9 x 5 = 45 of its 48 MMA columns
constexpr int kMaxGrid = 160;                      // CTAs whose pair slots fit the kernel's share of the scratch
constexpr int kPairTokens = kTokens;               // token rows of a CTA's pair slot (9 KB per CTA)
static_assert((size_t)kMaxGrid * kPairTokens * kRT * 8 <= fp4::kPairBytes, "pair slots");

struct Fp4Params {
    Fp4Out out;                     // residual, C, 1 / global_scale, M, N and the output options
    Fp4Out out2;                    // ... of the second weight of a dual call (row tiles from tiles0 on)
    int tiles0;                     // row tiles of the first weight (all of them unless the call is dual)
    const float* unscale;           // per token: 1 / c of the pre-pass
    const __nv_bfloat16* A;         // the kernel expands the activations itself: [M, K] BF16 rows a_stride apart,
    long long a_stride;             // ... columns from k_valid on count as zero and are never read
    int k_valid;
    const unsigned char* sfb;       // the pre-pass's block scales: [K/256][column groups of 32][32 lanes][16 bytes]
    unsigned char* scratch;         // status word at 0, launch counter at 64
    unsigned char* pairs;           // [CTA][kPairTokens][128 rows] x {FP32 value, tag}
    int M, N, K;
    int NCp, groups;                // MMA columns (tokens x terms padded to 16), groups of 32 of them
    int units, kchunks;
    int stages, hps;                // ring depth, half-units per stage (1 or 2)
    int slots, act_all;             // resident activation chunks; 1 = slot index is the k-chunk
};


constexpr int kOwnTokens = 2;       // most tokens the kernel expands itself
constexpr int kOwnThreads = 8 * 32; // warps 4-11
constexpr int kOwnMaxChunks = 8;    // ... and most resident 256-k chunks x tokens it does so for

template <int TERMS, bool OWN, bool DUAL = false>
__global__ void __launch_bounds__(kThreads, 1)
decode_fp4_kernel(const __grid_constant__ CUtensorMap tm_packed, const __grid_constant__ CUtensorMap tm_scale,
                  const __grid_constant__ CUtensorMap tm_packed2, const __grid_constant__ CUtensorMap tm_scale2,
                  const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ Fp4Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int stages = p.stages, hps = p.hps;
    const int b_bytes = p.NCp * 128;                                        // one resident activation chunk (NCp rows x 256 k)
    unsigned char* s_w = smem;                                              // stages x hps x 16 KB, 1024-aligned
    unsigned char* s_b = s_w + stages * hps * kPackedBytes;                 // slots x NCp x 128 B, 1024-aligned (NCp % 8 == 0)
    unsigned char* s_raw = s_b + p.slots * b_bytes;                         // stages x hps x 2 KB: scales as they lie in HBM
    unsigned char* s_sfb = s_raw + stages * hps * kScaleBytes;              // slots x groups x 512 B: the activations' scales
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_sfb + p.slots * p.groups * 512);
    uint64_t* empty_bar = full_bar + kMaxStages;
    uint64_t* sfa_bar = empty_bar + kMaxStages;      // scales of a stage are in tensor memory
    uint64_t* b_bar = sfa_bar + kMaxStages;          // [0] resident activation codes loaded, [1] their scales in shared memory
    uint64_t* tfull = b_bar + 2;                     // [2] accumulator complete
    uint64_t* tempty = tfull + 2;                    // [2] accumulator read
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    volatile unsigned int* s_epoch = reinterpret_cast<volatile unsigned int*>(s_tmem + 2);
    unsigned int* s_amax = s_tmem + 3;                                      // [2] largest magnitude of a token (BF16 bits)
    float* s_unscale = reinterpret_cast<float*>(s_tmem + 5);                // [2] 1 / c of a token

    unsigned int* status = reinterpret_cast<unsigned int*>(p.scratch);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int u_begin = (int)((long long)cta * p.units / G);      // half-units [u_begin, u_end) of this CTA
    const int u_end = (int)((long long)(cta + 1) * p.units / G);
    const int kc_begin = u_begin % p.kchunks;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
            ptx::mbar_init(&sfa_bar[s], 4);
        }
        ptx::mbar_init(&b_bar[0], 1);
        ptx::mbar_init(&b_bar[1], OWN ? 1 : 4);
        s_amax[0] = s_amax[1] = 0u;
        for (int i = 0; i < 2; ++i) { ptx::mbar_init(&tfull[i], 1); ptx::mbar_init(&tempty[i], 4); }
        *s_abort = 0;
        *s_epoch = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) tmem_alloc_512(s_tmem);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    ptx::griddep_launch_dependents();

    if (OWN && warp >= 4) {
        // ------------------------------------------------------------------ the activations, expanded here (see act_fp4.cu for the scheme)
        using namespace fp4q;
        const int tq = tid - 4 * 32;
        ptx::griddep_wait();                                  // A is the output of the kernel before this one
        const int chunks = p.k_valid / 8;
#pragma unroll
        for (int m = 0; m < kOwnTokens; ++m) {
            if (m >= p.M) continue;
            const uint4* src = reinterpret_cast<const uint4*>(p.A + (size_t)m * p.a_stride);
            unsigned int amax = 0;
            for (int i0 = tq; i0 < chunks; i0 += kOwnThreads * 4) {
                uint4 x[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * kOwnThreads;
                    x[j] = i < chunks ? __ldcg(src + i) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t v[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) amax = max(amax, max(v[q] & 0x7FFFu, (v[q] >> 16) & 0x7FFFu));
                }
            }
            amax = __reduce_max_sync(0xffffffffu, amax);
            if (lane == 0 && amax) atomicMax(&s_amax[m], amax);
        }
        ptx::named_barrier_sync(2, kOwnThreads);
        float c[kOwnTokens];
#pragma unroll
        for (int m = 0; m < kOwnTokens; ++m) {
            const int se = token_scale_exponent(s_amax[m]);
            c[m] = __uint_as_float((uint32_t)se << 23);
            if (tq == m) s_unscale[m] = token_unscale(s_amax[m], se);
        }
        // One task = a quarter (4 elements) of a 16-element block of one token in one resident chunk; a quad of
        // lanes holds the block.  64 tasks per token and chunk, so whole warps are in or out of range together.
        const int total = p.M * p.slots * 64;
        const int kc0 = p.act_all ? 0 : kc_begin;
        for (int id0 = tq; id0 < total; id0 += kOwnThreads * 4) {
            uint2 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int id = id0 + u * kOwnThreads;
                x[u] = make_uint2(0u, 0u);
                if (id < total) {
                    const int part = id & 3, bl = (id >> 2) & 15, rest = id >> 6;
                    const int m = rest / p.slots, j = rest - m * p.slots;
                    int kcj = kc0 + j;
                    if (kcj >= p.kchunks) kcj -= p.kchunks;
                    const int k = kcj * kKC + bl * 16 + part * 4;
                    if (k < p.k_valid) x[u] = __ldcg(reinterpret_cast<const uint2*>(p.A + (size_t)m * p.a_stride + k));
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int id = id0 + u * kOwnThreads;
                if (id >= total) continue;                        // uniform across the warp
                const int part = id & 3, bl = (id >> 2) & 15, rest = id >> 6;
                const int m = rest / p.slots, j = rest - m * p.slots;
                const float cm = m == 0 ? c[0] : c[1];
                float r[4] = {__uint_as_float(x[u].x << 16) * cm, __uint_as_float(x[u].x & 0xFFFF0000u) * cm,
                              __uint_as_float(x[u].y << 16) * cm, __uint_as_float(x[u].y & 0xFFFF0000u) * cm};
                float bmax = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
                bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
                bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
                const int p0 = first_term_exponent(bmax);
                // Operand layout (K-major, 128-byte swizzle, as TMA would have written it): row = MMA column, a row
                // holds the chunk's 256 codes in eight 16-byte pieces, piece i of row r at position i ^ (r % 8).
                unsigned char* row0 = s_b + j * b_bytes;
                unsigned char* sf0 = s_sfb + j * p.groups * 512 + (bl >> 2) * 4 + (bl & 3);
#pragma unroll
                for (int t = 0; t < TERMS; ++t) {
                    const int pw = term_exponent(p0, t);
                    const uint32_t w = take_term(r, pw);
                    const int col = m * TERMS + t;
                    *reinterpret_cast<uint16_t*>(row0 + col * 128 + (((bl >> 1) ^ (col & 7)) << 4) + (bl & 1) * 8 + part * 2) = (uint16_t)w;
                    if (part == 0) sf0[(col & 31) * 16] = (uint8_t)ue4m3_pow2(pw);
                }
            }
        }
        ptx::fence_proxy_async_smem();                        // the tensor core reads the codes through the asynchronous proxy
        ptx::named_barrier_sync(2, kOwnThreads);
        if (tq == 0) {
            ptx::mbar_arrive(&b_bar[0]);
            ptx::mbar_arrive(&b_bar[1]);
        }
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ weight stream
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
            if (DUAL) {
                ptx::prefetch_tensormap(&tm_packed2);
                ptx::prefetch_tensormap(&tm_scale2);
            }
            const uint64_t pol = ptx::policy_evict_first();
            int stage = 0;
            uint32_t ph = 0;
            int hu = u_begin, tile = u_begin / p.kchunks, kc = kc_begin;
            while (hu < u_end) {
                const int tile_end = hu - kc + p.kchunks;
                const int seg_end = tile_end < u_end ? tile_end : u_end;
                const bool second = DUAL && tile >= p.tiles0;     // a dual call: the second weight's row tiles follow the first's
                const int row0 = (second ? tile - p.tiles0 : tile) * kRT;
                const CUtensorMap* mp = second ? &tm_packed2 : &tm_packed;
                const CUtensorMap* ms = second ? &tm_scale2 : &tm_scale;
                while (hu < seg_end) {
                    const int cnt = (seg_end - hu) >= hps ? hps : 1;
                    ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, 0xA00u + (unsigned)stage);
                    ptx::mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)(kPackedBytes + kScaleBytes) * cnt);
                    for (int h = 0; h < cnt; ++h) {
                        const int k0 = (kc + h) * kKC;
                        ptx::tma_load_2d(s_w + (stage * hps + h) * kPackedBytes, mp, &full_bar[stage], k0 >> 1, row0, pol);
                        ptx::tma_load_2d(s_raw + (stage * hps + h) * kScaleBytes, ms, &full_bar[stage], k0 >> 4, row0, pol);
                    }
                    hu += cnt;
                    kc += cnt;
                    if (++stage == stages) { stage = 0; ph ^= 1u; }
                }
                if (kc >= p.kchunks) { kc = 0; ++tile; }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ resident activations (the pre-pass's output)
        if (lane == 0 && !OWN) {
            ptx::prefetch_tensormap(&tm_act);
            ptx::griddep_wait();
            const uint64_t pol = ptx::policy_evict_last();
            ptx::mbar_arrive_expect_tx(&b_bar[0], (uint32_t)(p.slots * b_bytes));
            const int kc0 = p.act_all ? 0 : kc_begin;
            for (int j = 0; j < p.slots; ++j) {
                int kc = kc0 + j;
                if (kc >= p.kchunks) kc -= p.kchunks;
                ptx::tma_load_2d(s_b + j * b_bytes, &tm_act, &b_bar[0], kc * (kKC / 2), 0, pol);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = fp4_idesc(p.NCp);
            ptx::mbar_wait(&b_bar[0], 0u, s_abort, status, 0xA10u);
            int stage = 0, acc = 0;
            uint32_t ph = 0, pt = 0;
            int hu = u_begin, kc = kc_begin;
            while (hu < u_end) {
                const int tile_end = hu - kc + p.kchunks;
                const int seg_end = tile_end < u_end ? tile_end : u_end;
                ptx::mbar_wait(&tempty[acc], ((pt >> acc) & 1u) ^ 1u, s_abort, status, 0xA20u + (unsigned)acc);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kAccStride);
                bool first = true;
                while (hu < seg_end) {
                    const int cnt = (seg_end - hu) >= hps ? hps : 1;
                    ptx::mbar_wait(&sfa_bar[stage], ph, s_abort, status, 0xA30u + (unsigned)stage);
                    tc_fence_after();
                    for (int h = 0; h < cnt; ++h) {
                        const int slot = p.act_all ? kc + h : (hu - u_begin) + h;
                        const uint32_t sfa_t = tmem_base + kSfCol + 32 * (uint32_t)(stage * hps + h), sfb_t = sfa_t + 16;
                        const uint32_t a_addr = ptx::smem_u32(s_w + (stage * hps + h) * kPackedBytes);
                        const uint32_t b_addr = ptx::smem_u32(s_b + slot * b_bytes);
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            umma_fp4(d_tmem, umma_desc_sw128(a_addr + 32 * s), umma_desc_sw128(b_addr + 32 * s), idesc,
                                     sfa_t + 4 * s, sfb_t + 4 * s, first ? 0u : 1u);
                            first = false;
                        }
                    }
                    umma_commit(&empty_bar[stage]);        // the stage's codes and its scales in tensor memory are free once these MMAs have read them
                    hu += cnt;
                    kc += cnt;
                    if (++stage == stages) { stage = 0; ph ^= 1u; }
                }
                umma_commit(&tfull[acc]);
                pt ^= 1u << acc;
                acc ^= 1;
                if (kc >= p.kchunks) kc = 0;
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------------ scales into tensor memory
        // Warp q (= warp id % 4) writes lane quarter q; the four warps write the same data, which is the
        // replication the tensor core wants.  Lane L holds, for MMA s of the half-unit, the scale words of weight
        // rows L, L + 32, L + 64, L + 96 in columns 4 s .. 4 s + 3, and the words of activation columns L and
        // 32 + L in columns 16 + 4 s and 17 + 4 s (an MMA's scale base sits on a multiple of four columns).
        const int q = warp - 4;
        ptx::mbar_wait(&b_bar[1], 0u, s_abort, status, 0xA11u);      // the activations' scales are in shared memory
        int stage = 0;
        uint32_t ph = 0;
        int hu = u_begin, kc = kc_begin;
        while (hu < u_end) {
            const int tile_end = hu - kc + p.kchunks;
            const int seg_end = tile_end < u_end ? tile_end : u_end;
            while (hu < seg_end) {
                const int cnt = (seg_end - hu) >= hps ? hps : 1;
                ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0xA40u + (unsigned)stage);
                for (int h = 0; h < cnt; ++h) {
                    const int slot = p.act_all ? kc + h : (hu - u_begin) + h;
                    const unsigned char* raw = s_raw + (stage * hps + h) * kScaleBytes + lane * 16;
                    uint32_t ra[16], rb[16];
#pragma unroll
                    for (int r1 = 0; r1 < 4; ++r1) {
                        const uint4 x = *reinterpret_cast<const uint4*>(raw + r1 * 512);
                        ra[r1] = x.x & 0x7F7F7F7Fu;            // bit 7 carries nothing (src/engine/dense_gemm_fp4_sm110.cu:30-41)
                        ra[4 + r1] = x.y & 0x7F7F7F7Fu;
                        ra[8 + r1] = x.z & 0x7F7F7F7Fu;
                        ra[12 + r1] = x.w & 0x7F7F7F7Fu;
                    }
                    const uint4 b0 = *reinterpret_cast<const uint4*>(s_sfb + (slot * p.groups) * 512 + lane * 16);
                    uint4 b1 = make_uint4(0u, 0u, 0u, 0u);
                    if (p.groups > 1) b1 = *reinterpret_cast<const uint4*>(s_sfb + (slot * p.groups + 1) * 512 + lane * 16);
                    rb[0] = b0.x; rb[1] = b1.x; rb[2] = 0u; rb[3] = 0u;
                    rb[4] = b0.y; rb[5] = b1.y; rb[6] = 0u; rb[7] = 0u;
                    rb[8] = b0.z; rb[9] = b1.z; rb[10] = 0u; rb[11] = 0u;
                    rb[12] = b0.w; rb[13] = b1.w; rb[14] = 0u; rb[15] = 0u;
                    const uint32_t t = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(kSfCol + 32 * (stage * hps + h));
                    tmem_st16(t, ra);
                    tmem_st16(t + 16, rb);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sfa_bar[stage]);
                hu += cnt;
                kc += cnt;
                if (++stage == stages) { stage = 0; ph ^= 1u; }
            }
            if (kc >= p.kchunks) kc = 0;
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ epilogue: thread = weight row
        const int ew = warp - 8;                              // tensor-memory lanes 32 ew .. +31 (= warp id % 4)
        const int te = ew * 32 + lane;
        ptx::griddep_wait();                                  // C, the residual and the scratch belong to earlier kernels until now
        // this launch's tag for the split-tile pairs: one atomic per CTA on one address, about a microsecond
        // under contention, so it is left in flight while the scales are copied
        unsigned int epoch_taken = 0;
        if (te == 0) epoch_taken = ptx::take_launch_epoch(p.scratch);
        unsigned char* pairs = p.pairs;
        if (!OWN) {
            // The activations' block scales of the CTA's k range into shared memory (512 bytes per resident chunk
            // and column group, as the pre-pass left them); the warps of the scale path wait for this.
            const int kc0 = p.act_all ? 0 : kc_begin;
            const int words = p.slots * p.groups * 32;              // 16-byte words
            for (int i = te; i < words; i += kEpiThreads) {
                const int j = i / (p.groups * 32), rest = i - j * (p.groups * 32);
                int kcj = kc0 + j;
                if (kcj >= p.kchunks) kcj -= p.kchunks;
                reinterpret_cast<uint4*>(s_sfb)[i] = __ldcg(reinterpret_cast<const uint4*>(p.sfb + (size_t)kcj * p.groups * 512) + rest);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&b_bar[1]);
        }
        if (te == 0) *s_epoch = epoch_taken;
        ptx::named_barrier_sync(1, kEpiThreads);
        const unsigned int epoch = *s_epoch;
        int acc = 0;
        uint32_t pt = 0;
        int hu = u_begin, tile = u_begin / p.kchunks, kc = kc_begin;
        while (hu < u_end) {
            const int kc_first = kc;
            const int tile_end = hu - kc + p.kchunks;
            const int seg_end = tile_end < u_end ? tile_end : u_end;
            const bool owner = kc_first == 0;
            const bool complete = owner && seg_end == tile_end;
            int last = cta;                                   // contributors are CTAs cta+1 .. last
            if (owner && !complete)
                while (last + 1 < G && (long long)(last + 1) * p.units / G < tile_end) ++last;
            ptx::mbar_wait(&tfull[acc], (pt >> acc) & 1u, s_abort, status, 0xA50u + (unsigned)acc);
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)(acc * kAccStride);
            float v[kTokens];
#pragma unroll
            for (int m = 0; m < kTokens; ++m) v[m] = 0.0f;
#pragma unroll
            for (int c0 = 0; c0 < 48; c0 += 16) {
                if (c0 < p.NCp) {
                    uint32_t r[16];
                    tmem_ld16(t_addr + c0, r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int c = c0 + i;                 // column c = token * TERMS + term (compile-time after unrolling)
                        if (c / TERMS < kTokens) v[c / TERMS] += __uint_as_float(r[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tempty[acc]);
            pt ^= 1u << acc;
            acc ^= 1;
            hu = seg_end;
            kc = kc_first + (seg_end - (tile_end - p.kchunks + kc_first));

#pragma unroll
            for (int m = 0; m < kTokens; ++m)
                if (m < p.M) v[m] *= OWN ? s_unscale[m < kOwnTokens ? m : 0] : p.unscale[m];
            if (!owner) {
                unsigned char* slot = pairs + (size_t)cta * (kPairTokens * kRT) * 8;
#pragma unroll
                for (int m = 0; m < kTokens; ++m)
                    if (m < p.M) ptx::st_volatile_v2(slot + (m * kRT + te) * 8, __float_as_uint(v[m]), epoch);
            } else {
                fp4_gather_pairs(v, pairs, (size_t)(kPairTokens * kRT) * 8, cta + 1, last, p.M, te, epoch, s_abort, status, 0xA60u);
                if (!DUAL || tile < p.tiles0) fp4_store_rows(v, p.out, tile, te);
                else fp4_store_rows(v, p.out2, tile - p.tiles0, te);
            }
            if (kc >= p.kchunks) { kc = 0; ++tile; }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_512(tmem_base);
    }
}

struct Fp4Plan {
    Fp4Params p;
    int grid, smem;
};

constexpr int kFixedSmem = 1024 + (3 * kMaxStages + 6) * 8 + 64;

bool plan_fp4(const LinearArgs& a, const nvfp4_device_info& dev, Fp4Plan* out) {
    Fp4Params& p = out->p;
    p = Fp4Params{};
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.NCp = (a.M * fp4::terms_for(a.M) + 15) / 16 * 16;
    p.groups = (p.NCp + 31) / 32;
    p.kchunks = a.K / kKC;
    p.tiles0 = (a.N + kRT - 1) / kRT;
    const long long units = (long long)p.tiles0 * (a.packed2 ? 2 : 1) * p.kchunks;
    if (units > 0x7fffffffLL || units < 1) return false;
    p.units = (int)units;
    int grid = dev.sm_count < kMaxGrid ? dev.sm_count : kMaxGrid;
    if (grid > p.units) grid = p.units;
    const int max_span = (p.units + grid - 1) / grid;
    p.act_all = p.kchunks <= max_span ? 1 : 0;
    p.slots = p.act_all ? p.kchunks : max_span;
    const long long resident = (long long)p.slots * (p.NCp * 128 + p.groups * 512);
    const long long avail = kSmemBudget - kFixedSmem - resident;
    const int unit = kPackedBytes + kScaleBytes;                    // codes + scales
    // Two half-units per stage when four such stages fit (one issuing thread keeps HBM busier with larger stages)
    p.hps = avail / (2 * unit) >= 4 ? 2 : 1;
    long long stages = avail / ((long long)p.hps * unit);
    if (stages < 3) return false;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages * p.hps > kMaxRingHalfUnits) stages = kMaxRingHalfUnits / p.hps;     // 32 tensor-memory columns of scales per half-unit of the ring
    p.stages = (int)stages;
    out->grid = grid;
    out->smem = kFixedSmem + (int)stages * p.hps * unit + (int)resident;
    return true;
}

}  // namespace

bool decode_fp4_supported(const LinearArgs& a, const nvfp4_device_info& dev) {
    if (a.M < 1 || a.M > kTokens || (a.K % kKC) != 0 || a.N < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u)) return false;
    if (a.px || !act_to_fp4_supported(a)) return false;
    if (a.packed2 && (!a.scale2 || !a.C2 || a.residual || a.swiglu_out || (reinterpret_cast<uintptr_t>(a.packed2) & 15u) ||
                      (reinterpret_cast<uintptr_t>(a.scale2) & 15u)))
        return false;
    if (a.swiglu_out && (a.residual || a.out_f32 || (a.N & 15))) return false;
    Fp4Plan pl;
    return plan_fp4(a, dev, &pl);
}

size_t decode_fp4_scratch_bytes(int K) { return fp4::act_scratch_bytes(K); }

cudaError_t configure_decode_fp4() {
    cudaError_t e = configure_large_smem(decode_fp4_kernel<5, false>, kSmemBudget);
    if (e == cudaSuccess) e = configure_large_smem(decode_fp4_kernel<6, false>, kSmemBudget);
    if (e == cudaSuccess) e = configure_large_smem(decode_fp4_kernel<6, true>, kSmemBudget);
    if (e == cudaSuccess) e = configure_large_smem(decode_fp4_kernel<5, false, true>, kSmemBudget);
    if (e == cudaSuccess) e = configure_large_smem(decode_fp4_kernel<6, false, true>, kSmemBudget);
    if (e == cudaSuccess) e = configure_large_smem(decode_fp4_kernel<6, true, true>, kSmemBudget);
    return e;
}

cudaError_t launch_decode_fp4(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t pairs_offset, void* act,
                              int* launches, cudaStream_t s) {
    Fp4Plan pl;
    if (!plan_fp4(a, dev, &pl)) return cudaErrorInvalidValue;
    Fp4Params& p = pl.p;
    unsigned char* codes = static_cast<unsigned char*>(act);
    unsigned char* sfb = codes + fp4::act_sfb_offset(a.K);
    float* unscale = reinterpret_cast<float*>(codes + fp4::act_unscale_offset(a.K));
    CUtensorMap tmp, tms, tma, tmp2, tms2;
    if (!make_map_cached(dev.maps, &tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, kRT,
                         CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, kRT,
                         CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_map_cached(dev.maps, &tma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, (uint64_t)a.K / 2, (uint64_t)p.NCp, 128,
                         (uint32_t)p.NCp, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    tmp2 = tmp;
    tms2 = tms;
    if (a.packed2 &&
        (!make_map_cached(dev.maps, &tmp2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.packed2, (uint64_t)a.K / 2, (uint64_t)a.N, 128, kRT,
                          CU_TENSOR_MAP_SWIZZLE_128B) ||
         !make_map_cached(dev.maps, &tms2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.scale2, (uint64_t)a.K / 16, (uint64_t)a.N, 16, kRT,
                          CU_TENSOR_MAP_SWIZZLE_NONE)))
        return cudaErrorInvalidValue;
    const int terms = fp4::terms_for(a.M);
    // One or two plain tokens on a short k range per CTA: the kernel expands them itself and no pre-pass runs.
    // (Measured: 0.7 us ahead of the pre-pass at 7 and 8 resident chunks, 1.8 us behind at 19 and 20.)
    const bool own = dev.fp4_own_quant && a.M <= kOwnTokens && terms == 6 && !a.swiglu_up && !a.norm_w && a.M * p.slots <= kOwnMaxChunks;
    cudaError_t e = cudaSuccess;
    if (!own) e = launch_act_to_fp4(a, terms, p.groups, codes, sfb, unscale, s);
    if (e != cudaSuccess) return e;
    p.A = static_cast<const __nv_bfloat16*>(a.A);
    p.a_stride = a.a_stride ? a.a_stride : a.K;
    p.k_valid = a.k_valid ? a.k_valid : a.K;
    p.out.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.out.C = static_cast<__nv_bfloat16*>(a.C);
    p.out.M = a.M;
    p.out.N = a.N;
    p.out.swiglu_out = a.swiglu_out ? 1 : 0;
    p.unscale = unscale;
    p.sfb = sfb;
    p.scratch = static_cast<unsigned char*>(scratch);
    p.pairs = p.scratch + pairs_offset;
    p.out.inv_gs = a.inv_gs;
    p.out.out_f32 = a.out_f32 ? 1 : 0;
    p.out2 = p.out;
    p.out2.C = static_cast<__nv_bfloat16*>(a.C2);
    p.out2.inv_gs = a.inv_gs2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (a.packed2)
        e = own ? cudaLaunchKernelEx(&cfg, decode_fp4_kernel<6, true, true>, tmp, tms, tmp2, tms2, tma, p)
                : (terms == 6 ? cudaLaunchKernelEx(&cfg, decode_fp4_kernel<6, false, true>, tmp, tms, tmp2, tms2, tma, p)
                              : cudaLaunchKernelEx(&cfg, decode_fp4_kernel<5, false, true>, tmp, tms, tmp2, tms2, tma, p));
    else
        e = own ? cudaLaunchKernelEx(&cfg, decode_fp4_kernel<6, true>, tmp, tms, tmp2, tms2, tma, p)
                : (terms == 6 ? cudaLaunchKernelEx(&cfg, decode_fp4_kernel<6, false>, tmp, tms, tmp2, tms2, tma, p)
                              : cudaLaunchKernelEx(&cfg, decode_fp4_kernel<5, false>, tmp, tms, tmp2, tms2, tma, p));
    if (launches) *launches = own ? 1 : 2;
    return e;
}

}  // namespace nvfp4
