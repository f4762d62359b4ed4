// Dequant-free GEMV for up to 16 tokens on the NVFP4 tensor-core path, activations streamed with the
// weights: the form of decode_fp4.cu for 10 to 16 tokens (up to 96 MMA columns), and for any shape whose
// activations would leave that kernel's ring too short.  The packed weights go from HBM to the tensor
// core untouched.
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
//   * the activations are the B operand: a pre-pass (act_fp4.cu) expands every BF16 token into five
//     or six NVFP4 term rows whose sum reproduces it to 8e-5 / 1e-5 of each block's largest element.
//     Warp 2 streams the 256-k slice of those rows (tokens x terms x 128 bytes, from L2: every CTA
//     reads the same 50..800 KB) and of their block scales into the same ring stage as the weights
//     it multiplies; it alone waits for the pre-pass, so the weights are on their way while the
//     pre-pass still runs, and all of shared memory is ring.  (Up to 48 MMA columns the other kernel,
//     which loads the CTA's k range of them once, is 1..2 us per call faster.);
//   * warps 4-7 move the 2 KB of block scales of each half-unit from shared into tensor memory
//     (tcgen05.st: row r of the MMA wants the four scales of a 64-k MMA in lane r % 32, column r / 32,
//     in every lane quarter), together with the activations' scales of the same k range; that is
//     the only touch the weights get.  (tcgen05.cp from re-ordered atoms does the same, but its four
//     copies per half-unit queue up in front of the MMAs in the tensor pipe: 5.7 TB/s measured);
//   * one thread of warp 1 issues four tcgen05.mma (128 rows x NCp columns x 64 k) per half-unit,
//     accumulating FP32 in tensor memory; tcgen05.commit recycles the ring stage;
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

constexpr int kMaxStages = 12;
constexpr int kThreads = 12 * 32;
constexpr int kEpiThreads = 4 * 32;
// Not all of an SM's 228 KB: the activation pre-pass of the NEXT call (launched with programmatic stream
// serialization while this kernel runs) must find room for its CTAs beside this kernel's, or the two
// calls serialize (5 us on a 10 us call, measured, when 544 bytes were left).
constexpr int kSmemBudget = 225 * 1024;
// Tensor memory: two accumulators of acc_stride columns (64, or 128 beyond 64 MMA columns), then per half-unit
// of the ring 32 columns: 16 of the weights' scales, 16 of the activations' (4 per MMA: up to 128 MMA columns).
constexpr int kMaxCols = fp4::kMaxCols;            // MMA columns (tokens x terms, padded to 16)
constexpr int kMaxGrid = 160;                      // CTAs whose pair slots fit the kernel's 2.5 MB of scratch
constexpr int kPairTokens = fp4::kMaxTokens;       // token rows of a CTA's pair slot (16 KB per CTA)
static_assert((size_t)kMaxGrid * kPairTokens * kRT * 8 <= fp4::kPairBytes, "pair slots");

struct Fp4Params {
    Fp4Out out;                     // residual, C, 1 / global_scale, M, N and the output options
    const float* unscale;           // per token: 1 / c of the pre-pass
    unsigned char* scratch;         // status word at 0, launch counter at 64
    unsigned char* pairs;           // [CTA][kPairTokens][128 rows] x {FP32 value, tag}
    int M, N, K;
    int NCp, groups;                // MMA columns (tokens x terms padded to 16), groups of 32 of them
    int acc_stride;                 // tensor-memory columns per accumulator
    int units, kchunks;
    int stages, hps;                // ring depth, half-units per stage (1 or 2)
};


// At most 136 registers: with more, the next call's pre-pass (launched while this kernel runs) finds no room in
// the register file beside a CTA of this kernel, and the two calls serialize.
template <int TERMS>
__global__ void __maxnreg__(136)
decode_fp4_stream_kernel(const __grid_constant__ CUtensorMap tm_packed, const __grid_constant__ CUtensorMap tm_scale,
                  const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_sfb,
                  const __grid_constant__ Fp4Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int stages = p.stages, hps = p.hps;
    const int b_bytes = p.NCp * 128;                                        // the activations' codes of one half-unit (NCp rows x 256 k)
    const int sfb_bytes = p.groups * 512;                                   // ... and their block scales
    unsigned char* s_w = smem;                                              // stages x hps x 16 KB, 1024-aligned
    const int nb = stages * hps;                                            // activation slices held in shared memory
    unsigned char* s_b = s_w + stages * hps * kPackedBytes;                 // nb x NCp x 128 B, 1024-aligned (NCp % 8 == 0)
    unsigned char* s_raw = s_b + nb * b_bytes;                              // stages x hps x 2 KB: scales as they lie in HBM
    unsigned char* s_sfb = s_raw + stages * hps * kScaleBytes;              // nb x groups x 512 B: the activations' scales
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_sfb + nb * sfb_bytes);     // weights of a stage have landed
    uint64_t* fullb_bar = full_bar + kMaxStages;     // activations of a stage have landed
    uint64_t* empty_bar = fullb_bar + kMaxStages;
    uint64_t* sfa_bar = empty_bar + kMaxStages;      // scales of a stage are in tensor memory
    uint64_t* tfull = sfa_bar + kMaxStages;          // [2] accumulator complete
    uint64_t* tempty = tfull + 2;                    // [2] accumulator read
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    volatile unsigned int* s_epoch = reinterpret_cast<volatile unsigned int*>(s_tmem + 2);

    unsigned int* status = reinterpret_cast<unsigned int*>(p.scratch);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int u_begin = (int)((long long)cta * p.units / G);      // half-units [u_begin, u_end) of this CTA
    const int u_end = (int)((long long)(cta + 1) * p.units / G);
    const int kc_begin = u_begin % p.kchunks;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&fullb_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
            ptx::mbar_init(&sfa_bar[s], 4);
        }
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

    if (warp == 0) {
        // ------------------------------------------------------------------ weight stream
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
            const uint64_t pol = ptx::policy_evict_first();
            int stage = 0;
            uint32_t ph = 0;
            int hu = u_begin, tile = u_begin / p.kchunks, kc = kc_begin;
            while (hu < u_end) {
                const int tile_end = hu - kc + p.kchunks;
                const int seg_end = tile_end < u_end ? tile_end : u_end;
                const int row0 = tile * kRT;
                while (hu < seg_end) {
                    const int cnt = (seg_end - hu) >= hps ? hps : 1;
                    ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, 0xB00u + (unsigned)stage);
                    ptx::mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)(kPackedBytes + kScaleBytes) * cnt);
                    for (int h = 0; h < cnt; ++h) {
                        const int k0 = (kc + h) * kKC;
                        ptx::tma_load_2d(s_w + (stage * hps + h) * kPackedBytes, &tm_packed, &full_bar[stage], k0 >> 1, row0, pol);
                        ptx::tma_load_2d(s_raw + (stage * hps + h) * kScaleBytes, &tm_scale, &full_bar[stage], k0 >> 4, row0, pol);
                    }
                    hu += cnt;
                    kc += cnt;
                    if (++stage == stages) { stage = 0; ph ^= 1u; }
                }
                if (kc >= p.kchunks) { kc = 0; ++tile; }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ activation stream (the pre-pass's output, from L2)
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_act);
            ptx::prefetch_tensormap(&tm_sfb);
            ptx::griddep_wait();                              // the pre-pass is the kernel before this one
            const uint64_t pol = ptx::policy_evict_last();
            int stage = 0;
            uint32_t ph = 0;
            int hu = u_begin, kc = kc_begin;
            while (hu < u_end) {
                const int tile_end = hu - kc + p.kchunks;
                const int seg_end = tile_end < u_end ? tile_end : u_end;
                while (hu < seg_end) {
                    const int cnt = (seg_end - hu) >= hps ? hps : 1;
                    ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, 0xB10u + (unsigned)stage);
                    ptx::mbar_arrive_expect_tx(&fullb_bar[stage], (uint32_t)(b_bytes + sfb_bytes) * cnt);
                    for (int h = 0; h < cnt; ++h) {
                        ptx::tma_load_2d(s_b + (stage * hps + h) * b_bytes, &tm_act, &fullb_bar[stage], (kc + h) * (kKC / 2), 0, pol);
                        ptx::tma_load_2d(s_sfb + (stage * hps + h) * sfb_bytes, &tm_sfb, &fullb_bar[stage], 0, (kc + h) * p.groups, pol);
                    }
                    hu += cnt;
                    kc += cnt;
                    if (++stage == stages) { stage = 0; ph ^= 1u; }
                }
                if (kc >= p.kchunks) kc = 0;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = fp4_idesc(p.NCp);
            const uint32_t sf_col = 2u * (uint32_t)p.acc_stride;
            int stage = 0, acc = 0;
            uint32_t ph = 0, pt = 0;
            int hu = u_begin, kc = kc_begin;
            while (hu < u_end) {
                const int tile_end = hu - kc + p.kchunks;
                const int seg_end = tile_end < u_end ? tile_end : u_end;
                ptx::mbar_wait(&tempty[acc], ((pt >> acc) & 1u) ^ 1u, s_abort, status, 0xB20u + (unsigned)acc);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.acc_stride);
                bool first = true;
                while (hu < seg_end) {
                    const int cnt = (seg_end - hu) >= hps ? hps : 1;
                    // the scales are in tensor memory (the warps that put them there waited for both operands; so does
                    // this thread, which is the one whose MMAs read them)
                    ptx::mbar_wait(&sfa_bar[stage], ph, s_abort, status, 0xB30u + (unsigned)stage);
                    ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0xB30u + (unsigned)stage);
                    ptx::mbar_wait(&fullb_bar[stage], ph, s_abort, status, 0xB30u + (unsigned)stage);
                    tc_fence_after();
                    for (int h = 0; h < cnt; ++h) {
                        const int bslot = stage * hps + h;
                        const uint32_t sfa_t = tmem_base + sf_col + 32 * (uint32_t)(stage * hps + h), sfb_t = sfa_t + 16;
                        const uint32_t a_addr = ptx::smem_u32(s_w + (stage * hps + h) * kPackedBytes);
                        const uint32_t b_addr = ptx::smem_u32(s_b + bslot * b_bytes);
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
        // rows L, L + 32, L + 64, L + 96 in columns 4 s .. 4 s + 3, and the words of activation columns L,
        // 32 + L, 64 + L in columns 16 + 4 s .. 18 + 4 s (an MMA's scale base sits on a multiple of four columns).
        const int q = warp - 4;
        const uint32_t sf_col = 2u * (uint32_t)p.acc_stride;
        int stage = 0;
        uint32_t ph = 0;
        int hu = u_begin, kc = kc_begin;
        while (hu < u_end) {
            const int tile_end = hu - kc + p.kchunks;
            const int seg_end = tile_end < u_end ? tile_end : u_end;
            while (hu < seg_end) {
                const int cnt = (seg_end - hu) >= hps ? hps : 1;
                ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0xB40u + (unsigned)stage);
                ptx::mbar_wait(&fullb_bar[stage], ph, s_abort, status, 0xB40u + (unsigned)stage);
                for (int h = 0; h < cnt; ++h) {
                    const int bslot = stage * hps + h;
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
                    const unsigned char* sb = s_sfb + bslot * sfb_bytes + lane * 16;
                    const uint4 b0 = *reinterpret_cast<const uint4*>(sb);
                    uint4 b1 = make_uint4(0u, 0u, 0u, 0u), b2 = b1;
                    if (p.groups > 1) b1 = *reinterpret_cast<const uint4*>(sb + 512);
                    if (p.groups > 2) b2 = *reinterpret_cast<const uint4*>(sb + 1024);
                    rb[0] = b0.x; rb[1] = b1.x; rb[2] = b2.x; rb[3] = 0u;
                    rb[4] = b0.y; rb[5] = b1.y; rb[6] = b2.y; rb[7] = 0u;
                    rb[8] = b0.z; rb[9] = b1.z; rb[10] = b2.z; rb[11] = 0u;
                    rb[12] = b0.w; rb[13] = b1.w; rb[14] = b2.w; rb[15] = 0u;
                    const uint32_t t = tmem_base + ((uint32_t)(q * 32) << 16) + sf_col + (uint32_t)(32 * (stage * hps + h));
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
        if (te == 0) *s_epoch = ptx::take_launch_epoch(p.scratch);      // this launch's tag for the split-tile pairs
        unsigned char* pairs = p.pairs;
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
            ptx::mbar_wait(&tfull[acc], (pt >> acc) & 1u, s_abort, status, 0xB50u + (unsigned)acc);
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)(acc * p.acc_stride);
            float v[fp4::kMaxTokens];
#pragma unroll
            for (int m = 0; m < fp4::kMaxTokens; ++m) v[m] = 0.0f;
#pragma unroll
            for (int c0 = 0; c0 < kMaxCols; c0 += 16) {
                if (c0 < p.NCp) {
                    uint32_t r[16];
                    tmem_ld16(t_addr + c0, r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int c = c0 + i;                 // column c = token * TERMS + term (compile-time after unrolling)
                        if (c / TERMS < fp4::kMaxTokens) v[c / TERMS] += __uint_as_float(r[i]);
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
            for (int m = 0; m < fp4::kMaxTokens; ++m)
                if (m < p.M) v[m] *= p.unscale[m];
            if (!owner) {
                unsigned char* slot = pairs + (size_t)cta * (kPairTokens * kRT) * 8;
#pragma unroll
                for (int m = 0; m < fp4::kMaxTokens; ++m)
                    if (m < p.M) ptx::st_volatile_v2(slot + (m * kRT + te) * 8, __float_as_uint(v[m]), epoch);
            } else {
                fp4_gather_pairs(v, pairs, (size_t)(kPairTokens * kRT) * 8, cta + 1, last, p.M, te, epoch, s_abort, status, 0xB60u);
                fp4_store_rows(v, p.out, tile, te);
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

constexpr int kFixedSmem = 1024 + (4 * kMaxStages + 4) * 8 + 64;

bool plan_fp4(const LinearArgs& a, const nvfp4_device_info& dev, Fp4Plan* out) {
    Fp4Params& p = out->p;
    p = Fp4Params{};
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.NCp = (a.M * fp4::terms_for(a.M) + 15) / 16 * 16;
    if (p.NCp > kMaxCols) return false;
    p.groups = (p.NCp + 31) / 32;
    p.acc_stride = p.NCp <= 64 ? 64 : 128;
    p.kchunks = a.K / kKC;
    const long long units = (long long)((a.N + kRT - 1) / kRT) * p.kchunks;
    if (units > 0x7fffffffLL || units < 1) return false;
    p.units = (int)units;
    int grid = dev.sm_count < kMaxGrid ? dev.sm_count : kMaxGrid;
    if (grid > p.units) grid = p.units;
    const int ring_half_units = (512 - 2 * p.acc_stride) / 32;       // 32 tensor-memory columns of scales per half-unit of the ring
    const int w_unit = kPackedBytes + kScaleBytes, b_unit = p.NCp * 128 + p.groups * 512;     // per half-unit: the weights' codes and scales, the activations'
    // Every ring stage carries the slice of the activations its weights multiply.
    const long long avail = kSmemBudget - kFixedSmem;
    const int unit = w_unit + b_unit;
    // Two half-units per stage when three such stages fit (fewer, larger hand-overs between the warps)
    p.hps = avail / (2 * unit) >= 3 ? 2 : 1;
    long long stages = avail / ((long long)p.hps * unit);
    if (stages < 3) return false;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages * p.hps > ring_half_units) stages = ring_half_units / p.hps;
    p.stages = (int)stages;
    out->grid = grid;
    out->smem = kFixedSmem + (int)stages * p.hps * unit;
    return true;
}

}  // namespace

bool decode_fp4_stream_supported(const LinearArgs& a, const nvfp4_device_info& dev) {
    if (a.M < 1 || a.M > fp4::kMaxTokens || (a.K % kKC) != 0 || a.N < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u)) return false;
    if (a.px || a.packed2 || !act_to_fp4_supported(a)) return false;
    if (a.swiglu_out && (a.residual || a.out_f32 || (a.N & 15))) return false;
    Fp4Plan pl;
    return plan_fp4(a, dev, &pl);
}

cudaError_t configure_decode_fp4_stream() {
    cudaError_t e = configure_large_smem(decode_fp4_stream_kernel<5>, kSmemBudget);
    if (e != cudaSuccess) return e;
    return configure_large_smem(decode_fp4_stream_kernel<6>, kSmemBudget);
}

cudaError_t launch_decode_fp4_stream(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t pairs_offset, void* act,
                              int* launches, cudaStream_t s) {
    Fp4Plan pl;
    if (!plan_fp4(a, dev, &pl)) return cudaErrorInvalidValue;
    Fp4Params& p = pl.p;
    unsigned char* codes = static_cast<unsigned char*>(act);
    unsigned char* sfb = codes + fp4::act_sfb_offset(a.K);
    float* unscale = reinterpret_cast<float*>(codes + fp4::act_unscale_offset(a.K));
    CUtensorMap tmp, tms, tma, tmf;
    if (!make_map_cached(dev.maps, &tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, kRT,
                         CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, kRT,
                         CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_map_cached(dev.maps, &tma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, (uint64_t)a.K / 2, (uint64_t)p.NCp, 128,
                         (uint32_t)p.NCp, CU_TENSOR_MAP_SWIZZLE_128B) ||
        // the activations' block scales: one row of 512 bytes (128 words) per k-chunk and column group
        !make_map_cached(dev.maps, &tmf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sfb, 128, (uint64_t)p.kchunks * p.groups, 128,
                         (uint32_t)p.groups, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    const int terms = fp4::terms_for(a.M);
    cudaError_t e = launch_act_to_fp4(a, terms, p.groups, codes, sfb, unscale, s);
    if (e != cudaSuccess) return e;
    p.out.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.out.C = static_cast<__nv_bfloat16*>(a.C);
    p.out.M = a.M;
    p.out.N = a.N;
    p.out.swiglu_out = a.swiglu_out ? 1 : 0;
    p.unscale = unscale;
    p.scratch = static_cast<unsigned char*>(scratch);
    p.pairs = p.scratch + pairs_offset;
    p.out.inv_gs = a.inv_gs;
    p.out.out_f32 = a.out_f32 ? 1 : 0;
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
    e = terms == 6 ? cudaLaunchKernelEx(&cfg, decode_fp4_stream_kernel<6>, tmp, tms, tma, tmf, p)
                   : cudaLaunchKernelEx(&cfg, decode_fp4_stream_kernel<5>, tmp, tms, tma, tmf, p);
    if (launches) *launches = 2;
    return e;
}

}  // namespace nvfp4
