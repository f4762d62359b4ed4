// Prefill GEMM for M > 16: fused NVFP4 dequantisation + tcgen05 tensor-core GEMM.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W = e2m1(code) * ue4m3(scale) / global_scale
//
// One persistent CTA per SM works on 128-token x 256-weight-row output tiles, two token tiles of
// one weight tile at a time where the shape allows (both read the same dequantised B blocks, one
// accumulator each), whole waves of such pairs first in an interleaved order; the tiles left over
// are split along k over all CTAs (stream-K) and summed from FP32 partial tiles in a fixed order.
//   warp 0      TMA producer: activation tiles (128 tokens x 64 k, FP16, 128-byte swizzle) into a
//               4-stage ring, raw weight stages (256 rows x 256 k of packed codes + scales, 36 KB)
//               into a 2-stage ring.  Plain tiled TMA, never cluster multicast.
//   warps 8-15  dequantise: thread = one weight row; per 64-k block two 128-bit loads of codes,
//               cvt.rn.f16x2.e2m1x2 + one f16x2 multiply by the block scale (exact products), eight
//               128-bit stores into the K-major, 128-byte-swizzled B operand tile (2 buffers).
//   warp 1      one elected thread issues tcgen05.mma (kind::f16, M=128, N=256, K=16) from the two
//               shared-memory operands into a TMEM accumulator (2 x 256 columns, double buffered)
//               and commits completion to the mbarriers that recycle the operand buffers.
//   warps 4-7   epilogue: tcgen05.ld the FP32 accumulator (lane = token), undo the per-token
//               activation scale and apply 1/global_scale in FP32, add the residual, round once to
//               BF16, 64 contiguous bytes per thread per step.
//
// Operands are FP16 because the hardware E2M1 conversion produces FP16 and every e2m1 x ue4m3
// product is exact in FP16.  A small pre-pass turns the BF16 activations into FP16 with an exact
// per-token power-of-two scale (largest magnitude -> [2^14, 2^15)) in the handle workspace, so
// BF16's wider exponent range costs nothing; accumulation is FP32 in TMEM.  The arithmetic is
// the reference's GEMM (src/engine/dense_gemm_fp4_sm110.cu:558-583) with exact instead of
// BF16-rounded weights (identical when global_scale = 1) and no materialised [N,K] matrix.
//
// Every mbarrier wait is bounded; a wait that runs out records its code in the handle's status
// word and the kernel winds down (TMEM is always freed).
#include <cuda.h>
#include <cmath>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "ptx.cuh"
#include "umma.cuh"

namespace nvfp4 {
namespace {

using namespace umma;

constexpr int BM = 128;            // tokens per tile   (UMMA M)
constexpr int BN = 256;            // weight rows per tile (UMMA N)
constexpr int BK = 64;             // k per MMA operand block (128 bytes of FP16: one swizzle row)
constexpr int WK = 256;            // k per raw weight stage (4 operand blocks)
constexpr int kAStages = 4, kWStages = 2, kBBufs = 2, kAccs = 2;
constexpr int kBBufsDense = 4;     // BF16 weights: the raw-weight ring is not needed and holds two more B blocks
constexpr int kABytes = BM * BK * 2;          // 16 KB
constexpr int kBBytes = BN * BK * 2;          // 32 KB
constexpr int kWPackedBytes = BN * WK / 2;    // 32 KB
constexpr int kWScaleBytes = BN * WK / 16;    // 4 KB
constexpr int kThreads = 512;
constexpr int kDequantWarps = 8, kEpiWarps = 4;
constexpr int kSmemBytes = 1024 + kAStages * kABytes + kWStages * (kWPackedBytes + kWScaleBytes) +
                           kBBufs * kBBytes + 256 /*barriers, tmem slot, abort*/;

constexpr int kPartialVec = BM * BN / 4;      // float4 elements of one FP32 partial tile

struct PrefillParams {
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    const float* unscale;      // per token: 1 / activation scale
    unsigned int* status;
    float inv_gs;
    int M, N, K;
    int m_tiles, n_tiles;
    // stream-K region: tiles [0, sk_tiles).  A tile cut by a span boundary is finished by the CTA
    // holding its first stage, which adds the other CTAs' FP32 partial tiles in CTA order.
    int sk_tiles;
    int sk_pairs;              // the same region counted in pairs of token tiles (see Schedule)
    float4* partials;          // [grid][2][64 column chunks][128 token rows] FP32 x 4
    unsigned int* flags;       // [grid][2], the launch's tag once that partial tile is stored
    int swiglu_out;            // weight rows interleaved in slabs of 16 (8 gate, 8 up): C is [M, N/2] = bf16(silu(gate) * up)
    int dense;                 // 1 = BF16 weights and activations as they are: no token scale, no 2^8, no global scale
    int out_f32;               // C is FP32 [M,N]: the scaled sums unrounded, no residual (partials a caller reduces itself)
    // wround: the weight operand is bf16(lut * (scale * inv_gs)) * wshift (a power of two that keeps it in FP16's normal
    // range; 8 significant bits, so exact), the reference's arithmetic above 8 tokens, instead of exact lut * scale / 2^8.
    int wround;
    float wshift;
    float out_mul;             // what the epilogue multiplies the sums by besides the token factor: 2^8 / gs, or 1 / wshift
};

// ---------------------------------------------------------------- tcgen05 helpers
// kind::f16, A = B = FP16, D = FP32, both operands K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t kInstrDescBf16 = kInstrDesc | (1u << 7) | (1u << 10);   // A and B formats: BF16

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Reduction of one split tile.  Every CTA holding a part of the tile calls this once its own
// parts are stored: it waits (bounded) for the partial tiles of all P participants, sums them
// in CTA order over its own 1/P of the tile and writes that part of the output.  All
// participants add in the same order, so the result does not depend on timing.
// t = 0..nthreads-1, nthreads a multiple of 128.
__device__ __forceinline__ void reduce_split_tile(const PrefillParams& p, unsigned int epoch, int tile, int kstages, int t,
                                                  int nthreads, volatile int* s_abort) {
    int first, last;
    split_tile_participants(p.sk_tiles, kstages, tile, first, last);
    if (!wait_split_tile_flags(p.flags, epoch, first, last, t, s_abort, p.status)) return;
    const int P = last - first + 1, me = blockIdx.x - first;
    const int j0 = (int)((long long)me * kPartialVec / P) & ~(BM - 1);
    const int j1 = me + 1 == P ? kPartialVec : ((int)((long long)(me + 1) * kPartialVec / P) & ~(BM - 1));
    const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;
    const int m = mt * BM + (t & (BM - 1));
    const float mul = p.dense ? 1.0f : (m < p.M ? p.unscale[m] : 0.0f) * p.out_mul;
    const float4* head = p.partials + ((size_t)first * 2 + 1) * kPartialVec;
    // sum of the participants' partials of one chunk (4 columns x this token row), in CTA order
    auto chunk_sum = [&](int j) {
        float4 s = __ldcg(head + j);
        for (int c = first + 1; c <= last; c += 8) {
            float4 x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)      // eight loads in flight; absent participants add zero
                x[i] = c + i <= last ? __ldcg(p.partials + (size_t)(c + i) * 2 * kPartialVec + j)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) { s.x += x[i].x; s.y += x[i].y; s.z += x[i].z; s.w += x[i].w; }
        }
        return s;
    };
    for (int j = j0 + t; j < j1; j += nthreads) {
        const int n = nt * BN + (j / BM) * 4;          // first of the 4 columns of this chunk
        if (p.swiglu_out) {
            // columns 16s..16s+7 are gate values, 16s+8..16s+15 their up values: a gate chunk takes the up
            // chunk two chunks further (wherever it lies in the tile) and writes 4 outputs; up chunks are skipped
            if ((n & 15) >= 8 || m >= p.M || n >= p.N) continue;
            const float4 g = chunk_sum(j), u = chunk_sum(j + 2 * BM);
            const float gf[4] = {g.x, g.y, g.z, g.w}, uf[4] = {u.x, u.y, u.z, u.w};
            float f[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                f[i] = silu(__bfloat162float(__float2bfloat16_rn(gf[i] * mul))) * __bfloat162float(__float2bfloat16_rn(uf[i] * mul));
            const __nv_bfloat162 b0 = __floats2bfloat162_rn(f[0], f[1]);
            const __nv_bfloat162 b1 = __floats2bfloat162_rn(f[2], f[3]);
            *reinterpret_cast<uint2*>(p.C + (size_t)m * (p.N / 2) + 8 * (n >> 4) + (n & 15)) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
            continue;
        }
        const float4 s = chunk_sum(j);
        if (m < p.M && n < p.N) {                      // N % 8 == 0: a chunk of 4 is inside or outside
            const size_t o = (size_t)m * p.N + n;
            float f[4] = {s.x * mul, s.y * mul, s.z * mul, s.w * mul};
            if (p.out_f32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + o) = make_float4(f[0], f[1], f[2], f[3]);
                continue;
            }
            if (p.residual) {
                const uint2 rr = *reinterpret_cast<const uint2*>(p.residual + o);
                f[0] += bf16_bits_to_float(rr.x & 0xFFFFu);
                f[1] += bf16_bits_to_float(rr.x >> 16);
                f[2] += bf16_bits_to_float(rr.y & 0xFFFFu);
                f[3] += bf16_bits_to_float(rr.y >> 16);
            }
            const __nv_bfloat162 b0 = __floats2bfloat162_rn(f[0], f[1]);
            const __nv_bfloat162 b1 = __floats2bfloat162_rn(f[2], f[3]);
            *reinterpret_cast<uint2*>(p.C + o) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
        }
    }
}

// DENSE: the weight is BF16 [N,K] (tm_packed is its tensor map, boxes of 64 k x 256 rows; tm_scale is
// unused) and the activations are the caller's BF16 rows: the producer loads the B blocks straight
// into the operand buffers, the dequantisation warps have nothing to do.
template <bool DENSE, bool WROUND = false>
__global__ void __launch_bounds__(kThreads, 1)
prefill_umma_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_packed,
                    const __grid_constant__ CUtensorMap tm_scale, const PrefillParams p) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by an offset on the shared-memory array itself: the pointer keeps its
    // address space, so every access below is a shared-memory instruction with a 32-bit address
    // (rounding a generic 64-bit pointer instead turns them into generic loads and stores).
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* s_a = smem;                                        // kAStages x 16 KB
    unsigned char* s_b = s_a + kAStages * kABytes;                    // kBBufs x 32 KB
    unsigned char* s_wp = s_b + kBBufs * kBBytes;                     // kWStages x 32 KB packed codes
    unsigned char* s_ws = s_wp + kWStages * kWPackedBytes;            // kWStages x 4 KB scales
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_ws + kWStages * kWScaleBytes);
    uint64_t* afull = bars;                  // [kAStages]
    uint64_t* aempty = afull + kAStages;     // [kAStages]
    uint64_t* wfull = aempty + kAStages;     // [kWStages]
    uint64_t* wempty = wfull + kWStages;     // [kWStages]
    constexpr int NB = DENSE ? kBBufsDense : kBBufs;   // B operand buffers (DENSE: s_b runs on into the raw-weight ring)
    uint64_t* bfull = wempty + kWStages;     // [NB]
    uint64_t* bempty = bfull + kBBufsDense;  // [NB]
    uint64_t* tfull = bempty + kBBufsDense;  // [kAccs]
    uint64_t* tempty = tfull + kAccs;        // [kAccs]
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tempty + kAccs);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    volatile unsigned int* s_epoch = reinterpret_cast<volatile unsigned int*>(s_tmem + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kstages = p.K / WK;
    const bool all_reduce = p.sk_tiles == p.m_tiles * p.n_tiles;

    if (tid == 0) {
        for (int i = 0; i < kAStages; ++i) { ptx::mbar_init(&afull[i], 1); ptx::mbar_init(&aempty[i], 1); }
        for (int i = 0; i < kWStages; ++i) { ptx::mbar_init(&wfull[i], 1); ptx::mbar_init(&wempty[i], kDequantWarps); }
        for (int i = 0; i < NB; ++i) { ptx::mbar_init(&bfull[i], DENSE ? 1 : kDequantWarps); ptx::mbar_init(&bempty[i], 1); }
        for (int i = 0; i < kAccs; ++i) { ptx::mbar_init(&tfull[i], 1); ptx::mbar_init(&tempty[i], kEpiWarps); }
        *s_abort = 0;
        // The tag of this launch's stream-K flags, from the counter in the scratch.  (This kernel is
        // launched without programmatic serialisation: the previous launch has completed.)
        *s_epoch = ptx::take_launch_epoch(p.status);
        ptx::fence_mbar_init();
    }
    if (warp == 1) {   // one warp owns the TMEM allocation: 512 columns = two 128 x 256 FP32 accumulators
        tmem_alloc_512(s_tmem);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    const unsigned int epoch = *s_epoch;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_act);
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
            const uint64_t pol_w = ptx::policy_evict_first(), pol_a = ptx::policy_evict_last();
            int sa = 0, sw = 0, sb = 0;
            uint32_t pa = 0, pw = 0, pb = 0;
            Schedule sched(p.sk_tiles, p.sk_pairs, p.m_tiles, p.n_tiles, kstages);
            Segment sg;
            while (sched.next(sg)) {
                const int nt = sg.tile / p.m_tiles, mt = sg.tile % p.m_tiles;
                for (int ks = sg.ks0; ks < sg.ks1; ++ks) {
                    if (!DENSE) {
                        ptx::mbar_wait(&wempty[sw], pw ^ 1u, s_abort, p.status, 0x410u + sw);
                        ptx::mbar_arrive_expect_tx(&wfull[sw], kWPackedBytes + kWScaleBytes);
                        ptx::tma_load_2d(s_wp + sw * kWPackedBytes, &tm_packed, &wfull[sw], ks * (WK / 2), nt * BN, pol_w);
                        ptx::tma_load_2d(s_ws + sw * kWScaleBytes, &tm_scale, &wfull[sw], ks * (WK / 16), nt * BN, pol_w);
                        if (++sw == kWStages) { sw = 0; pw ^= 1u; }
                    }
                    for (int j = 0; j < WK / BK; ++j) {
                        if (DENSE) {      // the B block of this 64-k step, as the tensor core wants it
                            ptx::mbar_wait(&bempty[sb], pb ^ 1u, s_abort, p.status, 0x410u + sb);
                            ptx::mbar_arrive_expect_tx(&bfull[sb], kBBytes);
                            ptx::tma_load_2d(s_b + sb * kBBytes, &tm_packed, &bfull[sb], ks * WK + j * BK, nt * BN, pol_w);
                            if (++sb == NB) { sb = 0; pb ^= 1u; }
                        }
                        for (int i = 0; i < sg.pair; ++i) {       // one activation tile per token tile of the pair
                            ptx::mbar_wait(&aempty[sa], pa ^ 1u, s_abort, p.status, 0x400u + sa);
                            ptx::mbar_arrive_expect_tx(&afull[sa], kABytes);
                            ptx::tma_load_2d(s_a + sa * kABytes, &tm_act, &afull[sa], ks * WK + j * BK, (mt + i) * BM, pol_a);
                            if (++sa == kAStages) { sa = 0; pa ^= 1u; }
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // A pair of token tiles shares every dequantised B block: eight MMAs per 64-k block instead
            // of four for the same shared-memory fill, into both accumulators at once.  Single tiles
            // alternate between the two accumulators so that the epilogue of one overlaps the next.
            int sa = 0, sb = 0, next_acc = 0;
            uint32_t pa = 0, pb = 0, ptbits = 0;      // bit a of ptbits: phase parity of accumulator a
            Schedule sched(p.sk_tiles, p.sk_pairs, p.m_tiles, p.n_tiles, kstages);
            Segment sg;
            while (sched.next(sg)) {
                const int acc0 = sg.pair == 2 ? 0 : next_acc;
                for (int i = 0; i < sg.pair; ++i)
                    ptx::mbar_wait(&tempty[acc0 + i], ((ptbits >> (acc0 + i)) & 1u) ^ 1u, s_abort, p.status, 0x440u + acc0 + i);
                tc_fence_after();
                for (int kb = 0; kb < (sg.ks1 - sg.ks0) * (WK / BK); ++kb) {
                    ptx::mbar_wait(&bfull[sb], pb, s_abort, p.status, 0x430u + sb);
                    // Both operands arrive through shared memory (TMA, or generic stores followed by
                    // fence.proxy.async before the arrive): no tcgen05 fence is needed per k-block.
                    const uint32_t b_addr = ptx::smem_u32(s_b + sb * kBBytes);
                    for (int i = 0; i < sg.pair; ++i) {
                        ptx::mbar_wait(&afull[sa], pa, s_abort, p.status, 0x420u + sa);
                        const uint32_t a_addr = ptx::smem_u32(s_a + sa * kABytes);
                        const uint32_t d_tmem = tmem_base + (uint32_t)(acc0 + i) * BN;
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            umma_f16(d_tmem, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32),
                                     (kb > 0 || k > 0) ? 1u : 0u, DENSE ? kInstrDescBf16 : kInstrDesc);
                        }
                        umma_commit(&aempty[sa]);  // operand buffers are free once these MMAs have read them
                        if (++sa == kAStages) { sa = 0; pa ^= 1u; }
                    }
                    umma_commit(&bempty[sb]);
                    if (++sb == NB) { sb = 0; pb ^= 1u; }
                }
                for (int i = 0; i < sg.pair; ++i) {
                    umma_commit(&tfull[acc0 + i]);  // accumulator complete
                    ptbits ^= 1u << (acc0 + i);
                }
                if (sg.pair == 1) next_acc ^= 1;
            }
        }
    } else if (warp >= 8 && !DENSE) {
        // ------------------------------------------------------------------ dequantise: thread = weight row
        const int row = tid - 8 * 32;                     // 0..255
        const int sw7 = row & 7;
        int sw = 0, sb = 0;
        uint32_t pw = 0, pb = 0;
        Schedule sched(p.sk_tiles, p.sk_pairs, p.m_tiles, p.n_tiles, kstages);
        Segment sg;
        while (sched.next(sg)) {
            for (int ks = sg.ks0; ks < sg.ks1; ++ks) {
                ptx::mbar_wait(&wfull[sw], pw, s_abort, p.status, 0x450u + sw);
                const unsigned char* wp = s_wp + sw * kWPackedBytes + row * 128;
                const uint4 sc16 = *reinterpret_cast<const uint4*>(s_ws + sw * kWScaleBytes + row * 16);
                const uint32_t scw[4] = {mask_scale_bytes(sc16.x), mask_scale_bytes(sc16.y), mask_scale_bytes(sc16.z),
                                         mask_scale_bytes(sc16.w)};
#pragma unroll
                for (int j = 0; j < WK / BK; ++j) {
                    // packed bytes [32j, 32j+32) of the row = logical 16-byte chunks 2j, 2j+1
                    const uint4 q0 = *reinterpret_cast<const uint4*>(wp + (((2 * j) ^ sw7) << 4));
                    const uint4 q1 = *reinterpret_cast<const uint4*>(wp + (((2 * j + 1) ^ sw7) << 4));
                    const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    ptx::mbar_wait(&bempty[sb], pb ^ 1u, s_abort, p.status, 0x460u + sb);
                    unsigned char* bp = s_b + sb * kBBytes + row * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {          // chunk c = 8 consecutive k = one 32-bit word of codes
                        uint32_t e[4];
                        ptx::cvt_e2m1x8_to_f16x2(q[c], e);
                        if (WROUND) {
                            // the reference's dequantisation, operation for operation: FP32 block scale times 1/gs, FP32
                            // product with the code's value, one rounding to BF16; then a power of two into FP16 (exact)
                            const float bs = ue4m3_to_float((scw[j] >> (8 * (c >> 1))) & 0xFFu) * p.inv_gs;
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 l = __half22float2(*reinterpret_cast<const __half2*>(&e[i]));
                                const float2 b = __bfloat1622float2(__floats2bfloat162_rn(l.x * bs, l.y * bs));
                                o[i] = ptx::pack_f16x2(b.x * p.wshift, b.y * p.wshift);
                            }
                            *reinterpret_cast<uint4*>(bp + ((c ^ sw7) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                            continue;
                        }
                        const uint32_t S = scale_byte_to_f16x2(scw[j], c >> 1);     // scale / 2^8, undone in the epilogue
                        *reinterpret_cast<uint4*>(bp + ((c ^ sw7) << 4)) =
                            make_uint4(ptx::mul_f16x2(e[0], S), ptx::mul_f16x2(e[1], S), ptx::mul_f16x2(e[2], S),
                                       ptx::mul_f16x2(e[3], S));
                    }
                    ptx::fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&bfull[sb]);
                    if (++sb == kBBufs) { sb = 0; pb ^= 1u; }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&wempty[sw]);
                if (++sw == kWStages) { sw = 0; pw ^= 1u; }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------------ epilogue: thread = token row
        const int ew = warp - 4;                          // TMEM lanes 32*ew .. 32*ew+31
        int next_acc = 0;                                     // mirrors the MMA issuer's choice of accumulators
        uint32_t ptbits = 0;                                  // bit a: phase parity of accumulator a
        const int te = ew * 32 + lane;                        // 0..127: TMEM lane, token row of the tile
        const long long sk_units = (long long)p.sk_tiles * kstages;
        int pend[2] = {-1, -1};                               // split tiles whose partial this CTA has stored
        Schedule sched(p.sk_tiles, p.sk_pairs, p.m_tiles, p.n_tiles, kstages);
        Segment sg;
        bool more = sched.next(sg);
        while (more) {
          for (int pi = 0; pi < sg.pair; ++pi) {              // the tiles of a pair one after the other
            const int tile = sg.tile + pi;
            const int acc = sg.pair == 2 ? pi : next_acc;
            const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;
            const int m = mt * BM + te;
            const bool complete = sg.ks0 == 0 && sg.ks1 == kstages;
            ptx::mbar_wait(&tfull[acc], (ptbits >> acc) & 1u, s_abort, p.status, 0x470u + acc);
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)acc * BN;
            if (!complete) {
                // Part of a split tile: raw FP32 sums to this CTA's partial tile.  Layout
                // [column chunk of 4][token row], so a warp's store covers 512 contiguous bytes.
                const int which = sg.ks0 == 0 ? 1 : 0;        // head of a tile (span end) or tail (span start)
                float4* slot = p.partials + ((size_t)blockIdx.x * 2 + which) * kPartialVec;
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(t_addr + c0, r);
#pragma unroll
                    for (int v = 0; v < 8; ++v)
                        __stcg(slot + (c0 / 4 + v) * BM + te,
                               make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                           __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3])));
                }
                __threadfence();
                ptx::named_barrier_sync(1, kEpiWarps * 32);   // all 128 rows stored before the flag goes up
                if (te == 0) ptx::st_release_gpu(&p.flags[blockIdx.x * 2 + which], epoch);
                pend[which] = tile;
            } else {
                const float mul = DENSE ? 1.0f : (m < p.M ? p.unscale[m] : 0.0f) * p.out_mul;
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(t_addr + c0, r);
                    const int n0 = nt * BN + c0;
                    if (p.swiglu_out) {
                        // 32 columns = two slabs of 8 gate values and their 8 up values (N % 32 == 0 here)
                        if (m < p.M && n0 < p.N) {
#pragma unroll
                            for (int sv = 0; sv < 2; ++sv) {
                                uint32_t ov[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    float f[2];
#pragma unroll
                                    for (int e = 0; e < 2; ++e) {
                                        const float gate = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[sv * 16 + 2 * i + e]) * mul));
                                        const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[sv * 16 + 8 + 2 * i + e]) * mul));
                                        f[e] = silu(gate) * up;
                                    }
                                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(f[0], f[1]);
                                    ov[i] = *reinterpret_cast<const uint32_t*>(&b2);
                                }
                                *reinterpret_cast<uint4*>(p.C + (size_t)m * (p.N / 2) + (n0 >> 1) + 8 * sv) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
                            }
                        }
                    } else
                    if (m < p.M && n0 < p.N) {
                        const size_t o = (size_t)m * p.N + n0;
                        if (p.out_f32) {
                            float* dst = reinterpret_cast<float*>(p.C) + o;
#pragma unroll
                            for (int i = 0; i < 32; i += 4)      // N % 8 == 0: whole groups of 4
                                if (n0 + i < p.N) *reinterpret_cast<float4*>(dst + i) =
                                    make_float4(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul,
                                                __uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
                        } else
                        if (n0 + 32 <= p.N) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                float f[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]) * mul;
                                if (p.residual) {
                                    const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + o + v * 8);
                                    const uint32_t rv[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        f[2 * i] += bf16_bits_to_float(rv[i] & 0xFFFFu);
                                        f[2 * i + 1] += bf16_bits_to_float(rv[i] >> 16);
                                    }
                                }
                                uint32_t ov[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                                    ov[i] = *reinterpret_cast<const uint32_t*>(&b2);
                                }
                                *reinterpret_cast<uint4*>(p.C + o + v * 8) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {       // unrolled: r[] stays in registers
                                if (n0 + i >= p.N) continue;
                                float f = __uint_as_float(r[i]) * mul;
                                if (p.residual) f += __bfloat162float(p.residual[o + i]);
                                p.C[o + i] = __float2bfloat16_rn(f);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tempty[acc]);
            ptbits ^= 1u << acc;
          }
            if (sg.pair == 1) next_acc ^= 1;
            more = sched.next(sg);

            // Whole tiles follow the stream-K region: these four warps reduce the split tiles now,
            // behind the MMAs of the next tiles.  (With no whole tiles all warps do it at the end.)
            if (!all_reduce && (pend[0] >= 0 || pend[1] >= 0) && (!more || sg.tile >= p.sk_tiles)) {
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    if (pend[w] >= 0) reduce_split_tile(p, epoch, pend[w], kstages, te, kEpiWarps * 32, s_abort);
                    pend[w] = -1;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_512(tmem_base);
    }
    if (all_reduce) {
        // Every tile was split and nothing else is left to do: all 16 warps reduce.
        int split[2];
        split_tiles_of_cta(p.sk_tiles, kstages, split);
#pragma unroll
        for (int w = 0; w < 2; ++w)
            if (split[w] >= 0) reduce_split_tile(p, epoch, split[w], kstages, tid, kThreads, s_abort);
    }
}

size_t act_bytes(int M, int K) { return ((size_t)M * K * 2 + 255) / 256 * 256; }

}  // namespace

bool prefill_umma_supported(const LinearArgs& a) {
    if (a.M < 1 || (a.K % WK) != 0 || (a.N % 8) != 0) return false;
    if (a.swiglu_out && ((a.N % 32) != 0 || a.residual)) return false;
    if (a.out_f32 && (a.swiglu_out || a.residual)) return false;
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u)) return false;
    return true;
}

constexpr size_t kPartialTileBytes = (size_t)kPartialVec * 16;
constexpr int kMaxPrefillGrid = 160;
constexpr size_t kStreamKBytes = 4096 + 2 * kMaxPrefillGrid * kPartialTileBytes;

size_t prefill_umma_reserved_bytes() { return kStreamKBytes; }

// Stream-K flags and partial tiles (fixed place, so a flag word only ever holds launch tags),
// then the FP16 copy of the activations and one FP32 per token.
size_t prefill_umma_scratch_bytes(int max_M, int /*max_N*/, int max_K) {
    if (max_M <= 16) return 0;
    return kStreamKBytes + act_bytes(max_M, max_K) + ((size_t)max_M * 4 + 255) / 256 * 256;
}

cudaError_t configure_prefill_umma() {
    cudaError_t e = configure_large_smem(prefill_umma_kernel<true>, kSmemBytes);
    if (e == cudaSuccess) e = configure_large_smem(prefill_umma_kernel<false, true>, kSmemBytes);
    if (e != cudaSuccess) return e;
    return configure_large_smem(prefill_umma_kernel<false>, kSmemBytes);
}

// Plans the tiles of one launch (fills sk_tiles / sk_pairs) and returns the grid.
static int plan_tiles(PrefillParams& p, const nvfp4_device_info& dev) {
    // Whole tiles are handed out in pairs of consecutive token tiles of one weight tile (a pair
    // shares every dequantised B block, which is what the kernel is bound by); whole waves of
    // pairs run pair by pair, the pairs left over are split tile by tile along k over all CTAs
    // when that is shorter than one more wave.  Costs in stage-times: a pair's stage ~1.5 (eight
    // MMAs instead of four on the same shared-memory fill), a single tile's 1, the split ~6
    // (partial tiles written, flags, reduction), measured on gate_up/down shapes at 64..8192 tokens.
    const int tiles = p.m_tiles * p.n_tiles;
    const int ppn = (p.m_tiles + 1) / 2, pairs = p.n_tiles * ppn;
    const int kstages = p.K / WK;
    int grid = dev.sm_count < kMaxPrefillGrid ? dev.sm_count : kMaxPrefillGrid;
    if ((long long)tiles * kstages < grid) grid = tiles * kstages;   // then every tile is split, one stage per CTA
    auto tiles_of_pairs = [&](int np) { return (np / ppn) * p.m_tiles + ((np % ppn) * 2 < p.m_tiles ? (np % ppn) * 2 : p.m_tiles); };
    const double pair_cost = p.m_tiles >= 2 ? 1.5 : 1.0;
    p.sk_tiles = 0;
    p.sk_pairs = 0;
    const int left = pairs % grid;
    if (dev.prefill_stream_k && left > 0) {
        int skp = left;
        if ((long long)tiles_of_pairs(skp) * kstages < grid) skp += pairs >= grid ? grid : 0;   // every CTA gets at least one stage
        const int skt = tiles_of_pairs(skp);
        const double whole = (double)((pairs + grid - 1) / grid) * kstages * pair_cost;
        const double split = (double)((pairs - skp) / grid) * kstages * pair_cost + (double)(((long long)skt * kstages + grid - 1) / grid) + 6.0;
        if (split < whole && (long long)skt * kstages >= grid) { p.sk_pairs = skp; p.sk_tiles = skt; }
    }
    return grid;
}

// scratch: [0, 256) status word (shared with the GEMV kernel); from `offset` the stream-K flags
// (4 KB) and partial tiles, then the FP16 activations and the per-token factors.
cudaError_t launch_prefill_umma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t scratch_bytes,
                                size_t offset, int* launches, cudaStream_t s) {
    const size_t need = prefill_umma_scratch_bytes(a.M, a.N, a.K);
    if (offset + need > scratch_bytes) return cudaErrorMemoryAllocation;
    char* sk = static_cast<char*>(scratch) + offset;
    char* base = sk + kStreamKBytes;
    __half* ah = reinterpret_cast<__half*>(base);
    float* unscale = reinterpret_cast<float*>(base + act_bytes(a.M, a.K));
    CUtensorMap tma, tmp, tms;
    if (!make_map_cached(dev.maps, &tma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ah, (uint64_t)a.K, (uint64_t)a.M, BK, BM,
                  CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, BN,
                  CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, BN,
                  CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    cudaError_t e = launch_act_to_f16(a.A, a.M, a.K, ah, unscale, s);
    if (e != cudaSuccess) return e;
    PrefillParams p{};
    p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.C = static_cast<__nv_bfloat16*>(a.C);
    p.unscale = unscale;
    p.status = static_cast<unsigned int*>(scratch);
    p.inv_gs = a.inv_gs;
    p.out_mul = kBlockScaleUnfold * a.inv_gs;
    if (a.round_weights) {
        // largest weight 6 * 448 / gs -> just under 2^15 (FP16's largest binade); the smallest, 0.5 * 2^-9 / gs, then sits at 2^-7
        int ex = 0;
        std::frexp(2688.0f * a.inv_gs, &ex);                 // 2688 / gs = f * 2^ex, f in [0.5, 1)
        p.wround = 1;
        p.wshift = std::ldexp(1.0f, 15 - ex);
        p.out_mul = std::ldexp(1.0f, ex - 15);
    }
    p.swiglu_out = a.swiglu_out ? 1 : 0;
    p.out_f32 = a.out_f32 ? 1 : 0;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.m_tiles = (a.M + BM - 1) / BM;
    p.n_tiles = (a.N + BN - 1) / BN;
    p.flags = reinterpret_cast<unsigned int*>(sk);
    p.partials = reinterpret_cast<float4*>(sk + 4096);
    const int grid = plan_tiles(p, dev);
    if (p.wround) prefill_umma_kernel<false, true><<<grid, kThreads, kSmemBytes, s>>>(tma, tmp, tms, p);
    else prefill_umma_kernel<false><<<grid, kThreads, kSmemBytes, s>>>(tma, tmp, tms, p);
    if (launches) *launches = 2;
    return cudaGetLastError();
}

bool dense_umma_supported(const DenseArgs& a) {
    if (a.M < 1 || (a.K % WK) != 0 || (a.N % 8) != 0) return false;
    return (reinterpret_cast<uintptr_t>(a.W) & 15u) == 0;
}

size_t dense_umma_scratch_bytes() { return kStreamKBytes; }

// The same kernel on a BF16 weight [N,K] and the caller's BF16 activations: no pre-pass, the B
// blocks come straight from the weight by TMA.  scratch as above (status word at 0, stream-K flags
// and partial tiles from `offset`).
cudaError_t launch_dense_umma(const DenseArgs& a, nvfp4_device_info& dev, void* scratch, size_t scratch_bytes, size_t offset,
                              int* launches, cudaStream_t s) {
    if (offset + kStreamKBytes > scratch_bytes) return cudaErrorMemoryAllocation;
    char* sk = static_cast<char*>(scratch) + offset;
    CUtensorMap tma, tmw;
    if (!make_map_cached(dev.maps, &tma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.A, (uint64_t)a.K, (uint64_t)a.M, BK, BM,
                  CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tmw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.W, (uint64_t)a.K, (uint64_t)a.N, BK, BN,
                  CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    PrefillParams p{};
    p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.C = static_cast<__nv_bfloat16*>(a.C);
    p.status = static_cast<unsigned int*>(scratch);
    p.inv_gs = 1.0f;
    p.dense = 1;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.m_tiles = (a.M + BM - 1) / BM;
    p.n_tiles = (a.N + BN - 1) / BN;
    p.flags = reinterpret_cast<unsigned int*>(sk);
    p.partials = reinterpret_cast<float4*>(sk + 4096);
    const int grid = plan_tiles(p, dev);
    prefill_umma_kernel<true><<<grid, kThreads, kSmemBytes, s>>>(tma, tmw, tmw, p);
    if (launches) *launches = 1;
    return cudaGetLastError();
}

cudaError_t configure_kernels(const nvfp4_device_info&) {
    cudaError_t e = configure_decode_mma();
    if (e == cudaSuccess) e = configure_prefill_umma();
    if (e == cudaSuccess) e = configure_skinny_umma();
    if (e == cudaSuccess) e = configure_decode_wide();
    if (e == cudaSuccess) e = configure_dense_gemv();
    if (e == cudaSuccess) e = configure_decode_fp4();
    if (e == cudaSuccess) e = configure_decode_fp4_stream();
    return e;
}

}  // namespace nvfp4
