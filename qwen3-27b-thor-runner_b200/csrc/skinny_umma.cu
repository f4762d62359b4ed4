// Linear layer for a few dozen tokens (1 <= M <= 128 supported, routed here for 17..64 by
// default): the dequantised weights are the A operand of tcgen05.mma and live in tensor memory,
// the activations are the B operand.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W = e2m1(code) * ue4m3(scale) / global_scale
//
// With few tokens the layer is bound by streaming the packed weights from HBM, so the kernel is
// built around that stream: the weight tile (128 rows) is the M side of the MMA, the tokens
// (padded to a multiple of 16) are the N side, and the dequantised FP16 weights never touch
// shared memory:
//   warp 0      TMA producer of raw weight stages: 128 rows x 256 k of packed codes (16 KB) and
//               their block scales (2 KB) into a ring of up to 8 stages.  Plain tiled TMA.
//   warp 2      TMA producer of activation stages: tokens x 256 k of the FP16 activation copy (made
//               by a small pre-pass kernel with an exact per-token power-of-two scale) as four
//               128-byte-swizzled K-major blocks.  Starts once that pre-pass has finished
//               (programmatic dependent launch); the weight stream above does not wait for it.
//   warps 8-15  dequantise: thread = weight row = TMEM lane.  cvt.rn.f16x2.e2m1x2 + one f16x2
//               multiply by the block scale (every product is exact in FP16), then tcgen05.st of
//               the FP16 row segment into a ring of 64-column (128-k) A units in tensor memory;
//               warps 8-11 fill the even units, warps 12-15 the odd ones, one lane quarter each.
//   warp 1      one elected thread issues tcgen05.mma kind::f16 (A = FP16 in TMEM, B = FP16
//               shared-memory descriptor, D = FP32 in TMEM, M = 128, N = tokens, K = 16) and
//               commits completion to the mbarriers that recycle the buffers.
//   warps 4-7   epilogue: tcgen05.ld of the FP32 accumulator (lane = weight row, column = token),
//               per-token unscale, 1/global_scale and the residual in FP32, one rounding to BF16.
// The (row tile, 256-k stage) units are spread evenly over one persistent CTA per SM (stream-K);
// a row tile shared by several CTAs is summed from FP32 partial tiles in CTA order, each CTA
// reducing its own slice, so the result does not depend on timing.
//
// Arithmetic is the reference's small-M kernel (src/engine/dense_gemm_fp4_sm110.cu:96-233):
// exact dequantised weights, BF16 activations, FP32 accumulation, one multiplication by
// 1/global_scale, residual added in FP32 before the only rounding.
//
// Measured on B200 (gate_up 34816 x 5120): 43-50 us for 1..64 tokens, flat in M.  The issuing
// thread sustains one tcgen05.mma with a TMEM A operand (128 x N x 16) per ~137 clocks whatever N
// is, i.e. ~1.1 us per 128-row x 256-k stage, so the kernel streams weights at ~2.3 TB/s: slower
// than the register-fed mma.sync GEMV for M <= 8 (26-30 us), faster than two GEMV launches or
// the 128-token-tile GEMM between them.  kind::f16 takes both operands in ONE 16-bit format:
// an instruction descriptor with A = FP16 and B = BF16 raises an illegal-instruction fault,
// hence the FP16 activation copy.
//
// Every mbarrier wait is bounded; a wait that runs out records its code in the handle's status
// word and the kernel winds down (TMEM is always freed).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "ptx.cuh"
#include "umma.cuh"

namespace nvfp4 {
namespace {

using namespace umma;

constexpr int TR = 128;            // weight rows per tile (UMMA M = TMEM lanes)
constexpr int BK = 64;             // k per activation operand block (128 bytes of BF16)
constexpr int WK = 256;            // k per stage
constexpr int kMaxTokens = 128;    // UMMA N <= 128 here: two accumulators + the A ring = 512 TMEM columns
constexpr int kWPackedBytes = TR * WK / 2;     // 16 KB
constexpr int kWScaleBytes = TR * WK / 16;     // 2 KB
constexpr int kMaxWStages = 8, kMaxXStages = 4, kMaxAUnits = 6, kAccs = 2;
constexpr int kThreads = 512;
constexpr int kDequantWarps = 8, kEpiWarps = 4;
constexpr int kAUnitK = 128;       // k per A unit in tensor memory: half a stage, filled by four warps
constexpr int kAUnitCols = kAUnitK / 2;   // 64 columns of FP16 pairs per lane
constexpr int kSmemBudget = 200 * 1024;
constexpr size_t kSlotFloats = (size_t)kMaxTokens * TR;   // one FP32 partial tile: [token][row]

struct SkinnyParams {
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    const float* unscale;      // per token: 1 / activation scale
    unsigned int* status;
    float inv_gs;
    int M, N, K;
    int NT;                    // UMMA N: tokens rounded up to a multiple of 16
    int row_tiles, sk_tiles;   // tiles [0, sk_tiles) are split by k over all CTAs
    int w_stages, x_stages;
    int acc_cols;              // TMEM columns per accumulator (two accumulators from column 0)
    int a_units, a_col0;       // ring of A units (64 columns each) behind the accumulators
    uint32_t idesc;
    float* partials;           // [grid][2][kMaxTokens][128] FP32
    unsigned int* flags;       // [grid][2], the launch's tag once that partial tile is stored
};

__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One token of one weight row: scale, residual, round, store.
__device__ __forceinline__ void store_output(const SkinnyParams& p, int m, int n, float v) {
    const size_t o = (size_t)m * p.N + n;
    float f = v * (p.unscale[m] * kBlockScaleUnfold * p.inv_gs);
    if (p.residual) f += __bfloat162float(p.residual[o]);
    p.C[o] = __float2bfloat16_rn(f);
}

// Reduction of one split row tile (see reduce_split_tile of the prefill kernel: same protocol).
// The P participants each take 1/P of the tokens; with fewer tokens than participants the
// rows are split instead.  t = 0..nthreads-1, nthreads a multiple of 128.
__device__ __forceinline__ void reduce_split_rows(const SkinnyParams& p, unsigned int epoch, int tile, int kstages, int t,
                                                  int nthreads, volatile int* s_abort) {
    int first, last;
    split_tile_participants(p.sk_tiles, kstages, tile, first, last);
    if (!wait_split_tile_flags(p.flags, epoch, first, last, t, s_abort, p.status)) return;
    const int P = last - first + 1, me = blockIdx.x - first;
    const int total = p.M * TR;                      // elements [token][row] of the tile that matter
    const int e0 = (int)((long long)me * total / P), e1 = (int)((long long)(me + 1) * total / P);
    const float* head = p.partials + ((size_t)first * 2 + 1) * kSlotFloats;
    for (int e = e0 + t; e < e1; e += nthreads) {
        float s = __ldcg(head + e);
        for (int c = first + 1; c <= last; c += 8) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)          // eight loads in flight; absent participants add zero
                x[i] = c + i <= last ? __ldcg(p.partials + (size_t)(c + i) * 2 * kSlotFloats + e) : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s += x[i];
        }
        const int m = e / TR, n = tile * TR + (e % TR);
        if (n < p.N) store_output(p, m, n, s);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
skinny_umma_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_packed,
                   const __grid_constant__ CUtensorMap tm_scale, const SkinnyParams p) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment by an offset on the shared-memory array itself: the pointer keeps its
    // address space, so every access below is a shared-memory instruction with a 32-bit address
    // (rounding a generic 64-bit pointer instead turns them into generic loads and stores).
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int xbytes = p.NT * (WK * 2);                               // one activation stage: 4 blocks of NT x 128 B
    unsigned char* s_x = smem;                                        // x_stages x xbytes
    unsigned char* s_wp = s_x + p.x_stages * xbytes;                  // w_stages x 16 KB packed codes
    unsigned char* s_ws = s_wp + p.w_stages * kWPackedBytes;          // w_stages x 2 KB scales
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_ws + p.w_stages * kWScaleBytes);
    uint64_t* wfull = bars;                        // [kMaxWStages]
    uint64_t* wempty = wfull + kMaxWStages;        // [kMaxWStages]
    uint64_t* xfull = wempty + kMaxWStages;        // [kMaxXStages]
    uint64_t* xempty = xfull + kMaxXStages;        // [kMaxXStages]
    uint64_t* afull = xempty + kMaxXStages;        // [kMaxAUnits]
    uint64_t* aempty = afull + kMaxAUnits;         // [kMaxAUnits]
    uint64_t* tfull = aempty + kMaxAUnits;         // [kAccs]
    uint64_t* tempty = tfull + kAccs;              // [kAccs]
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tempty + kAccs);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    volatile unsigned int* s_epoch = reinterpret_cast<volatile unsigned int*>(s_tmem + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kstages = p.K / WK;
    const bool all_reduce = p.sk_tiles == p.row_tiles;

    if (tid == 0) {
        for (int i = 0; i < kMaxWStages; ++i) { ptx::mbar_init(&wfull[i], 1); ptx::mbar_init(&wempty[i], kDequantWarps); }
        for (int i = 0; i < kMaxXStages; ++i) { ptx::mbar_init(&xfull[i], 1); ptx::mbar_init(&xempty[i], 1); }
        for (int i = 0; i < kMaxAUnits; ++i) { ptx::mbar_init(&afull[i], kDequantWarps / 2); ptx::mbar_init(&aempty[i], 1); }
        for (int i = 0; i < kAccs; ++i) { ptx::mbar_init(&tfull[i], 1); ptx::mbar_init(&tempty[i], kEpiWarps); }
        *s_abort = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) tmem_alloc_512(s_tmem);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    ptx::griddep_launch_dependents();      // the next kernel in the stream may start its own prologue

    if (warp == 0) {
        // ------------------------------------------------------------------ weight stream
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
            const uint64_t pol = ptx::policy_evict_first();
            int sw = 0;
            uint32_t pw = 0;
            Schedule sched(p.sk_tiles, p.row_tiles, kstages);
            Segment sg;
            while (sched.next(sg)) {
                for (int ks = sg.ks0; ks < sg.ks1; ++ks) {
                    ptx::mbar_wait(&wempty[sw], pw ^ 1u, s_abort, p.status, 0x510u + sw);
                    ptx::mbar_arrive_expect_tx(&wfull[sw], kWPackedBytes + kWScaleBytes);
                    ptx::tma_load_2d(s_wp + sw * kWPackedBytes, &tm_packed, &wfull[sw], ks * (WK / 2), sg.tile * TR, pol);
                    ptx::tma_load_2d(s_ws + sw * kWScaleBytes, &tm_scale, &wfull[sw], ks * (WK / 16), sg.tile * TR, pol);
                    if (++sw == p.w_stages) { sw = 0; pw ^= 1u; }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ activation stream
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_act);
            ptx::griddep_wait();           // the activations are the preceding kernel's output
            const uint64_t pol = ptx::policy_evict_last();
            int sx = 0;
            uint32_t px = 0;
            Schedule sched(p.sk_tiles, p.row_tiles, kstages);
            Segment sg;
            while (sched.next(sg)) {
                for (int ks = sg.ks0; ks < sg.ks1; ++ks) {
                    ptx::mbar_wait(&xempty[sx], px ^ 1u, s_abort, p.status, 0x500u + sx);
                    ptx::mbar_arrive_expect_tx(&xfull[sx], (uint32_t)xbytes);
#pragma unroll
                    for (int j = 0; j < WK / BK; ++j)
                        ptx::tma_load_2d(s_x + sx * xbytes + j * (p.NT * 128), &tm_act, &xfull[sx], ks * WK + j * BK, 0, pol);
                    if (++sx == p.x_stages) { sx = 0; px ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int sx = 0, au = 0, acc = 0;
            uint32_t px = 0, pa = 0, pt = 0;
            Schedule sched(p.sk_tiles, p.row_tiles, kstages);
            Segment sg;
            while (sched.next(sg)) {
                ptx::mbar_wait(&tempty[acc], pt ^ 1u, s_abort, p.status, 0x540u + acc);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.acc_cols);
                for (int ks = sg.ks0; ks < sg.ks1; ++ks) {
                    ptx::mbar_wait(&xfull[sx], px, s_abort, p.status, 0x520u + sx);
                    const uint64_t xdesc = umma_desc_sw128(ptx::smem_u32(s_x + sx * xbytes));
#pragma unroll
                    for (int h = 0; h < WK / kAUnitK; ++h) {
                        ptx::mbar_wait(&afull[au], pa, s_abort, p.status, 0x530u + au);
                        tc_fence_after();
                        const uint32_t a_tmem = tmem_base + (uint32_t)(p.a_col0 + au * kAUnitCols);
#pragma unroll
                        for (int k = 0; k < kAUnitK / 16; ++k) {
                            const int kk = h * (kAUnitK / 16) + k;      // 16-k step inside the stage
                            // 64-k block kk/4 of the stage (NT x 128 B each), 32 bytes per step inside it
                            const uint64_t bdesc = xdesc + (uint64_t)(((kk >> 2) * (p.NT * 128) + (kk & 3) * 32) >> 4);
                            umma_f16_ts(d_tmem, a_tmem + k * 8, bdesc, p.idesc, (ks > sg.ks0 || kk > 0) ? 1u : 0u);
                        }
                        umma_commit(&aempty[au]);  // the A unit is free once these MMAs have read it
                        if (++au == p.a_units) { au = 0; pa ^= 1u; }
                    }
                    umma_commit(&xempty[sx]);
                    if (++sx == p.x_stages) { sx = 0; px ^= 1u; }
                }
                umma_commit(&tfull[acc]);
                if (++acc == kAccs) { acc = 0; pt ^= 1u; }
            }
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ dequantise into TMEM
        const int dw = warp - 8;
        const int quarter = dw & 3;                       // TMEM lanes 32*quarter .. +31 (= warp id % 4)
        const int half = dw >> 2;                         // k 128*half .. +127 of the stage = A unit 2*stage + half
        const int row = quarter * 32 + lane;
        const int sw7 = row & 7;
        int sw = 0, au = half;                            // this warp fills every other unit of the ring (a_units is even)
        uint32_t pw = 0, pa = 0;
        Schedule sched(p.sk_tiles, p.row_tiles, kstages);
        Segment sg;
        while (sched.next(sg)) {
            for (int ks = sg.ks0; ks < sg.ks1; ++ks) {
                ptx::mbar_wait(&wfull[sw], pw, s_abort, p.status, 0x550u + sw);
                const unsigned char* wp = s_wp + sw * kWPackedBytes + row * 128;
                uint4 q[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) q[c] = *reinterpret_cast<const uint4*>(wp + (((4 * half + c) ^ sw7) << 4));
                const uint2 sc = *reinterpret_cast<const uint2*>(s_ws + sw * kWScaleBytes + row * 16 + 8 * half);
                ptx::mbar_wait(&aempty[au], pa ^ 1u, s_abort, p.status, 0x560u + au);
                tc_fence_after();
                const uint32_t a_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(p.a_col0 + au * kAUnitCols);
#pragma unroll
                for (int c = 0; c < 4; ++c) {              // chunk c: 32 k = two block scales = 16 columns
                    const uint32_t w[4] = {q[c].x, q[c].y, q[c].z, q[c].w};
                    const uint32_t scw = mask_scale_bytes(c < 2 ? sc.x : sc.y);
                    const uint32_t S0 = scale_byte_to_f16x2(scw, 2 * (c & 1));          // scale / 2^8, undone in the epilogue
                    const uint32_t S1 = scale_byte_to_f16x2(scw, 2 * (c & 1) + 1);
                    uint32_t r[16];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t e[4];
                        ptx::cvt_e2m1x8_to_f16x2(w[i], e);
                        const uint32_t S = i < 2 ? S0 : S1;
#pragma unroll
                        for (int j = 0; j < 4; ++j) r[4 * i + j] = ptx::mul_f16x2(e[j], S);
                    }
                    tmem_st16(a_addr + c * 16, r);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&afull[au]);
                    ptx::mbar_arrive(&wempty[sw]);
                }
                if (++sw == p.w_stages) { sw = 0; pw ^= 1u; }
                au += 2;
                if (au >= p.a_units) { au -= p.a_units; pa ^= 1u; }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue: thread = weight row
        const int ew = warp - 4;                          // TMEM lanes 32*ew .. +31 (= warp id % 4)
        const int te = ew * 32 + lane;
        int acc = 0;
        uint32_t pt = 0;
        int pend[2] = {-1, -1};
        ptx::griddep_wait();                              // C, the residual and the scratch belong to earlier kernels until now
        // the tag of this launch's split-tile flags, from the counter in the scratch; the four epilogue warps share it
        if (te == 0) *s_epoch = ptx::take_launch_epoch(p.status);
        ptx::named_barrier_sync(1, kEpiWarps * 32);
        const unsigned int epoch = *s_epoch;
        Schedule sched(p.sk_tiles, p.row_tiles, kstages);
        Segment sg;
        bool more = sched.next(sg);
        while (more) {
            const int n = sg.tile * TR + te;
            const bool complete = sg.ks0 == 0 && sg.ks1 == kstages;
            ptx::mbar_wait(&tfull[acc], pt, s_abort, p.status, 0x570u + acc);
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)(acc * p.acc_cols);
            const int which = sg.ks0 == 0 ? 1 : 0;        // head of a tile (span end) or tail (span start)
            float* slot = p.partials + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;
            for (int c0 = 0; c0 < p.NT; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(t_addr + c0, r);
                if (complete) {
                    if (n < p.N) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c0 + i < p.M) store_output(p, c0 + i, n, __uint_as_float(r[i]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)           // [token][row]: a warp stores 128 contiguous bytes
                        if (c0 + i < p.M) __stcg(slot + (c0 + i) * TR + te, __uint_as_float(r[i]));
                }
            }
            if (!complete) {
                __threadfence();
                ptx::named_barrier_sync(1, kEpiWarps * 32);   // all 128 rows stored before the flag goes up
                if (te == 0) ptx::st_release_gpu(&p.flags[blockIdx.x * 2 + which], epoch);
                pend[which] = sg.tile;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tempty[acc]);
            if (++acc == kAccs) { acc = 0; pt ^= 1u; }
            more = sched.next(sg);
            // Whole tiles follow the stream-K region: these four warps reduce the split tiles now,
            // behind the MMAs of the next tiles.  (With no whole tiles all warps do it at the end.)
            if (!all_reduce && (pend[0] >= 0 || pend[1] >= 0) && (!more || sg.tile >= p.sk_tiles)) {
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    if (pend[w] >= 0) reduce_split_rows(p, epoch, pend[w], kstages, te, kEpiWarps * 32, s_abort);
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
        ptx::griddep_wait();
        const unsigned int epoch = *s_epoch;           // written by the epilogue warps before the barrier above
        int split[2];
        split_tiles_of_cta(p.sk_tiles, kstages, split);
#pragma unroll
        for (int w = 0; w < 2; ++w)
            if (split[w] >= 0) reduce_split_rows(p, epoch, split[w], kstages, tid, kThreads, s_abort);
    }
}

struct SkinnyPlan {
    SkinnyParams p;
    int grid;
    int smem;
};

bool plan_skinny(const LinearArgs& a, const nvfp4_device_info& dev, SkinnyPlan* out) {
    SkinnyParams& p = out->p;
    p = SkinnyParams{};
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.NT = (a.M + 15) / 16 * 16;
    p.row_tiles = (a.N + TR - 1) / TR;
    const int kstages = a.K / WK;
    const int xbytes = p.NT * WK * 2;
    p.x_stages = p.NT <= 32 ? 4 : (p.NT <= 64 ? 3 : 2);
    int ws = (kSmemBudget - p.x_stages * xbytes) / (kWPackedBytes + kWScaleBytes);
    if (ws > kMaxWStages) ws = kMaxWStages;
    if (ws < 2) return false;
    p.w_stages = ws;
    out->smem = 1024 + p.x_stages * xbytes + ws * (kWPackedBytes + kWScaleBytes) + 512;
    // Tensor memory (512 columns): two accumulators, then as many 64-column A units as fit (even count).
    p.acc_cols = p.NT <= 64 ? 64 : 128;
    p.a_units = p.NT <= 64 ? 6 : 4;
    p.a_col0 = 512 - p.a_units * kAUnitCols;
    // kind::f16: D = FP32, A = B = FP16, both K-major, M = 128, N = NT
    p.idesc = (1u << 4) | ((uint32_t)(p.NT >> 3) << 17) | ((uint32_t)(TR >> 4) << 24);
    int grid = dev.sm_count < 160 ? dev.sm_count : 160;
    if ((long long)p.row_tiles * kstages < grid) grid = p.row_tiles * kstages;
    // Whole waves of row tiles run tile by tile; the rest is split by k over all CTAs when that is
    // shorter than one more wave of whole tiles (the split costs about `skinny_split_cost` stages).
    p.sk_tiles = 0;
    const int left = p.row_tiles % grid;
    if (left > 0) {
        int sk = left;
        if (sk * kstages < grid) sk += p.row_tiles >= grid ? grid : 0;
        const long long whole = (long long)((p.row_tiles + grid - 1) / grid) * kstages;
        const long long split = (long long)((p.row_tiles - sk) / grid) * kstages + ((long long)sk * kstages + grid - 1) / grid +
                                dev.skinny_split_cost;
        if (split < whole && (long long)sk * kstages >= grid) p.sk_tiles = sk;
    }
    out->grid = grid;
    return true;
}

}  // namespace

bool skinny_umma_supported(const LinearArgs& a) {
    if (a.M < 1 || a.M > kMaxTokens || (a.K % WK) != 0 || a.N < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u) ||
        (reinterpret_cast<uintptr_t>(a.A) & 15u))
        return false;
    return true;
}

cudaError_t configure_skinny_umma() {
    return configure_large_smem(skinny_umma_kernel, 1024 + kSmemBudget + 1536);
}

// scratch: [0, 256) status word; from `offset` the same layout as the prefill kernel's scratch
// (flags, partial tiles, FP16 activations, per-token factors): a handle serves one stream at a
// time, so the two kernels never use it at the same time.
cudaError_t launch_skinny_umma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, size_t scratch_bytes,
                               size_t offset, int* launches, cudaStream_t s) {
    SkinnyPlan pl;
    if (!plan_skinny(a, dev, &pl)) return cudaErrorInvalidValue;
    if (offset + prefill_umma_scratch_bytes(a.M > 16 ? a.M : 17, a.N, a.K) > scratch_bytes) return cudaErrorMemoryAllocation;
    char* sk = static_cast<char*>(scratch) + offset;
    char* base = sk + prefill_umma_reserved_bytes();              // FP16 activations, then one FP32 per token
    float* unscale = reinterpret_cast<float*>(base + ((size_t)a.M * a.K * 2 + 255) / 256 * 256);
    CUtensorMap tma, tmp, tms;
    if (!make_map_cached(dev.maps, &tma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, (uint64_t)a.K, (uint64_t)a.M, BK, pl.p.NT,
                  CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, TR,
                  CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_cached(dev.maps, &tms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, TR,
                  CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    cudaError_t e = launch_act_to_f16(a.A, a.M, a.K, base, unscale, s);
    if (e != cudaSuccess) return e;
    pl.p.unscale = unscale;
    pl.p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    pl.p.C = static_cast<__nv_bfloat16*>(a.C);
    pl.p.status = static_cast<unsigned int*>(scratch);
    pl.p.inv_gs = a.inv_gs;
    pl.p.flags = reinterpret_cast<unsigned int*>(sk);
    pl.p.partials = reinterpret_cast<float*>(sk + 4096);
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
    e = cudaLaunchKernelEx(&cfg, skinny_umma_kernel, tma, tmp, tms, pl.p);
    if (launches) *launches = 2;
    return e;
}

}  // namespace nvfp4
