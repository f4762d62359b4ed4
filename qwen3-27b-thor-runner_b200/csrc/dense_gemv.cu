// GEMV for BF16 weights, up to 8 tokens per launch: the skeleton of the NVFP4 GEMV (decode_mma.cu)
// without the dequantisation.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W row-major BF16 (the reference's "[K,N] column
//   major" of invoke_dense_gemv / invoke_dense_gemv_add, src/engine/dense_gemm.h:64-95)
//
// In a quantised checkpoint the lm_head and the linear-attention projections stay BF16; they are
// read once per token like the FP4 weights and are bound by HBM the same way.
//   * one persistent CTA per SM: a producer lane streams 128-row x 128-k units (two TMA boxes of
//     64 k, 128-byte swizzle, no multicast; 32 KB per ring stage), row-tile-major, split evenly
//     over the CTAs (stream-K);
//   * 16 consumer warps in two groups: group h takes box h of every stage, each warp 16 rows x
//     64 k: four LDS.128 of weights (rows g and g+8, chunks 2t and 2t+1: conflict-free under the
//     swizzle), two LDS.128 of activations, four mma.sync m16n8k16 BF16 -> FP32.  The k order
//     inside an MMA is the lane's own 8 consecutive k on both operands, so no ldmatrix is needed;
//   * the activations of the CTA's k range stay resident in shared memory as they are (BF16), in
//     rows of 256 + 16 bytes per token and unit, which spreads the quarter-warps' LDS.128 over all
//     bank groups; staging is one copy and one barrier;
//   * a row tile split over several CTAs is finished by the CTA that holds its first unit: the
//     others store FP32 partials as {value, launch epoch} pairs (8-byte single transactions: the
//     pair is its own arrival flag), the owner adds them in CTA order, adds the residual, rounds
//     once.  Every wait is bounded and reports through the status word of the scratch.
#include <cuda.h>
#include <cuda_bf16.h>

#include "gemv_common.cuh"
#include "nvfp4_internal.h"
#include "ptx.cuh"
#include "umma.cuh"

namespace nvfp4 {
namespace {

using namespace gemv;

constexpr int kUK = 128;                          // k per unit
constexpr int kBoxBytes = kRT * 64 * 2;           // 16 KB: 128 rows x 64 k
constexpr int kUnitBytes = 2 * kBoxBytes;         // 32 KB per stage
constexpr int kTokRowBytes = 2 * 128 + 16;        // a token's 128 k of one unit + padding (17 bank groups)
constexpr int kDenseMaxTokens = 8;
constexpr int kDenseStages = 6;
constexpr int kDenseThreads = (2 * kGroupWarps + 1) * 32;
constexpr int kDenseConsumers = 2 * kGroupWarps * 32;
constexpr int kDenseSmem = 227 * 1024;

struct DenseParams {
    const __nv_bfloat16* A;
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    unsigned char* scratch;   // status word
    unsigned char* pairs;     // [CTA][8 tokens][128 rows] x {FP32 value, epoch}
    int M, N, K;
    int units, kchunks;       // units in all, units per row tile
    int stages;
    int act_slots, act_all;   // resident activation slots (units of 128 k); 1 = slot index is the k-chunk
    unsigned int epoch;
};

__global__ void __launch_bounds__(kDenseThreads, 1)
dense_gemv_kernel(const __grid_constant__ CUtensorMap tm_w, const DenseParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int stages = p.stages;
    unsigned char* s_w = smem;                                              // stages x 32 KB, 1024-aligned
    unsigned char* s_act = s_w + stages * kUnitBytes;                       // slots x M x 272 B
    float* s_out = reinterpret_cast<float*>(s_act + p.act_slots * p.M * kTokRowBytes);   // 2 FP32 hand-over tiles
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_out + 2 * kDenseMaxTokens * kOutLd);
    uint64_t* empty_bar = full_bar + kDenseStages;
    volatile int* s_abort = reinterpret_cast<volatile int*>(empty_bar + kDenseStages);

    unsigned int* status = reinterpret_cast<unsigned int*>(p.scratch);
    unsigned char* pairs = p.pairs;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int u_begin = (int)((long long)cta * p.units / G);
    const int u_end = (int)((long long)(cta + 1) * p.units / G);
    const int kc_begin = u_begin % p.kchunks;

    if (warp == 2 * kGroupWarps) {
        // ------------------------------------------------------------------ producer warp
        if (lane == 0) {
            for (int s = 0; s < stages; ++s) {
                ptx::mbar_init(&full_bar[s], 1);
                ptx::mbar_init(&empty_bar[s], 2 * kGroupWarps);
            }
            *s_abort = 0;
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::named_barrier_arrive(2, kDenseThreads);
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_w);
            const uint64_t pol = ptx::policy_evict_first();
            int stage = 0;
            uint32_t ph = 0;
            int tile = u_begin / p.kchunks, kc = kc_begin;
            for (int u = u_begin; u < u_end; ++u) {
                ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, 0x800u + (unsigned)stage);
                ptx::mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)kUnitBytes);
                unsigned char* dst = s_w + stage * kUnitBytes;
                ptx::tma_load_2d(dst, &tm_w, &full_bar[stage], kc * kUK, tile * kRT, pol);
                ptx::tma_load_2d(dst + kBoxBytes, &tm_w, &full_bar[stage], kc * kUK + 64, tile * kRT, pol);
                if (++kc == p.kchunks) { kc = 0; ++tile; }
                if (++stage == stages) { stage = 0; ph ^= 1u; }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int grp = warp / kGroupWarps, gw = warp % kGroupWarps;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = gw * 16 + g;                                  // tile rows r0 and r0 + 8 (both = g mod 8)
    const int off_w0 = grp * kBoxBytes + r0 * 128 + (((2 * t) ^ g) << 4);
    const int off_w1 = grp * kBoxBytes + r0 * 128 + (((2 * t + 1) ^ g) << 4);
    const int tok = g < p.M ? g : 0;                             // MMA column g; columns >= M are never stored

    ptx::griddep_launch_dependents();
    ptx::named_barrier_sync(2, kDenseThreads);                   // mbarriers initialised
    ptx::griddep_wait();                                         // activations, residual, outputs and scratch belong to earlier kernels until now

    {   // resident activations: chunk id = (slot * M + token) * 16 + c, 16 bytes = 8 consecutive k
        const int per_slot = p.M * 16;
        const int total = p.act_slots * per_slot;
        const int kc0 = p.act_all ? 0 : kc_begin;
        for (int base = tid; base < total; base += 4 * kDenseConsumers) {
            uint4 x[4];
            int dst[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int id = base + u * kDenseConsumers;
                dst[u] = -1;
                x[u] = make_uint4(0u, 0u, 0u, 0u);
                if (id < total) {
                    const int j = id / per_slot, r = id - j * per_slot;
                    const int tk = r >> 4, c = r & 15;
                    int kc = kc0 + j;
                    if (kc >= p.kchunks) kc -= p.kchunks;
                    x[u] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)tk * p.K + kc * kUK) + c);
                    dst[u] = (j * p.M + tk) * kTokRowBytes + c * 16;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (dst[u] >= 0) *reinterpret_cast<uint4*>(s_act + dst[u]) = x[u];
        }
        ptx::named_barrier_sync(1, kDenseConsumers);
    }

    int stage = 0;
    uint32_t ph = 0;
    int u = u_begin, tile = u_begin / p.kchunks, kc = kc_begin;
    int seg_parity = 0;
    while (u < u_end) {
        const int kc_first = kc;
        const int tile_end = u - kc + p.kchunks;
        const int seg_end = tile_end < u_end ? tile_end : u_end;
        const bool owner = (kc_first == 0);
        const bool complete = owner && (seg_end == tile_end);
        const int m0 = 2 * t, m1 = 2 * t + 1;
        const int rr[4] = {r0, r0, r0 + 8, r0 + 8};
        const int mm[4] = {m0, m1, m0, m1};
        int last = cta;                                          // contributors are CTAs cta+1 .. last
        if (grp == 0 && owner && !complete)
            while (last + 1 < G && (long long)(last + 1) * p.units / G < tile_end) ++last;

        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (; u < seg_end; ++u, ++kc) {
            const int slot = p.act_all ? kc : u - u_begin;
            ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0x820u + (unsigned)stage);
            const unsigned char* wp = s_w + stage * kUnitBytes;
            const unsigned char* ap = s_act + (slot * p.M + tok) * kTokRowBytes + grp * 128 + t * 32;
            const uint4 wa0 = *reinterpret_cast<const uint4*>(wp + off_w0);
            const uint4 wa1 = *reinterpret_cast<const uint4*>(wp + off_w1);
            const uint4 wb0 = *reinterpret_cast<const uint4*>(wp + off_w0 + 8 * 128);
            const uint4 wb1 = *reinterpret_cast<const uint4*>(wp + off_w1 + 8 * 128);
            const uint4 x0 = *reinterpret_cast<const uint4*>(ap);
            const uint4 x1 = *reinterpret_cast<const uint4*>(ap + 16);
            // per MMA: rows g / g+8, the lane's k pairs (0,1) and (2,3) resp. (4,5) and (6,7) of one chunk
            const uint32_t a0[4] = {wa0.x, wb0.x, wa0.y, wb0.y}, a1[4] = {wa0.z, wb0.z, wa0.w, wb0.w};
            const uint32_t a2[4] = {wa1.x, wb1.x, wa1.y, wb1.y}, a3[4] = {wa1.z, wb1.z, wa1.w, wb1.w};
            ptx::mma_bf16_16x8x16(acc, a0, x0.x, x0.y);
            ptx::mma_bf16_16x8x16(acc2, a1, x0.z, x0.w);
            ptx::mma_bf16_16x8x16(acc, a2, x1.x, x1.y);
            ptx::mma_bf16_16x8x16(acc2, a3, x1.z, x1.w);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[stage]);
            if (++stage == stages) { stage = 0; ph ^= 1u; }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += acc2[i];

        // ------------------------------------------------------------ segment epilogue
        // Warp gw of group 1 hands its sums to warp gw of group 0 through shared memory (two tiles
        // alternating per segment, one 64-thread barrier); group 0 finishes the 16 rows.
        float* xchg = s_out + (seg_parity ? kDenseMaxTokens * kOutLd : 0);
        seg_parity ^= 1;
        if (grp == 1) {
            xchg[m0 * kOutLd + r0] = acc[0];
            xchg[m1 * kOutLd + r0] = acc[1];
            xchg[m0 * kOutLd + r0 + 8] = acc[2];
            xchg[m1 * kOutLd + r0 + 8] = acc[3];
        }
        ptx::named_barrier_sync(4 + gw, 64);
        if (grp == 0) {
            float v[4] = {acc[0] + xchg[m0 * kOutLd + r0], acc[1] + xchg[m1 * kOutLd + r0],
                          acc[2] + xchg[m0 * kOutLd + r0 + 8], acc[3] + xchg[m1 * kOutLd + r0 + 8]};
            if (!owner) {
                unsigned char* slot = pairs + (size_t)cta * (kDenseMaxTokens * kRT) * 8;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (mm[i] < p.M) ptx::st_volatile_v2(slot + (mm[i] * kRT + rr[i]) * 8, __float_as_uint(v[i]), p.epoch);
            } else {
                // contributors in CTA order (a fixed summation order), two at a time: their eight
                // loads are issued before any is looked at; the wait for an old epoch is bounded
                const long long t0 = clock64();
                bool failed = false;
                for (int c0 = cta + 1; c0 <= last && !failed; c0 += 2) {
                    const bool two = c0 + 1 <= last;
                    const unsigned char* src = pairs + (size_t)c0 * (kDenseMaxTokens * kRT) * 8;
                    while (true) {
                        uint2 x[2][4];
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                x[j][i] = make_uint2(0u, p.epoch);
                                if (mm[i] < p.M && (j == 0 || two))
                                    x[j][i] = ptx::ld_volatile_v2(src + ((size_t)j * (kDenseMaxTokens * kRT) + mm[i] * kRT + rr[i]) * 8);
                            }
                        bool ready = true;
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) ready &= (x[j][i].y == p.epoch);
                        if (ready) {
#pragma unroll
                            for (int j = 0; j < 2; ++j)
#pragma unroll
                                for (int i = 0; i < 4; ++i) v[i] += __uint_as_float(x[j][i].x);
                            break;
                        }
                        if (*s_abort || clock64() - t0 > ptx::kWaitBudgetClocks) {
                            *s_abort = 1;
                            atomicCAS(status, 0u, 0x830u);
                            failed = true;
                            break;
                        }
                    }
                }
                // hand the slots back cleared: a replayed launch carries the same tag (decode_mma.cu explains)
                if (!failed)
                    for (int c = cta + 1; c <= last; ++c) {
                        unsigned char* src = pairs + (size_t)c * (kDenseMaxTokens * kRT) * 8;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (mm[i] < p.M) ptx::st_volatile_v2(src + ((size_t)mm[i] * kRT + rr[i]) * 8, 0u, 0u);
                    }
                __syncwarp();
                const int row_base = tile * kRT;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = row_base + rr[i];
                    if (mm[i] >= p.M || n >= p.N) continue;
                    const size_t o = (size_t)mm[i] * p.N + n;
                    float x = v[i];
                    if (p.residual) x += __bfloat162float(p.residual[o]);
                    p.C[o] = __float2bfloat16_rn(x);
                }
            }
        }
        if (kc >= p.kchunks) { kc = 0; ++tile; }
    }
}

struct DensePlan {
    DenseParams p;
    int grid, smem;
};

bool plan_dense(const DenseArgs& a, int m, const nvfp4_device_info& dev, void* scratch, DensePlan* out) {
    DenseParams p{};
    p.A = static_cast<const __nv_bfloat16*>(a.A);
    p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.C = static_cast<__nv_bfloat16*>(a.C);
    p.scratch = static_cast<unsigned char*>(scratch);
    p.pairs = p.scratch + dev.gemv_pairs_offset;
    p.M = m; p.N = a.N; p.K = a.K;
    p.kchunks = a.K / kUK;
    const long long units = (long long)((a.N + kRT - 1) / kRT) * p.kchunks;
    if (units > 0x7fffffffLL) return false;
    p.units = (int)units;
    int grid = dev.sm_count < kMaxGrid ? dev.sm_count : kMaxGrid;
    if (grid > p.units) grid = p.units;
    const int max_span = (p.units + grid - 1) / grid;
    p.act_all = p.kchunks <= max_span ? 1 : 0;
    p.act_slots = p.act_all ? p.kchunks : max_span;
    const long long act = (long long)p.act_slots * m * kTokRowBytes;
    const int fixed = 1024 + 2 * kDenseMaxTokens * kOutLd * 4 + 2 * kDenseStages * 8 + 64;
    long long stages = (kDenseSmem - fixed - act) / kUnitBytes;
    if (stages < 3) return false;
    if (stages > kDenseStages) stages = kDenseStages;
    p.stages = (int)stages;
    out->p = p;
    out->grid = grid;
    out->smem = fixed + (int)stages * kUnitBytes + (int)act;
    return true;
}

int dense_tokens_per_launch(const DenseArgs& a, const nvfp4_device_info& dev) {
    DensePlan pl;
    for (int m = a.M < kDenseMaxTokens ? a.M : kDenseMaxTokens; m >= 1; --m)
        if (plan_dense(a, m, dev, nullptr, &pl)) return m;
    return 0;
}

}  // namespace

bool dense_gemv_supported(const DenseArgs& a, const nvfp4_device_info& dev) {
    if (a.M < 1 || a.M > 16 || (a.K % kUK) != 0 || a.N < 1) return false;
    if (reinterpret_cast<uintptr_t>(a.W) & 15u) return false;
    return dense_tokens_per_launch(a, dev) > 0;
}

cudaError_t configure_dense_gemv() {
    return configure_large_smem(dense_gemv_kernel, kDenseSmem);
}

// scratch: the handle workspace (status word at 0, pairs at dev.gemv_pairs_offset, shared with the
// NVFP4 GEMV: launches on one stream follow each other, and every launch has its own epoch).
cudaError_t launch_dense_gemv(const DenseArgs& a, nvfp4_device_info& dev, void* scratch, int* launches, cudaStream_t s) {
    CUtensorMap tm;
    if (!umma::make_map_cached(dev.maps, &tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.W, (uint64_t)a.K, (uint64_t)a.N, 64, kRT,
                        CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    const int per = dense_tokens_per_launch(a, dev);
    if (per <= 0) return cudaErrorInvalidValue;
    int n = 0;
    for (int m0 = 0; m0 < a.M; m0 += per) {      // more than `per` tokens: one launch per group (each streams the weights again)
        DenseArgs b = a;
        const int m = a.M - m0 < per ? a.M - m0 : per;
        b.A = static_cast<const char*>(a.A) + (size_t)m0 * a.K * 2;
        b.C = static_cast<char*>(a.C) + (size_t)m0 * a.N * 2;
        if (a.residual) b.residual = static_cast<const char*>(a.residual) + (size_t)m0 * a.N * 2;
        DensePlan pl;
        if (!plan_dense(b, m, dev, scratch, &pl)) return cudaErrorInvalidValue;
        pl.p.epoch = next_launch_tag();
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(pl.grid);
        cfg.blockDim = dim3(kDenseThreads);
        cfg.dynamicSmemBytes = pl.smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, dense_gemv_kernel, tm, pl.p);
        ++n;
        if (e != cudaSuccess) { if (launches) *launches = n; return e; }
    }
    if (launches) *launches = n;
    return cudaSuccess;
}

}  // namespace nvfp4
