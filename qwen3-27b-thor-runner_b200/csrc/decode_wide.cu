// Dequant-GEMV for 9..16 tokens in one launch: the GEMV kernel's consumer math (decode_mma.cu) with
// a second 8-token MMA tile per weight fragment and the activations streamed through the ring.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W = e2m1(code) * ue4m3(scale) / global_scale
//
// Why a second kernel: the conversion of the packed codes is what the GEMV kernel's consumer warps
// spend their time on, and it does not depend on the number of tokens, so 16 tokens cost little
// more than 8 if they share it -- but the FP16 activations of 16 tokens no longer fit resident in
// shared memory next to the ring (160 KB for K = 5120).  Here they travel with the weights:
//   * a pre-pass (act_f16.cu) writes the FP16 copy of the activations, scaled per token by an
//     exact power of two, into the handle workspace;
//   * the work unit is 256 weight rows x 256 k (32 KB of codes + 4 KB of scales), one per ring
//     stage; the units, row-pair-major, are split evenly over the CTAs (stream-K);
//   * warp 16 streams the units with plain tiled TMA (no multicast); warp 17 copies the unit's
//     activations (16 token rows x 256 k) with 16-byte cp.async into the padded row layout of the
//     GEMV kernel (four 64-k blocks of 128 + 16 bytes per token: the consumers' LDS.128 then use
//     immediate offsets and hit all bank groups; the 128-byte TMA swizzle would give 4-way
//     conflicts with this thread-to-k mapping), once the pre-pass has finished (programmatic
//     dependent launch: the weight stream does not wait for it);
//   * each of the 16 consumer warps owns 16 of the unit's 256 rows over the whole k range of its
//     CTA: codes expanded in registers exactly as in the GEMV kernel, then mma.sync m16n8k16
//     against the two token tiles (tokens 0..7 and 8..15), FP32 accumulators.  All warps read the
//     same 9 KB of activations, so a stage is 45 KB and five of them fit;
//   * a row pair whose k range is split over several CTAs is finished warp by warp, without any
//     CTA-wide step: contributors store their FP32 partials as 8-byte {value, launch epoch} pairs
//     (one transaction each: the pair is its own arrival flag), the CTA that holds the row pair's
//     first unit adds them in CTA order, applies 2^8 / global_scale and the residual in FP32 and
//     rounds once.  The tag comes from a counter in the scratch (ptx.cuh: take_launch_epoch), not from
//     the host, so a captured launch can be replayed.  (Clearing the pairs after use, as the 8-token
//     kernel does, doubles this kernel's pair traffic: 16 tokens x 256 rows per contributor; measured
//     +3.9 us on the down projection, against -0.3..-1.0 us for the counter.)  Every wait is bounded
//     and reports through the status word.
// Options shared with the 8-token kernel: the SwiGLU epilogue on row-interleaved gate/up weights and
// the sum over a tensor-parallel group inside the kernel ({value, epoch} pairs pushed to every
// rank's exchange buffer, reduced in rank order once the CTA has no weight left to stream).
// Arithmetic: the reference's small-M kernel (src/engine/dense_gemm_fp4_sm110.cu:155-258) up to
// FP32 summation order.
#include <cuda.h>
#include <cuda_bf16.h>

#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "gemv_common.cuh"
#include "exchange_layout.h"
#include "ptx.cuh"
#include "umma.cuh"

namespace nvfp4 {
namespace {

using namespace gemv;

constexpr int kUnitRows = 2 * kRT;                // 256 weight rows per unit
constexpr int kConsumerWarps = kUnitRows / 16;    // 16: one 16-row slab each
constexpr int kThreads = kConsumerWarps * 32 + 64;   // + weight producer warp + activation producer warp
constexpr int kTT = 2;                            // 8-token MMA tiles per launch
constexpr int kTokens = 8 * kTT;
constexpr int kUnitPackedBytes = kUnitRows * kKC / 2;     // 32 KB
constexpr int kUnitScaleBytes = kUnitRows * kKC / 16;     // 4 KB
constexpr int kActBytes = kTokens * kActRowBytes;         // 9 KB
constexpr int kStageBytes = kUnitPackedBytes + kUnitScaleBytes + kActBytes;   // 45 KB
constexpr int kMaxStages = 5;
constexpr int kSmemBudget = 227 * 1024;
constexpr int kWideMaxGrid = 160;                 // CTAs whose partial slabs fit in front of the 8-token kernel's pairs
static_assert(kPartialOffset + (size_t)kWideMaxGrid * kTokens * kUnitRows * 8 <= kPairOffset, "scratch layout");

struct WideParams {
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    const float* unscale;      // per token: 1 / activation scale
    const unsigned short* act; // [M, K] FP16 copy of the activations
    unsigned char* scratch;
    float inv_gs;
    int M, N, K;
    int units, kchunks;
    int stages;
    // Tensor-parallel K split: world > 0 = push the sums to the ranks' exchange buffers and reduce over
    // the group at the end of this kernel, exactly as the 8-token kernel does (decode_mma.cu).
    unsigned char* xpeer[xchg::kMaxWorld];
    int xrank, xworld, xslot_pairs;
    int swiglu_out;            // rows interleaved in slabs of 16 (8 gate rows, their 8 up rows): C is [M, N/2] = bf16(silu(gate) * up)
};

__global__ void __launch_bounds__(kThreads, 1)
decode_wide_kernel(const __grid_constant__ CUtensorMap tm_packed, const __grid_constant__ CUtensorMap tm_scale,
                   const WideParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int stages = p.stages;
    unsigned char* s_packed = smem;                                   // stages x 32 KB, 1024-aligned
    unsigned char* s_act = s_packed + stages * kUnitPackedBytes;      // stages x 9 KB
    unsigned char* s_scale = s_act + stages * kActBytes;              // stages x 4 KB
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_scale + stages * kUnitScaleBytes);
    uint64_t* empty_bar = full_bar + kMaxStages;
    volatile int* s_abort = reinterpret_cast<volatile int*>(empty_bar + kMaxStages);
    volatile unsigned int* s_epoch = reinterpret_cast<volatile unsigned int*>(s_abort) + 1;   // 0 until consumer thread 0 has taken the tag

    unsigned int* status = reinterpret_cast<unsigned int*>(p.scratch);
    unsigned char* pairs = p.scratch + kPartialOffset;     // [CTA][16 tokens][256 rows] x {FP32 value, epoch}

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const int u_begin = (int)((long long)cta * p.units / G);     // units [u_begin, u_end) of this CTA
    const int u_end = (int)((long long)(cta + 1) * p.units / G);
    const int kc_begin = u_begin % p.kchunks;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1 + 32);             // the weight producer's expect_tx arrive + the 32 copying lanes
            ptx::mbar_init(&empty_bar[s], kConsumerWarps);    // every consumer warp releases every stage
        }
        *s_abort = 0;
        *s_epoch = 0u;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    ptx::griddep_launch_dependents();

    if (warp >= kConsumerWarps) {
        // ------------------------------------------------------------------ the two producer warps
        const bool acts = warp == kConsumerWarps + 1;
        if (!acts && lane != 0) return;
        if (acts) {
            ptx::griddep_wait();                              // the FP16 activations are the pre-pass kernel's output
        } else {
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
        }
        const uint64_t pol = ptx::policy_evict_first();
        int stage = 0;
        uint32_t ph = 0;
        int pair = u_begin / p.kchunks, kc = kc_begin;
        for (int u = u_begin; u < u_end; ++u) {
            ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, (acts ? 0x610u : 0x600u) + (unsigned)stage);
            const int k0 = kc * kKC;
            if (acts) {
                // chunk id = token * 32 + c: 16 bytes = 8 consecutive k of one token; token rows >= M are zero-filled
                unsigned char* dst = s_act + stage * kActBytes;
#pragma unroll 4
                for (int id = lane; id < kTokens * 32; id += 32) {
                    const int tok = id >> 5, c = id & 31;
                    const bool live = tok < p.M;
                    const unsigned short* src = p.act + (size_t)(live ? tok : 0) * p.K + k0 + c * 8;
                    ptx::cp_async_16(dst + tok * kActRowBytes + act_chunk_offset(c), src, live ? 16u : 0u);
                }
                ptx::cp_async_mbar_arrive_noinc(&full_bar[stage]);
            } else {
                ptx::mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)(kUnitPackedBytes + kUnitScaleBytes));
                ptx::tma_load_2d(s_packed + stage * kUnitPackedBytes, &tm_packed, &full_bar[stage], k0 >> 1, pair * kUnitRows, pol);
                ptx::tma_load_2d(s_scale + stage * kUnitScaleBytes, &tm_scale, &full_bar[stage], k0 >> 4, pair * kUnitRows, pol);
            }
            if (++kc == p.kchunks) { kc = 0; ++pair; }
            if (++stage == stages) { stage = 0; ph ^= 1u; }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int g = lane >> 2, t = lane & 3;
    const int r0 = warp * 16 + g;                              // unit rows r0 and r0 + 8
    const int off_w0 = r0 * 128 + (((2 * t) ^ g) << 4);       // row r0, logical 16-byte chunk 2t (swizzle: chunk ^ (row & 7))
    const int off_w1 = r0 * 128 + (((2 * t + 1) ^ g) << 4);
    const int off_s = r0 * 16 + 4 * t;                         // 4 scale bytes: blocks 4t..4t+3 of the row
    const int off_a = g * kActRowBytes + t * kActBlockBytes;   // token g (second tile: g + 8), 64-k block t; chunks at immediate offsets

    ptx::griddep_wait();          // outputs, residual, unscale and the cross-CTA scratch belong to earlier kernels until now
    // This launch's tag for the split-tile pairs: thread 0 takes it from the counter in the scratch and
    // leaves it in shared memory; the warps pick it up at their first segment epilogue, long after.
    unsigned int epoch_taken = 0;
    if (tid == 0) epoch_taken = ptx::take_launch_epoch(p.scratch);      // left in flight: parked at thread 0's first epilogue
    unsigned int epoch = 0;
    unsigned int xepoch = 0, xset = 0;      // group reduction: this launch's epoch and slot set
    if (p.xworld > 0) {
        xepoch = *reinterpret_cast<volatile unsigned int*>(p.xpeer[p.xrank] + xchg::kEpochOff) + 1u;
        xset = xepoch & 1u;
    }

    int stage = 0;
    uint32_t ph = 0;
    int u = u_begin, pair = u_begin / p.kchunks, kc = kc_begin;
    while (u < u_end) {
        const int kc_first = kc;
        const int pair_end = u - kc + p.kchunks;               // first unit of the next row pair
        const int seg_end = pair_end < u_end ? pair_end : u_end;
        float acc[kTT][4];
#pragma unroll
        for (int j = 0; j < kTT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

        for (; u < seg_end; ++u) {
            ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0x620u + (unsigned)stage);
            const unsigned char* wp = s_packed + stage * kUnitPackedBytes;
            const unsigned char* sp = s_scale + stage * kUnitScaleBytes + off_s;
            const unsigned char* ap = s_act + stage * kActBytes + off_a;
            const uint4 wa0 = *reinterpret_cast<const uint4*>(wp + off_w0);
            const uint4 wa1 = *reinterpret_cast<const uint4*>(wp + off_w1);
            const uint4 wb0 = *reinterpret_cast<const uint4*>(wp + off_w0 + 8 * 128);
            const uint4 wb1 = *reinterpret_cast<const uint4*>(wp + off_w1 + 8 * 128);
            const uint32_t qa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
            const uint32_t qb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
            uint32_t Sa[4], Sb[4];                             // block scales / 2^8 as f16x2, formed from the bytes
            {
                const uint32_t ba = mask_scale_bytes(*reinterpret_cast<const uint32_t*>(sp));
                const uint32_t bb = mask_scale_bytes(*reinterpret_cast<const uint32_t*>(sp + 8 * 16));
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    Sa[b] = scale_byte_to_f16x2(ba, b);
                    Sb[b] = scale_byte_to_f16x2(bb, b);
                }
            }
            float acc2[kTT][4];                                // second accumulators: halve the MMA dependency chains
#pragma unroll
            for (int j = 0; j < kTT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc2[j][i] = 0.0f;
#pragma unroll
            for (int uu = 0; uu < 8; ++uu) {
                uint32_t da[4], db[4];
                expand_u32(qa[uu], Sa[uu >> 1], da);
                expand_u32(qb[uu], Sb[uu >> 1], db);
                const uint32_t a_lo[4] = {da[0], db[0], da[1], db[1]};   // k 0..3 of this 8-group: rows g, g+8
                const uint32_t a_hi[4] = {da[2], db[2], da[3], db[3]};   // k 4..7
#pragma unroll
                for (int j = 0; j < kTT; ++j) {
                    const uint4 x = *reinterpret_cast<const uint4*>(ap + j * (8 * kActRowBytes) + uu * 16);   // token tile j: tokens 8j..8j+7
                    ptx::mma_f16_16x8x16(acc[j], a_lo, x.x, x.y);
                    ptx::mma_f16_16x8x16(acc2[j], a_hi, x.z, x.w);
                }
            }
#pragma unroll
            for (int j = 0; j < kTT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] += acc2[j][i];
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[stage]);
            if (++stage == stages) { stage = 0; ph ^= 1u; }
        }
        kc += seg_end - (pair_end - p.kchunks + kc_first);     // units consumed in this segment

        // ------------------------------------------------------------ segment epilogue, warp by warp
        // Thread (g,t) holds rows r0, r0+8 x tokens 8j+2t, 8j+2t+1 of the row pair.
        const bool owner = (kc_first == 0);
        const bool complete = owner && (seg_end == pair_end);
        int last = cta;                                        // contributors are CTAs cta+1 .. last
        if (owner && !complete)
            while (last + 1 < G && (long long)(last + 1) * p.units / G < pair_end) ++last;
        const int row_base = pair * kUnitRows;
        const int rr[4] = {r0, r0, r0 + 8, r0 + 8};
        if (tid == 0 && epoch_taken != 0u) {
            *s_epoch = epoch_taken;
            epoch_taken = 0u;
        }
        if (epoch == 0u && !(owner && complete)) {
            const long long te0 = clock64();
            while ((epoch = *s_epoch) == 0u) {
                if (*s_abort || clock64() - te0 > ptx::kWaitBudgetClocks) {
                    *s_abort = 1;
                    atomicCAS(status, 0u, 0x640u);
                    break;
                }
            }
        }
        float v[kTT][4];
#pragma unroll
        for (int j = 0; j < kTT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = 8 * j + 2 * t + (i & 1);
                v[j][i] = m < p.M ? acc[j][i] * p.unscale[m] : 0.0f;
            }
        if (!owner) {
            // the pair is its own arrival flag: an aligned 8-byte store is one transaction
            unsigned char* slot = pairs + (size_t)cta * (kTokens * kUnitRows) * 8;
#pragma unroll
            for (int j = 0; j < kTT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = 8 * j + 2 * t + (i & 1);
                    if (m < p.M) ptx::st_volatile_v2(slot + (m * kUnitRows + rr[i]) * 8, __float_as_uint(v[j][i]), epoch);
                }
        } else {
            // contributors in CTA order (a fixed summation order); the eight loads of one contributor
            // are issued before any is looked at; the wait for an old epoch is bounded
            const long long t0 = clock64();
            bool failed = false;
            for (int c = cta + 1; c <= last && !failed; ++c) {
                const unsigned char* src = pairs + (size_t)c * (kTokens * kUnitRows) * 8;
                while (true) {
                    uint2 x[kTT][4];
#pragma unroll
                    for (int j = 0; j < kTT; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int m = 8 * j + 2 * t + (i & 1);
                            x[j][i] = make_uint2(0u, epoch);
                            if (m < p.M) x[j][i] = ptx::ld_volatile_v2(src + (m * kUnitRows + rr[i]) * 8);
                        }
                    bool ready = true;
#pragma unroll
                    for (int j = 0; j < kTT; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) ready &= (x[j][i].y == epoch);
                    if (ready) {
#pragma unroll
                        for (int j = 0; j < kTT; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[j][i] += __uint_as_float(x[j][i].x);
                        break;
                    }
                    if (*s_abort || clock64() - t0 > ptx::kWaitBudgetClocks) {
                        *s_abort = 1;
                        atomicCAS(status, 0u, 0x630u);
                        failed = true;
                        break;
                    }
                }
            }
            __syncwarp();
            if (p.swiglu_out) {
                // the warp's slab is one gate/up slab: row r0 is a gate row (i = 0, 1), row r0 + 8 its up row
                // (i = 2, 3); both rounded to BF16 as the separate kernels would store them, then SwiGLU
                const int n_out = (row_base >> 1) + warp * 8 + g;
#pragma unroll
                for (int j = 0; j < kTT; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int m = 8 * j + 2 * t + i;
                        if (m >= p.M || row_base + r0 >= p.N) continue;
                        const float gate = __bfloat162float(__float2bfloat16_rn((v[j][i] * kBlockScaleUnfold) * p.inv_gs));
                        const float up = __bfloat162float(__float2bfloat16_rn((v[j][i + 2] * kBlockScaleUnfold) * p.inv_gs));
                        p.C[(size_t)m * (p.N / 2) + n_out] = __float2bfloat16_rn(silu(gate) * up);
                    }
            } else
#pragma unroll
            for (int j = 0; j < kTT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = 8 * j + 2 * t + (i & 1);
                    const int n = row_base + rr[i];
                    if (m >= p.M || n >= p.N) continue;
                    float x = (v[j][i] * kBlockScaleUnfold) * p.inv_gs;
                    const size_t o = (size_t)m * p.N + n;
                    if (p.xworld > 0) {   // the unrounded sum goes to slot [set][this rank] of every rank's buffer
                        const size_t pair = ((size_t)xset * p.xworld + p.xrank) * p.xslot_pairs + o;
                        for (int q = 0; q < p.xworld; ++q)
                            ptx::st_volatile_v2(p.xpeer[q] + xchg::kSlotsOff + pair * 8, __float_as_uint(x), xepoch);
                        continue;
                    }
                    if (p.residual) x += __bfloat162float(p.residual[o]);
                    p.C[o] = __float2bfloat16_rn(x);
                }
        }
        if (kc >= p.kchunks) { kc = 0; ++pair; }
    }

    // ---------------------------------------------------------------- reduction over the group
    // Every CTA takes 1/gridDim of the M x N outputs: it polls its own rank's buffer until the pairs of
    // all ranks carry this launch's epoch (bounded), adds them in rank order, adds the residual and
    // rounds once.  All CTAs of the grid are resident (one per SM) and an owner's push waits for nothing
    // that happens after it, so these waits cannot form a cycle.
    if (p.xworld > 0) {
        constexpr int kConsumers = kConsumerWarps * 32;
        unsigned char* mine = p.xpeer[p.xrank];
        const int E = p.M * p.N;
        const int e0 = (int)((long long)cta * E / G), e1 = (int)((long long)(cta + 1) * E / G);
        const long long t0 = clock64();
        bool failed = false;
        for (int e = e0 + tid; e < e1 && !failed; e += kConsumers) {
            float sum = 0.0f;
            for (int q = 0; q < p.xworld && !failed; ++q) {
                const unsigned char* src = mine + xchg::kSlotsOff + (((size_t)xset * p.xworld + q) * p.xslot_pairs + e) * 8;
                uint2 x = ptx::ld_volatile_v2(src);
                while (x.y != xepoch) {
                    if (clock64() - t0 > xchg::kWaitClocks) {
                        atomicCAS(reinterpret_cast<unsigned int*>(mine + xchg::kStatusOff), 0u, 0x710u + (unsigned)q);
                        failed = true;
                        break;
                    }
                    x = ptx::ld_volatile_v2(src);
                }
                sum += __uint_as_float(x.x);
            }
            if (failed) break;
            if (p.residual) sum += __bfloat162float(p.residual[e]);
            p.C[e] = __float2bfloat16_rn(sum);
        }
        // the last CTA to get here advances the launch counter for the next launch
        ptx::named_barrier_sync(1, kConsumers);
        if (tid == 0) {
            __threadfence();
            unsigned int* done = reinterpret_cast<unsigned int*>(mine + xchg::kDoneOff);
            if (atomicAdd(done, 1u) == (unsigned)G - 1u) {
                *done = 0u;
                *reinterpret_cast<volatile unsigned int*>(mine + xchg::kEpochOff) = xepoch;
            }
        }
    }
}

}  // namespace

bool decode_wide_supported(const LinearArgs& a) {
    if (a.M < 9 || a.M > kTokens || (a.K % kKC) != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u)) return false;
    if (a.swiglu_out && a.residual) return false;
    if (a.px && a.swiglu_out) return false;
    return !a.out_f32 && !a.swiglu_up && !a.a_stride && !a.k_valid && !a.norm_w;
}

size_t decode_wide_scratch_bytes(int sm_count) { return kPartialOffset + (size_t)sm_count * kTokens * kUnitRows * 8; }

cudaError_t configure_decode_wide() {
    return configure_large_smem(decode_wide_kernel, kSmemBudget);
}

// scratch: the handle workspace ([0, 16 KB) status word, then the partial pairs);
// act_f16 / unscale: room for the FP16 activation copy (M * K * 2 bytes) and M floats.
cudaError_t launch_decode_wide(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, void* act_f16, float* unscale,
                               int* launches, cudaStream_t s) {
    CUtensorMap tmp, tms;
    if (!umma::make_map_cached(dev.maps, &tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, 128, kUnitRows,
                        CU_TENSOR_MAP_SWIZZLE_128B) ||
        !umma::make_map_cached(dev.maps, &tms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, 16, kUnitRows,
                        CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    cudaError_t e = launch_act_to_f16(a.A, a.M, a.K, act_f16, unscale, s);
    if (e != cudaSuccess) return e;
    WideParams p{};
    p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.C = static_cast<__nv_bfloat16*>(a.C);
    p.unscale = unscale;
    p.act = static_cast<const unsigned short*>(act_f16);
    p.scratch = static_cast<unsigned char*>(scratch);
    p.inv_gs = a.inv_gs;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.swiglu_out = a.swiglu_out ? 1 : 0;
    if (a.px) {
        for (int q = 0; q < a.px->world; ++q) p.xpeer[q] = static_cast<unsigned char*>(a.px->peer[q]);
        p.xrank = a.px->rank;
        p.xworld = a.px->world;
        p.xslot_pairs = a.px->slot_pairs;
    }
    p.kchunks = a.K / kKC;
    p.units = (int)(((long long)a.N + kUnitRows - 1) / kUnitRows * p.kchunks);
    int grid = dev.sm_count < kWideMaxGrid ? dev.sm_count : kWideMaxGrid;
    if (grid > p.units) grid = p.units;
    const int fixed = 1024 + 2 * kMaxStages * 8 + 64;
    int stages = (kSmemBudget - fixed) / kStageBytes;
    if (stages > kMaxStages) stages = kMaxStages;
    p.stages = stages;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = fixed + stages * kStageBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_wide_kernel, tmp, tms, p);
    if (launches) *launches = 2;
    return e;
}

}  // namespace nvfp4
