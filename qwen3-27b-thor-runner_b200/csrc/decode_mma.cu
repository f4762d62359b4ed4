// Decode dequant-GEMV for M <= 16: a persistent, HBM-bound kernel.
//
//   C[M,N] = bf16( A[M,K] * W[N,K]^T (+ residual) ),  W = e2m1(code) * ue4m3(scale) / global_scale
//
// Structure (one CTA per SM, 1 producer warp + 8 consumer warps):
//   * The weight matrix is cut into units of 128 rows x 256 k (16 KB of packed codes + 2 KB of
//     block scales).  The units, ordered row-tile-major, are split evenly over the CTAs
//     ("stream-K"): every CTA streams the same number of bytes (+-1 unit) whatever N and K are.
//   * The producer warp feeds a multi-stage shared-memory ring: per unit two TMA tile copies
//     (packed codes with the 128-byte swizzle, scales) and 16-byte cp.async copies of the
//     activation slice, all completing on one mbarrier.  No cluster multicast anywhere.
//   * Each consumer warp owns 16 of the 128 rows.  Codes are expanded in registers: two E2M1
//     nibbles -> one bf16x2 register by mask, integer multiply (places sign and exponent/mantissa
//     bits) and mask, then one bf16x2 multiply by the block scale taken from a 256-entry
//     shared-memory table.  Every product lut*scale is exact in BF16 (2 + 4 significant bits).
//     The dot products run on the tensor cores (mma.sync m16n8k16, weights as the 16-row operand,
//     the <= 8 tokens as the 8-column operand) with FP32 accumulators -- CUDA cores alone cannot
//     convert AND multiply-accumulate 0.56 B/element at HBM speed for M > 1.
//   * A row tile whose K range is split over several CTAs is finished by the CTA that holds its
//     first unit: the others store FP32 partials to the handle's scratch and raise a flag; the
//     owner adds them in a fixed order (deterministic), applies 2^32/global_scale and the
//     residual in FP32 and rounds once to BF16.  Its wait on the flags is bounded.
//
// Arithmetic: group products are summed in FP32 by the MMA, block scales are applied exactly
// before the sum (they are exact), 1/global_scale once at the end.  This is the reference's
// GEMV arithmetic (src/engine/dense_gemm_fp4_sm110.cu:96-141, :192-240) up to FP32 summation
// order.
#include <cuda.h>
#include <cuda_bf16.h>

#include "nvfp4_format.cuh"
#include "nvfp4_internal.h"
#include "ptx.cuh"

namespace nvfp4 {
namespace {

constexpr int kRT = 128;                          // rows per unit
constexpr int kKC = 256;                          // k elements per unit
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;   // + producer warp
constexpr int kPackedBytes = kRT * kKC / 2;       // 16384
constexpr int kScaleBytes = kRT * kKC / 16;       // 2048
constexpr int kActRowBytes = kKC * 2;             // 512 per token
constexpr int kOutLd = kRT + 4;                   // padded row of the FP32 output tile
constexpr uint32_t kTxBytes = kPackedBytes + kScaleBytes;

// Scratch layout (handle workspace): status word, per-CTA flags, per-CTA partial tiles.
constexpr size_t kFlagsOffset = 256;
constexpr size_t kPartialOffset = 8192;
constexpr int kMaxGrid = (int)((kPartialOffset - kFlagsOffset) / 4);

template <int NT> struct Cfg {
    static constexpr int kStages = (NT == 1) ? 8 : 7;
    static constexpr int kActBytes = NT * 8 * kActRowBytes;
    static constexpr int kStageBytes = kPackedBytes + kScaleBytes + kActBytes;
    static constexpr int kOutBytes = NT * 8 * kOutLd * 4;
    static constexpr int kSmemBytes = 1024 /*align slack*/ + kStages * kStageBytes + kOutBytes + 1024 /*table*/ +
                                      2 * kStages * 8 + 64;
};

struct DecodeParams {
    const __nv_bfloat16* A;
    const __nv_bfloat16* residual;
    __nv_bfloat16* C;
    unsigned char* scratch;
    float final_scale;   // 2^32 / global_scale
    int M, N, K;
    int units, kchunks;  // total units, units per row tile
    unsigned int epoch;
};

// Two E2M1 codes (one per 16-bit half of x, already isolated at bit `shift` of each half)
// -> bf16x2 holding e2m1 * 2^-126 : sign at bit 15, (e e m) at bits 8..6 of each half.
// mul places the nibble at [15:12] and at [9:6]; the mask keeps the sign from the first copy and
// the magnitude from the second.
__device__ __forceinline__ uint32_t place_pair(uint32_t isolated, uint32_t mul) {
    return (isolated * mul) & 0x81C081C0u;
}

__device__ __forceinline__ void expand_u32(uint32_t q, uint32_t S, uint32_t (&d)[4]) {
    const uint32_t q2 = q >> 8;
    d[0] = ptx::mul_bf16x2(place_pair(q & 0x000F000Fu, 0x1040u), S);    // elements 0,4
    d[1] = ptx::mul_bf16x2(place_pair(q & 0x00F000F0u, 0x0104u), S);    // elements 1,5
    d[2] = ptx::mul_bf16x2(place_pair(q2 & 0x000F000Fu, 0x1040u), S);   // elements 2,6
    d[3] = ptx::mul_bf16x2(place_pair(q2 & 0x00F000F0u, 0x0104u), S);   // elements 3,7
}

template <int NT>
__global__ void __launch_bounds__(kThreads, 1)
decode_mma_kernel(const __grid_constant__ CUtensorMap tm_packed, const __grid_constant__ CUtensorMap tm_scale,
                  const DecodeParams p) {
    using C_ = Cfg<NT>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* s_packed = smem;                                          // kStages x 16 KB, 1024-aligned
    unsigned char* s_scale = s_packed + C_::kStages * kPackedBytes;          // kStages x 2 KB
    unsigned char* s_act = s_scale + C_::kStages * kScaleBytes;              // kStages x NT*4 KB
    float* s_out = reinterpret_cast<float*>(s_act + C_::kStages * C_::kActBytes);
    uint32_t* s_table = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(s_out) + C_::kOutBytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_table + 256);
    uint64_t* empty_bar = full_bar + C_::kStages;
    volatile int* s_abort = reinterpret_cast<volatile int*>(empty_bar + C_::kStages);

    unsigned int* status = reinterpret_cast<unsigned int*>(p.scratch);
    unsigned int* flags = reinterpret_cast<unsigned int*>(p.scratch + kFlagsOffset);
    float* partials = reinterpret_cast<float*>(p.scratch + kPartialOffset);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    const long long u_begin = (long long)cta * p.units / G;
    const long long u_end = (long long)(cta + 1) * p.units / G;

    if (tid == 0) {
        for (int s = 0; s < C_::kStages; ++s) {
            ptx::mbar_init(&full_bar[s], 1 + 32);             // expect_tx arrive + one cp.async arrive per producer lane
            ptx::mbar_init(&empty_bar[s], kConsumerWarps);
        }
        *s_abort = 0;
        ptx::fence_mbar_init();
    }
    // Block-scale table: code byte -> bf16x2 (both halves) of ue4m3(code) * 2^94.  With the 2^-126
    // of the placed E2M1 value the product is lut * scale * 2^-32, always a normal BF16.
    if (tid < 256) {
        const float s = ue4m3_to_float((uint32_t)tid) * 1.9807040628566084e28f;   // 2^94
        const uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(s));
        s_table[tid] = b | (b << 16);
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer warp
        if (lane == 0) {
            ptx::prefetch_tensormap(&tm_packed);
            ptx::prefetch_tensormap(&tm_scale);
        }
        const uint64_t pol_stream = ptx::policy_evict_first();
        int it = 0;
        for (long long u = u_begin; u < u_end; ++u, ++it) {
            const int stage = it % C_::kStages;
            const uint32_t ph = (uint32_t)((it / C_::kStages) & 1);
            ptx::mbar_wait(&empty_bar[stage], ph ^ 1u, s_abort, status, 0x100u + (unsigned)stage);
            const int tile = (int)(u / p.kchunks), kc = (int)(u % p.kchunks);
            const int row0 = tile * kRT, k0 = kc * kKC;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&full_bar[stage], kTxBytes);
                ptx::tma_load_2d(s_packed + stage * kPackedBytes, &tm_packed, &full_bar[stage], k0 >> 1, row0, pol_stream);
                ptx::tma_load_2d(s_scale + stage * kScaleBytes, &tm_scale, &full_bar[stage], k0 >> 4, row0, pol_stream);
            }
            unsigned char* act = s_act + stage * C_::kActBytes;
            for (int i = lane; i < p.M * 32; i += 32) {
                const int tok = i >> 5, c = i & 31;
                const int k = k0 + c * 8;
                const bool in = k < p.K;
                const __nv_bfloat16* src = p.A + (size_t)tok * p.K + (in ? k : 0);
                const int phys = (c & ~7) | ((c & 7) ^ (((c >> 3) & 3) | ((tok & 1) << 2)));
                ptx::cp_async_16(act + tok * kActRowBytes + phys * 16, src, in ? 16u : 0u);
            }
            ptx::cp_async_mbar_arrive_noinc(&full_bar[stage]);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int g = lane >> 2, t = lane & 3;
    const int r0 = warp * 16 + g;                       // tile rows r0 and r0 + 8
    // Shared-memory offsets that do not change from stage to stage.
    const int off_w0 = r0 * 128 + (((2 * t) ^ g) << 4);       // row r0, logical 16-byte chunk 2t   (swizzle: chunk ^ (row & 7))
    const int off_w1 = r0 * 128 + (((2 * t + 1) ^ g) << 4);   // row r0, chunk 2t+1
    const int off_s = r0 * 16 + 4 * t;                         // 4 scale bytes: blocks 4t..4t+3 of the row
    const int act_sw = t | ((g & 1) << 2);
    const int off_a = g * kActRowBytes + t * 128;              // token g, chunks 8t..8t+7 (low 3 bits swizzled)

    int it = 0;
    long long u = u_begin;
    while (u < u_end) {
        const int tile = (int)(u / p.kchunks);
        const int kc_first = (int)(u % p.kchunks);
        const long long tile_end = (long long)(tile + 1) * p.kchunks;
        const long long seg_end = tile_end < u_end ? tile_end : u_end;

        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[nt][j] = 0.0f;

        for (; u < seg_end; ++u, ++it) {
            const int stage = it % C_::kStages;
            const uint32_t ph = (uint32_t)((it / C_::kStages) & 1);
            ptx::mbar_wait(&full_bar[stage], ph, s_abort, status, 0x200u + (unsigned)stage);
            const unsigned char* wp = s_packed + stage * kPackedBytes;
            const unsigned char* sp = s_scale + stage * kScaleBytes;
            const unsigned char* ap = s_act + stage * C_::kActBytes;
            const uint4 wa0 = *reinterpret_cast<const uint4*>(wp + off_w0);
            const uint4 wa1 = *reinterpret_cast<const uint4*>(wp + off_w1);
            const uint4 wb0 = *reinterpret_cast<const uint4*>(wp + off_w0 + 8 * 128);
            const uint4 wb1 = *reinterpret_cast<const uint4*>(wp + off_w1 + 8 * 128);
            const uint32_t sa = *reinterpret_cast<const uint32_t*>(sp + off_s);
            const uint32_t sb = *reinterpret_cast<const uint32_t*>(sp + off_s + 8 * 16);
            const uint32_t qa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
            const uint32_t qb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
            uint32_t Sa = 0, Sb = 0;
#pragma unroll
            for (int uu = 0; uu < 8; ++uu) {
                if ((uu & 1) == 0) {
                    Sa = s_table[(sa >> (8 * (uu >> 1))) & 0xFFu];
                    Sb = s_table[(sb >> (8 * (uu >> 1))) & 0xFFu];
                }
                uint32_t da[4], db[4];
                expand_u32(qa[uu], Sa, da);
                expand_u32(qb[uu], Sb, db);
                const uint32_t a_lo[4] = {da[0], db[0], da[1], db[1]};   // elements (0,4 | 1,5) of this 8-group
                const uint32_t a_hi[4] = {da[2], db[2], da[3], db[3]};   // elements (2,6 | 3,7)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint4 x = *reinterpret_cast<const uint4*>(ap + nt * 8 * kActRowBytes + off_a + ((uu ^ act_sw) << 4));
                    // x = (x0,x1) (x2,x3) (x4,x5) (x6,x7)  ->  (x0,x4) (x1,x5) (x2,x6) (x3,x7)
                    const uint32_t b04 = ptx::prmt(x.x, x.z, 0x5410u), b15 = ptx::prmt(x.x, x.z, 0x7632u);
                    const uint32_t b26 = ptx::prmt(x.y, x.w, 0x5410u), b37 = ptx::prmt(x.y, x.w, 0x7632u);
                    ptx::mma_bf16_16x8x16(acc[nt], a_lo, b04, b15);
                    ptx::mma_bf16_16x8x16(acc[nt], a_hi, b26, b37);
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[stage]);
        }

        // ------------------------------------------------------------ segment epilogue
        const bool owner = (kc_first == 0);
        const bool complete = owner && (seg_end == tile_end);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s_out[(nt * 8 + 2 * t) * kOutLd + r0] = acc[nt][0];
            s_out[(nt * 8 + 2 * t + 1) * kOutLd + r0] = acc[nt][1];
            s_out[(nt * 8 + 2 * t) * kOutLd + r0 + 8] = acc[nt][2];
            s_out[(nt * 8 + 2 * t + 1) * kOutLd + r0 + 8] = acc[nt][3];
        }
        ptx::named_barrier_sync(1, kConsumerThreads);
        const int row_base = tile * kRT;
        if (!owner) {
            float* slot = partials + (size_t)cta * (NT * 8 * kRT);
            for (int i = tid; i < p.M * kRT; i += kConsumerThreads) {
                const int m = i / kRT, r = i % kRT;
                __stcg(slot + m * kRT + r, s_out[m * kOutLd + r]);
            }
            __threadfence();
            ptx::named_barrier_sync(1, kConsumerThreads);
            if (tid == 0) ptx::st_release_gpu(&flags[cta], p.epoch);
        } else {
            int last = cta;   // contributors are CTAs cta+1 .. last
            if (!complete) {
                while (last + 1 < G && (long long)(last + 1) * p.units / G < tile_end) ++last;
                if (tid == 0) {
                    const long long t0 = clock64();
                    for (int c = cta + 1; c <= last; ++c) {
                        while (ptx::ld_acquire_gpu(&flags[c]) != p.epoch) {
                            if (*s_abort) break;
                            if (clock64() - t0 > ptx::kWaitBudgetClocks) {
                                *s_abort = 1;
                                atomicCAS(status, 0u, 0x300u);
                                break;
                            }
                        }
                    }
                }
                ptx::named_barrier_sync(1, kConsumerThreads);
            }
            for (int i = tid; i < p.M * kRT; i += kConsumerThreads) {
                const int m = i / kRT, r = i % kRT;
                const int n = row_base + r;
                if (n >= p.N) continue;
                float v = s_out[m * kOutLd + r];
                for (int c = cta + 1; c <= last; ++c) v += __ldcg(partials + (size_t)c * (NT * 8 * kRT) + m * kRT + r);
                v *= p.final_scale;
                const size_t o = (size_t)m * p.N + n;
                if (p.residual) v += __bfloat162float(p.residual[o]);
                p.C[o] = __float2bfloat16_rn(v);
            }
        }
        ptx::named_barrier_sync(1, kConsumerThreads);   // s_out is reused by the next segment
    }
}

// ------------------------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}

bool make_u8_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_cols,
                 uint32_t box_rows, CUtensorMapSwizzle sw) {
    EncodeFn enc = get_encode();
    if (!enc) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool decode_mma_supported(const LinearArgs& a) {
    if (a.M < 1 || a.M > 16) return false;
    if ((a.K % 256) != 0) return false;   // scale rows (K/16 bytes) must be 16-byte multiples for the tile copy
    if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scale) & 15u)) return false;
    return true;
}

size_t decode_mma_scratch_bytes(const LinearArgs& a, const nvfp4_device_info& dev) {
    const int nt = a.M <= 8 ? 1 : 2;
    return kPartialOffset + (size_t)dev.sm_count * nt * 8 * kRT * 4;
}

cudaError_t configure_decode_mma() {
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<1>::kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg<2>::kSmemBytes);
}

cudaError_t launch_decode_mma(const LinearArgs& a, nvfp4_device_info& dev, void* scratch, int* launches,
                              cudaStream_t s) {
    CUtensorMap tmp, tms;
    if (!make_u8_map(&tmp, a.packed, (uint64_t)a.K / 2, (uint64_t)a.N, (uint64_t)a.K / 2, 128, kRT,
                     CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_u8_map(&tms, a.scale, (uint64_t)a.K / 16, (uint64_t)a.N, (uint64_t)a.K / 16, 16, kRT,
                     CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    DecodeParams p{};
    p.A = static_cast<const __nv_bfloat16*>(a.A);
    p.residual = static_cast<const __nv_bfloat16*>(a.residual);
    p.C = static_cast<__nv_bfloat16*>(a.C);
    p.scratch = static_cast<unsigned char*>(scratch);
    p.final_scale = a.inv_gs * 4294967296.0f;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.kchunks = a.K / kKC;
    const long long tiles = (a.N + kRT - 1) / kRT;
    p.units = (int)(tiles * p.kchunks);
    p.epoch = ++dev.decode_epoch;
    int grid = dev.sm_count < kMaxGrid ? dev.sm_count : kMaxGrid;
    if (grid > p.units) grid = p.units;
    if (a.M <= 8)
        decode_mma_kernel<1><<<grid, kThreads, Cfg<1>::kSmemBytes, s>>>(tmp, tms, p);
    else
        decode_mma_kernel<2><<<grid, kThreads, Cfg<2>::kSmemBytes, s>>>(tmp, tms, p);
    if (launches) *launches = 1;
    return cudaGetLastError();
}

}  // namespace nvfp4
