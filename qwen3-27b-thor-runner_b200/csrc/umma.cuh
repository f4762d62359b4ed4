// Pieces shared by the tcgen05 kernels: the persistent-CTA work list (whole tiles + stream-K
// remainder), shared-memory operand descriptors, commit / fence / tensor-memory load wrappers
// and the host-side tensor-map encoder.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "nvfp4_internal.h"
#include "ptx.cuh"

namespace nvfp4 {
namespace umma {

// Work of one CTA: first its share of the stream-K region (tiles [0, sk_tiles), cut into
// (tile, stage) units and split evenly over the CTAs), then whole tiles (or pairs of tiles)
// blockIdx.x + i * gridDim.x behind that region.  The interleaved order keeps the CTAs that share
// a weight tile in step, so the tile is fetched from HBM once and read from L2 by the others.
// Every role walks the same list.
struct Segment {
    int tile, ks0, ks1;
    int pair;     // 1, or 2: tiles `tile` and `tile + 1` (same weight rows, consecutive token tiles) over the whole k range
};
struct Schedule {
    long long u, u_end;
    int dp, dp_end, kstages;
    int m_tiles, pairs_per_nt;        // pairs_per_nt == 0: whole tiles are handed out one by one
    // Whole tiles one by one: tiles [0, sk_tiles) are the stream-K region.
    __device__ __forceinline__ Schedule(int sk_tiles, int tiles, int kst) {
        init_sk(sk_tiles, kst);
        dp = sk_tiles + blockIdx.x;
        dp_end = tiles;
        m_tiles = 1;
        pairs_per_nt = 0;
    }
    // Whole tiles in pairs of consecutive token tiles of one weight tile (the last pair of a
    // weight tile is a single when m_tiles is odd); the pairs [0, sk_pairs) -- tiles [0, sk_tiles)
    // -- are the stream-K region, handled tile by tile.
    __device__ __forceinline__ Schedule(int sk_tiles, int sk_pairs, int m_tiles_, int n_tiles, int kst) {
        init_sk(sk_tiles, kst);
        m_tiles = m_tiles_;
        pairs_per_nt = (m_tiles_ + 1) / 2;
        dp = sk_pairs + blockIdx.x;
        dp_end = n_tiles * pairs_per_nt;
    }
    __device__ __forceinline__ void init_sk(int sk_tiles, int kst) {
        const long long sk_units = (long long)sk_tiles * kst;
        u = (long long)blockIdx.x * sk_units / gridDim.x;
        u_end = (long long)(blockIdx.x + 1) * sk_units / gridDim.x;
        kstages = kst;
    }
    __device__ __forceinline__ bool next(Segment& s) {
        if (u < u_end) {
            s.tile = (int)(u / kstages);
            s.ks0 = (int)(u % kstages);
            const long long room = u_end - u;
            s.ks1 = (kstages - s.ks0) < room ? kstages : s.ks0 + (int)room;
            s.pair = 1;
            u += s.ks1 - s.ks0;
            return true;
        }
        if (dp < dp_end) {
            if (pairs_per_nt == 0) {
                s.tile = dp;
                s.pair = 1;
            } else {
                const int nt = dp / pairs_per_nt, mp = dp - nt * pairs_per_nt;
                s.tile = nt * m_tiles + 2 * mp;
                s.pair = m_tiles - 2 * mp >= 2 ? 2 : 1;
            }
            s.ks0 = 0;
            s.ks1 = kstages;
            dp += gridDim.x;
            return true;
        }
        return false;
    }
};

// ---------------------------------------------------------------- tcgen05 helpers
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    // K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(ptx::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_512(uint32_t* smem_slot) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(ptx::smem_u32(smem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_512(uint32_t tmem_base) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

// Split tiles the calling CTA holds a part of: [0] the one its span starts inside (partial slot
// 0), [1] the one its span ends inside (slot 1); -1 = none.
__device__ __forceinline__ void split_tiles_of_cta(int sk_tiles, int kstages, int out[2]) {
    out[0] = out[1] = -1;
    const long long sk_units = (long long)sk_tiles * kstages;
    const long long u0 = (long long)blockIdx.x * sk_units / gridDim.x;
    const long long u1 = (long long)(blockIdx.x + 1) * sk_units / gridDim.x;
    if (u0 >= u1) return;
    const int t0 = (int)(u0 / kstages), t1 = (int)((u1 - 1) / kstages);
    if (u0 % kstages != 0) out[0] = t0;
    else if (u1 - u0 < kstages) out[1] = t0;
    if (t1 != t0 && u1 - (long long)t1 * kstages < kstages) out[1] = t1;
}

// CTAs first..last hold the parts of split tile `tile`; the first one holds its head (slot 1),
// the others a middle or tail part (slot 0).
__device__ __forceinline__ void split_tile_participants(int sk_tiles, int kstages, int tile, int& first, int& last) {
    const long long sk_units = (long long)sk_tiles * kstages;
    const long long tile_begin = (long long)tile * kstages, tile_end = tile_begin + kstages;
    first = last = blockIdx.x;
    while (first > 0 && (long long)first * sk_units / gridDim.x > tile_begin) --first;
    while (last + 1 < (int)gridDim.x && (long long)(last + 1) * sk_units / gridDim.x < tile_end) ++last;
}

// Bounded wait until every participant's flag carries this launch's epoch.  Each lane of a warp
// polls another participant, so the flag round trips overlap.
__device__ __forceinline__ bool wait_split_tile_flags(const unsigned int* flags, unsigned int epoch, int first, int last,
                                                      int t, volatile int* s_abort, unsigned int* status) {
    const long long t0 = clock64();
    for (int c = first + (t & 31); c <= last; c += 32) {
        const unsigned int* f = &flags[c * 2 + (c == first ? 1 : 0)];
        while (ptx::ld_acquire_gpu(f) != epoch) {
            if (*s_abort) break;
            if (clock64() - t0 > ptx::kWaitBudgetClocks) {
                *s_abort = 1;
                atomicCAS(status, 0u, 0x480u);
                break;
            }
        }
    }
    __syncwarp();
    return *s_abort == 0;
}

// ---------------------------------------------------------------- host: tensor maps
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn get_encode() {
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

inline bool make_map(CUtensorMap* m, CUtensorMapDataType dt, int esize, const void* base, uint64_t cols, uint64_t rows,
              uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
    EncodeFn enc = get_encode();
    if (!enc) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * (uint64_t)esize};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same through a cache (may be null): weights are called again and again with the same geometry.
inline bool make_map_cached(TensorMapCache* cache, CUtensorMap* m, CUtensorMapDataType dt, int esize, const void* base,
                            uint64_t cols, uint64_t rows, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
    if (!cache) return make_map(m, dt, esize, base, cols, rows, box_cols, box_rows, sw);
    const uintptr_t a = reinterpret_cast<uintptr_t>(base);
    const unsigned slot = (unsigned)(((a >> 8) ^ (a >> 17) ^ (uintptr_t)box_rows ^ ((uintptr_t)box_cols << 3)) % TensorMapCache::kEntries);
    TensorMapCache::Entry& e = cache->e[slot];
    if (e.base == base && e.cols == cols && e.rows == rows && e.box_cols == box_cols && e.box_rows == box_rows &&
        e.dtype == (int)dt && e.esize == esize && e.swizzle == (int)sw) {
        *m = e.map;
        return true;
    }
    if (!make_map(m, dt, esize, base, cols, rows, box_cols, box_rows, sw)) return false;
    e.base = base; e.cols = cols; e.rows = rows; e.box_cols = box_cols; e.box_rows = box_rows;
    e.dtype = (int)dt; e.esize = esize; e.swizzle = (int)sw;
    e.map = *m;
    return true;
}

}  // namespace umma
}  // namespace nvfp4
