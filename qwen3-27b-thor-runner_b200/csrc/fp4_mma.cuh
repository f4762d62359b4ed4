// tcgen05 pieces shared by the NVFP4 tensor-core GEMVs (decode_fp4.cu, decode_fp4_stream.cu): the half-unit geometry,
// the kind::mxf4nvf4 instruction descriptor and MMA, and 16-column tensor-memory loads and stores.
#pragma once
#include <cstdint>

#include "umma.cuh"

namespace nvfp4 {
namespace fp4mma {

constexpr int kRT = 128;                           // weight rows per tile (UMMA M, tensor-memory lanes)
constexpr int kKC = 256;                           // k per half-unit
constexpr int kPackedBytes = kRT * kKC / 2;        // 16 KB
constexpr int kScaleBytes = kRT * kKC / 16;        // 2 KB of scales [row][16] per half-unit

// kind::mxf4nvf4: A = B = E2M1 (format 1), scales unsigned E4M3, both K-major, M = 128, N = NCp, K = 64.
__device__ __forceinline__ uint32_t fp4_idesc(int ncp) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(ncp >> 3) << 17) | ((uint32_t)(kRT >> 4) << 24);
}
__device__ __forceinline__ void umma_fp4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

}  // namespace fp4mma
}  // namespace nvfp4
