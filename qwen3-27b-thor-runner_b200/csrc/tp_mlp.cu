// Tensor-parallel NVFP4 MLP: per-rank shards, two linears + SwiGLU from the core library, and
// the sum of the down-projection partials over the ranks:
//   * up to 16 tokens, once the ranks have exchanged their buffer handles: the down-projection
//     GEMV itself (nvfp4_linear_reduce_peers) pushes its unrounded FP32 sums into every rank's
//     exchange buffer with plain peer stores over NVLink ({value, epoch} pairs, so the data is
//     its own flag), polls (bounded) its own buffer for the peers' pairs, adds the P partials in
//     rank order in FP32, adds the residual and rounds once.  No library collective, no
//     multicast, deterministic, one rounding.  (Mode 2 does the same with a separate
//     push-and-sum kernel behind an FP32 GEMV.)
//   * otherwise one NCCL all-reduce of the BF16 partials, the residual added in FP32 after it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstring>

#include "../../include/nvfp4_b200_tp.h"
#include "exchange_layout.h"

struct nvfp4_tp_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};

struct nvfp4_tp_mlp {
    nvfp4_handle* h = nullptr;
    nvfp4_tp_comm* comm = nullptr;
    int H = 0, I = 0, Ip = 0, Kp = 0, max_M = 0;     // Ip = I / world, Kp = Ip rounded up to 256
    uint8_t *gu_packed = nullptr, *gu_scale = nullptr, *dn_packed = nullptr, *dn_scale = nullptr;
    float gu_gs = 1.0f, dn_gs = 1.0f;
    void *gate_up_out = nullptr, *act = nullptr;      // [max_M, 2*Ip], [max_M, Kp] (pad columns stay zero)
    void* res_copy = nullptr;                          // [max_M, H]: the residual of an in-place call
    // Peer exchange (fused small-M reduction).  xbuf: this rank's buffer; peer[q]: rank q's buffer
    // as mapped into this process (peer[rank] == xbuf).
    unsigned char* xbuf = nullptr;
    unsigned char* peer[NVFP4_TP_MAX_WORLD] = {};
    float* partial = nullptr;                          // [kFusedMaxM, H] FP32: this rank's down-projection partial
    bool attached = false;
    int fused = 1;
};

namespace {

using namespace nvfp4::xchg;
constexpr int kFusedMaxM = kMaxTokens;
constexpr int kSwigluInStagingMaxM = 4;
constexpr int kXCtas = 32;               // most CTAs of the stand-alone exchange kernel
constexpr size_t kXStatusOff = kStatusOff, kXEpochOff = kEpochOff, kXDoneOff = kDoneOff, kXSlotsOff = kSlotsOff;
constexpr long long kXWaitClocks = kWaitClocks;

inline size_t xbuf_bytes(int world, int H) { return buffer_bytes(world, H); }

struct ExchangeParams {
    unsigned char* peer[NVFP4_TP_MAX_WORLD];
    const float* partial;            // this rank's [M, H] FP32 partial
    const __nv_bfloat16* residual;   // or null
    __nv_bfloat16* out;
    int rank, world, n4, H;          // n4 = M * H / 4
};

__device__ __forceinline__ void st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// One launch per rank, the same grid on every rank.  Every FP32 value travels as an 8-byte
// {value, launch epoch} pair (8-byte stores are single transactions), so the data is its own
// arrival flag: no fence, no separate flag write, one NVLink traversal.  A thread pushes its
// elements of the rank's partial into slot [set][rank] of every rank's buffer (16-byte stores
// = two pairs), then polls slots [set][0..P-1] of its own buffer until the pairs carry this
// launch's epoch (bounded), adds them in rank order, adds the residual and rounds once.  The
// two sets alternate per launch: a fast rank's next push never lands on pairs a slow rank still
// reads (it can only be two launches ahead after that rank has pushed the launch in between).
__global__ void __launch_bounds__(256) exchange_reduce_kernel(const ExchangeParams p) {
    unsigned char* mine = p.peer[p.rank];
    const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(mine + kXEpochOff) + 1u;
    const unsigned int set = epoch & 1u;
    const size_t slot_pairs = (size_t)kFusedMaxM * p.H;               // 8-byte pairs per slot
    const int tid = threadIdx.x;
    const size_t my_slot = ((size_t)set * p.world + p.rank) * slot_pairs * 8;
    for (int i = blockIdx.x * 256 + tid; i < p.n4; i += gridDim.x * 256) {
        const float4 v = reinterpret_cast<const float4*>(p.partial)[i];
        for (int q = 0; q < p.world; ++q) {
            unsigned char* dst = p.peer[q] + kXSlotsOff + my_slot + (size_t)i * 32;
            st_volatile_v4(dst, __float_as_uint(v.x), epoch, __float_as_uint(v.y), epoch);
            st_volatile_v4(dst + 16, __float_as_uint(v.z), epoch, __float_as_uint(v.w), epoch);
        }
    }
    const long long t0 = clock64();
    bool failed = false;
    for (int i = blockIdx.x * 256 + tid; i < p.n4 && !failed; i += gridDim.x * 256) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < p.world; ++q) {                          // rank 0 first, then 1, 2, ...: the same order on every rank
            const unsigned char* src = mine + kXSlotsOff + ((size_t)set * p.world + q) * slot_pairs * 8 + (size_t)i * 32;
            uint4 a, b;
            while (true) {
                a = ld_volatile_v4(src);
                b = ld_volatile_v4(src + 16);
                if (a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch) break;
                if (clock64() - t0 > kXWaitClocks) {
                    atomicCAS(reinterpret_cast<unsigned int*>(mine + kXStatusOff), 0u, 0x700u + (unsigned)q);
                    failed = true;
                    break;
                }
            }
            if (failed) break;
            s.x += __uint_as_float(a.x); s.y += __uint_as_float(a.z);
            s.z += __uint_as_float(b.x); s.w += __uint_as_float(b.z);
        }
        if (failed) break;
        if (p.residual) {
            const uint2 r = reinterpret_cast<const uint2*>(p.residual)[i];
            s.x += __uint_as_float(r.x << 16); s.y += __uint_as_float(r.x & 0xFFFF0000u);
            s.z += __uint_as_float(r.y << 16); s.w += __uint_as_float(r.y & 0xFFFF0000u);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(s.x, s.y), hi = __floats2bfloat162_rn(s.z, s.w);
        reinterpret_cast<uint2*>(p.out)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
    // the last CTA to finish advances the launch counter for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        unsigned int* done = reinterpret_cast<unsigned int*>(mine + kXDoneOff);
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0u;
            *reinterpret_cast<volatile unsigned int*>(mine + kXEpochOff) = epoch;
        }
    }
}

// out = bf16(float(out) + float(residual)), 8 elements per thread; n % 8 == 0 (H % 256 == 0).
__global__ void __launch_bounds__(256) add_residual_kernel(uint4* out, const uint4* residual, long long n8) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 a = out[i], b = residual[i];
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float lo = __uint_as_float(av[j] << 16) + __uint_as_float(bv[j] << 16);
            const float hi = __uint_as_float(av[j] & 0xFFFF0000u) + __uint_as_float(bv[j] & 0xFFFF0000u);
            const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
            o[j] = *reinterpret_cast<const uint32_t*>(&r);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace

extern "C" {

int nvfp4_tp_unique_id(void* out) {
    if (!out) return NVFP4_E_NULL;
    static_assert(sizeof(ncclUniqueId) == NVFP4_TP_UNIQUE_ID_BYTES, "unique id size");
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return NVFP4_E_TP;
    std::memcpy(out, &id, sizeof id);
    return NVFP4_OK;
}

int nvfp4_tp_comm_create(const void* uid, int rank, int world, nvfp4_tp_comm** out) {
    if (!out) return NVFP4_E_NULL;
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return NVFP4_E_TP;
    nvfp4_tp_comm* c = new nvfp4_tp_comm();
    c->rank = rank;
    c->world = world;
    if (world > 1) {
        if (!uid) { delete c; return NVFP4_E_NULL; }
        ncclUniqueId id;
        std::memcpy(&id, uid, sizeof id);
        if (ncclCommInitRank(&c->comm, world, id, rank) != ncclSuccess) { delete c; return NVFP4_E_TP; }
    }
    *out = c;
    return NVFP4_OK;
}

int nvfp4_tp_comm_destroy(nvfp4_tp_comm* c) {
    if (!c) return NVFP4_E_NULL;
    if (c->comm) ncclCommDestroy(c->comm);
    delete c;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_destroy(nvfp4_tp_mlp* m) {
    if (!m) return NVFP4_E_NULL;
    cudaFree(m->gu_packed); cudaFree(m->gu_scale); cudaFree(m->dn_packed); cudaFree(m->dn_scale);
    cudaFree(m->gate_up_out); cudaFree(m->act); cudaFree(m->res_copy);
    for (int q = 0; q < NVFP4_TP_MAX_WORLD; ++q)
        if (m->peer[q] && m->peer[q] != m->xbuf) cudaIpcCloseMemHandle(m->peer[q]);
    cudaFree(m->xbuf); cudaFree(m->partial);
    delete m;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_create(nvfp4_handle* h, nvfp4_tp_comm* comm, int H, int I, const uint8_t* gup, const uint8_t* gus,
                        float gu_gs, const uint8_t* dnp, const uint8_t* dns, float dn_gs, int max_M,
                        nvfp4_tp_mlp** out) {
    if (!h || !comm || !gup || !gus || !dnp || !dns || !out) return NVFP4_E_NULL;
    *out = nullptr;
    const int P = comm->world, r = comm->rank;
    if (H <= 0 || I <= 0 || max_M <= 0 || (H % 256) != 0 || (I % (16 * P)) != 0 || P > NVFP4_TP_MAX_WORLD) return NVFP4_E_SHAPE;
    nvfp4_tp_mlp* m = new nvfp4_tp_mlp();
    m->h = h; m->comm = comm; m->H = H; m->I = I; m->max_M = max_M;
    m->Ip = I / P;
    m->Kp = (m->Ip + 255) / 256 * 256;
    m->gu_gs = gu_gs; m->dn_gs = dn_gs;
    const size_t gu_rows = 2 * (size_t)m->Ip;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, bytes); };
    alloc((void**)&m->gu_packed, gu_rows * H / 2);
    alloc((void**)&m->gu_scale, gu_rows * H / 16);
    alloc((void**)&m->dn_packed, (size_t)H * m->Kp / 2);
    alloc((void**)&m->dn_scale, (size_t)H * m->Kp / 16);
    alloc(&m->gate_up_out, (size_t)max_M * gu_rows * 2);
    alloc(&m->act, (size_t)max_M * m->Kp * 2);
    alloc(&m->res_copy, (size_t)max_M * H * 2);
    alloc((void**)&m->xbuf, xbuf_bytes(P, H));
    alloc((void**)&m->partial, (size_t)kFusedMaxM * H * 4);
    if (e == cudaSuccess) e = cudaMemset(m->xbuf, 0, xbuf_bytes(P, H));
    if (e == cudaSuccess) e = cudaMemset(m->dn_packed, 0, (size_t)H * m->Kp / 2);   // zero codes and zero scales
    if (e == cudaSuccess) e = cudaMemset(m->dn_scale, 0, (size_t)H * m->Kp / 16);   // in the K padding
    if (e == cudaSuccess) e = cudaMemset(m->act, 0, (size_t)max_M * m->Kp * 2);     // pad activations stay zero
    // gate rows [r*Ip, (r+1)*Ip) then up rows I + [r*Ip, (r+1)*Ip): contiguous row blocks of the merged tensor.
    const size_t prow = (size_t)H / 2, srow = (size_t)H / 16;
    if (e == cudaSuccess) e = cudaMemcpy(m->gu_packed, gup + (size_t)r * m->Ip * prow, m->Ip * prow, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(m->gu_packed + m->Ip * prow, gup + ((size_t)I + (size_t)r * m->Ip) * prow, m->Ip * prow, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(m->gu_scale, gus + (size_t)r * m->Ip * srow, m->Ip * srow, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(m->gu_scale + m->Ip * srow, gus + ((size_t)I + (size_t)r * m->Ip) * srow, m->Ip * srow, cudaMemcpyDeviceToDevice);
    // down columns [r*Ip, (r+1)*Ip) of every row, into rows of Kp elements.
    if (e == cudaSuccess) e = cudaMemcpy2D(m->dn_packed, (size_t)m->Kp / 2, dnp + (size_t)r * m->Ip / 2, (size_t)I / 2, (size_t)m->Ip / 2, H, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(m->dn_scale, (size_t)m->Kp / 16, dns + (size_t)r * m->Ip / 16, (size_t)I / 16, (size_t)m->Ip / 16, H, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();   // the zeroed exchange buffer must be in place before a peer can push to it
    if (e != cudaSuccess) { nvfp4_tp_mlp_destroy(m); return (int)e; }
    *out = m;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_shard_bytes(nvfp4_tp_mlp* m, size_t* bytes) {
    if (!m || !bytes) return NVFP4_E_NULL;
    *bytes = 2 * (size_t)m->Ip * m->H * 9 / 16 + (size_t)m->H * m->Kp * 9 / 16;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_forward(nvfp4_tp_mlp* m, const void* X, int M, const void* residual, void* out, nvfp4_stream_t s) {
    if (!m || !X || !out) return NVFP4_E_NULL;
    if (M < 0 || M > m->max_M) return NVFP4_E_SHAPE;
    if (M == 0) return NVFP4_OK;
    const int P = m->comm->world;
    int st = nvfp4_linear(m->h, X, M, m->gu_packed, m->gu_scale, m->gu_gs, 2 * m->Ip, m->H, nullptr, m->gate_up_out, s);
    if (st) return st;
    const char* gate = static_cast<const char*>(m->gate_up_out);
    const char* up = gate + (size_t)m->Ip * 2;
    const bool in_kernel = m->attached && m->fused == 1;     // group reduction inside the down-projection kernel
    const bool standalone = m->attached && m->fused == 2;    // ... or by the separate push-and-sum kernel
    // Up to kSwigluInStagingMaxM tokens the down projection forms bf16(silu(gate) * up) while it
    // stages its activations, so the MLP is two kernels.  Every CTA of that kernel converts the
    // activations of its own k range, i.e. the SwiGLU is recomputed once per row tile; beyond a few
    // tokens that costs more than the separate SwiGLU launch it saves (measured: 8 tokens lose
    // 2.8 us, 1 token gains 0.9 us on the 2-GPU shard shapes).
    const bool swiglu_in_staging = M <= kSwigluInStagingMaxM;
    if (!swiglu_in_staging) {
        st = nvfp4_swiglu_strided(m->h, gate, up, M, m->Ip, 2LL * m->Ip, m->act, m->Kp, s);
        if (st) return st;
    }
    if (M <= kFusedMaxM && (in_kernel || (P == 1 && !standalone))) {
        // In a group the down projection also pushes its unrounded sums to all ranks and reduces
        // over them (rank order, FP32, residual, one rounding) before it ends.  `out` may alias
        // the residual.  Columns beyond I/P of the padded K count as zero.
        nvfp4_peer_exchange px{};
        for (int q = 0; q < P; ++q) px.peer[q] = m->peer[q];
        px.rank = m->comm->rank; px.world = P; px.slot_pairs = kFusedMaxM * m->H;
        nvfp4_linear_desc d{};
        if (swiglu_in_staging) { d.A = gate; d.swiglu_up = up; d.a_row_stride = 2LL * m->Ip; d.k_valid = m->Ip; }
        else d.A = m->act;
        d.M = M;
        d.packed = m->dn_packed; d.scale = m->dn_scale; d.global_scale = m->dn_gs; d.N = m->H; d.K = m->Kp;
        d.residual = residual; d.C = out;
        d.px = in_kernel ? &px : nullptr;
        st = nvfp4_linear_ex(m->h, &d, s);
        if (st != NVFP4_E_LIMIT) return st;      // a shape the GEMV kernel does not take: the general path below
    }
    if (swiglu_in_staging) {
        st = nvfp4_swiglu_strided(m->h, gate, up, M, m->Ip, 2LL * m->Ip, m->act, m->Kp, s);
        if (st) return st;
    }
    if (P == 1 && !standalone)
        return nvfp4_linear(m->h, m->act, M, m->dn_packed, m->dn_scale, m->dn_gs, m->H, m->Kp, residual, out, s);
    if (standalone && M <= kFusedMaxM) {
        // Two kernels: FP32 partial, then the stand-alone push-and-sum kernel (kept for comparison).
        st = nvfp4_linear_f32(m->h, m->act, M, m->dn_packed, m->dn_scale, m->dn_gs, m->H, m->Kp, m->partial, s);
        if (st == NVFP4_OK) {
            ExchangeParams xp{};
            for (int q = 0; q < P; ++q) xp.peer[q] = m->peer[q];
            xp.partial = m->partial;
            xp.residual = static_cast<const __nv_bfloat16*>(residual);
            xp.out = static_cast<__nv_bfloat16*>(out);
            xp.rank = m->comm->rank; xp.world = P; xp.H = m->H;
            xp.n4 = M * m->H / 4;
            int grid = (xp.n4 + 255) / 256;
            if (grid > kXCtas) grid = kXCtas;
            exchange_reduce_kernel<<<grid, 256, 0, s>>>(xp);
            return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_TP;
        }
        if (st != NVFP4_E_LIMIT) return st;
    }
    // The partials travel without the residual (a partial rounded to BF16 next to a residual ten
    // times its size would lose its low bits); it is added once, in FP32, after the sum.
    const void* res_src = residual;
    if (residual == out) {   // in place: keep a copy of the residual while `out` carries the partial
        if (cudaMemcpyAsync(m->res_copy, residual, (size_t)M * m->H * 2, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
            return NVFP4_E_TP;
        res_src = m->res_copy;
    }
    st = nvfp4_linear(m->h, m->act, M, m->dn_packed, m->dn_scale, m->dn_gs, m->H, m->Kp, nullptr, out, s);
    if (st) return st;
    if (ncclAllReduce(out, out, (size_t)M * m->H, ncclBfloat16, ncclSum, m->comm->comm, s) != ncclSuccess)
        return NVFP4_E_TP;
    if (res_src) {
        const long long n8 = (long long)M * m->H / 8;
        int blocks = (int)((n8 + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        add_residual_kernel<<<blocks, 256, 0, s>>>(static_cast<uint4*>(out), static_cast<const uint4*>(res_src), n8);
        if (cudaGetLastError() != cudaSuccess) return NVFP4_E_TP;
    }
    return NVFP4_OK;
}

int nvfp4_tp_mlp_p2p_handle(nvfp4_tp_mlp* m, void* out) {
    if (!m || !out) return NVFP4_E_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == NVFP4_TP_P2P_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t hd;
    if (cudaIpcGetMemHandle(&hd, m->xbuf) != cudaSuccess) return NVFP4_E_TP;
    std::memcpy(out, &hd, sizeof hd);
    return NVFP4_OK;
}

int nvfp4_tp_mlp_p2p_attach(nvfp4_tp_mlp* m, const void* handles) {
    if (!m) return NVFP4_E_NULL;
    if (m->attached) return NVFP4_E_TP;
    const int P = m->comm->world, r = m->comm->rank;
    if (P > 1 && !handles) return NVFP4_E_NULL;
    for (int q = 0; q < P; ++q) {
        if (q == r) { m->peer[q] = m->xbuf; continue; }
        cudaIpcMemHandle_t hd;
        std::memcpy(&hd, static_cast<const char*>(handles) + (size_t)q * NVFP4_TP_P2P_HANDLE_BYTES, sizeof hd);
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            for (int k = 0; k < q; ++k)
                if (k != r && m->peer[k]) { cudaIpcCloseMemHandle(m->peer[k]); m->peer[k] = nullptr; }
            return NVFP4_E_TP;
        }
        m->peer[q] = static_cast<unsigned char*>(ptr);
    }
    m->attached = true;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_set_fused(nvfp4_tp_mlp* m, int on) {
    if (!m) return NVFP4_E_NULL;
    m->fused = on < 0 || on > 2 ? 1 : on;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_status(nvfp4_tp_mlp* m, unsigned int* status) {
    if (!m || !status) return NVFP4_E_NULL;
    if (cudaDeviceSynchronize() != cudaSuccess) return NVFP4_E_TP;
    return cudaMemcpy(status, m->xbuf + kXStatusOff, 4, cudaMemcpyDeviceToHost) == cudaSuccess ? NVFP4_OK : NVFP4_E_TP;
}

}  // extern "C"
