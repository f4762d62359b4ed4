// Tensor-parallel plumbing shared by the blocks: the NCCL communicator, the peer-exchange object
// of the fused small-M reduction (CUDA IPC buffers, {value, epoch} pairs) and the row-split linear
// that ends both the MLP block and the attention-projection block:
//   * up to 16 tokens, with an attached exchange: the GEMV itself (nvfp4_linear_ex with px)
//     pushes its unrounded FP32 sums into every rank's exchange buffer with plain peer stores
//     over NVLink, polls (bounded) its own buffer for the peers' pairs, adds the P partials in
//     rank order in FP32, adds the residual and rounds once.  No library collective, no
//     multicast, deterministic, one rounding.  (Mode 2 does the same with a separate
//     push-and-sum kernel behind an FP32 GEMV.)
//   * otherwise one NCCL all-reduce of the BF16 partials, the residual added in FP32 after it.
#include <cuda_bf16.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "tp_internal.h"

namespace {

using namespace nvfp4::xchg;
using nvfp4::tp::kFusedMaxM;
constexpr int kXCtas = 32;               // most CTAs of the stand-alone exchange kernel
constexpr size_t kXStatusOff = kStatusOff, kXEpochOff = kEpochOff, kXDoneOff = kDoneOff, kXSlotsOff = kSlotsOff;
constexpr long long kXWaitClocks = kWaitClocks;

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

// This rank's slice of the reduce-scattered FP32 sums: out = bf16(sum + residual), one rounding.
// 8 elements per thread; n % 8 == 0.
__global__ void __launch_bounds__(256) finish_slice_kernel(const float4* sum, const uint4* residual, uint4* out, long long n8) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const float4 a = sum[2 * i], b = sum[2 * i + 1];
        float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if (residual) {
            const uint4 r = residual[i];
            const uint32_t rv[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[2 * j] += __uint_as_float(rv[j] << 16);
                f[2 * j + 1] += __uint_as_float(rv[j] & 0xFFFF0000u);
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 r2 = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            o[j] = *reinterpret_cast<const uint32_t*>(&r2);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace

namespace nvfp4 {
namespace tp {

int settle(nvfp4_tp_comm* comm, ncclResult_t r) {
    if (!comm || !comm->comm || comm->aborted) return NVFP4_E_TP;
    if (r == ncclSuccess) return NVFP4_OK;
    const auto t0 = std::chrono::steady_clock::now();
    while (r == ncclInProgress) {
        if (ncclCommGetAsyncError(comm->comm, &r) != ncclSuccess) { r = ncclInternalError; break; }
        if (r != ncclInProgress) break;
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > comm->deadline_ms) break;
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (r == ncclSuccess) return NVFP4_OK;
    // an error, or a peer that did not show up in time: give the communicator up (frees its resources, never blocks)
    ncclCommAbort(comm->comm);
    comm->comm = nullptr;
    comm->aborted = true;
    return NVFP4_E_TP;
}

int reserve_f32_partials(nvfp4_tp_comm* comm, int max_M, int H) {
    if (!comm || comm->world == 1) return NVFP4_OK;
    const size_t need = (size_t)max_M * H * 4;
    if (need <= comm->f32_bytes) return NVFP4_OK;
    if (cudaDeviceSynchronize() != cudaSuccess) return NVFP4_E_TP;      // nothing in flight may still use the old buffer
    cudaFree(comm->f32_scratch);
    comm->f32_scratch = nullptr;
    comm->f32_bytes = 0;
    if (cudaMalloc((void**)&comm->f32_scratch, need) != cudaSuccess) return NVFP4_E_TP;
    comm->f32_bytes = need;
    return NVFP4_OK;
}

int rowsplit_linear(nvfp4_handle* h, nvfp4_tp_comm* comm, nvfp4_tp_exchange* x, int mode, const nvfp4_linear_desc& d,
                    void* res_copy, cudaStream_t s) {
    const int P = comm->world;
    const int M = d.M, H = d.N;
    const bool attached = x && x->attached && x->H == H;
    const bool in_kernel = attached && mode == 1;     // group reduction inside the GEMV kernel
    const bool standalone = attached && mode == 2;    // ... or by the separate push-and-sum kernel
    const bool plain = !d.swiglu_up && !d.a_row_stride && !d.k_valid;
    if (M <= kFusedMaxM && (in_kernel || (P == 1 && !standalone))) {
        // In a group the GEMV also pushes its unrounded sums to all ranks and reduces over them
        // (rank order, FP32, residual, one rounding) before it ends.  C may alias the residual.
        nvfp4_peer_exchange px{};
        nvfp4_linear_desc e = d;
        if (in_kernel) {
            for (int q = 0; q < P; ++q) px.peer[q] = x->peer[q];
            px.rank = comm->rank; px.world = P; px.slot_pairs = kFusedMaxM * H;
            e.px = &px;
        } else {
            e.px = nullptr;
        }
        const int st = nvfp4_linear_ex(h, &e, s);
        if (st != NVFP4_E_LIMIT) return st;          // a shape the GEMV kernel does not take: the general paths below
    }
    if (!plain) return NVFP4_E_LIMIT;
    const bool use_standalone = standalone && M <= kFusedMaxM;
    if (P == 1 && !use_standalone)
        return nvfp4_linear(h, d.A, M, d.packed, d.scale, d.global_scale, H, d.K, d.residual, d.C, s);
    if (use_standalone) {
        // Two kernels: FP32 partial, then the stand-alone push-and-sum kernel (kept for comparison).
        int st = nvfp4_linear_f32(h, d.A, M, d.packed, d.scale, d.global_scale, H, d.K, x->partial, s);
        if (st == NVFP4_OK) {
            ExchangeParams xp{};
            for (int q = 0; q < P; ++q) xp.peer[q] = x->peer[q];
            xp.partial = x->partial;
            xp.residual = static_cast<const __nv_bfloat16*>(d.residual);
            xp.out = static_cast<__nv_bfloat16*>(d.C);
            xp.rank = comm->rank; xp.world = P; xp.H = H;
            xp.n4 = M * H / 4;
            int grid = (xp.n4 + 255) / 256;
            if (grid > kXCtas) grid = kXCtas;
            exchange_reduce_kernel<<<grid, 256, 0, s>>>(xp);
            return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_TP;
        }
        if (st != NVFP4_E_LIMIT) return st;
        if (P == 1) return nvfp4_linear(h, d.A, M, d.packed, d.scale, d.global_scale, H, d.K, d.residual, d.C, s);
    }
    // FP32 partials: every rank's unrounded sums are reduce-scattered in FP32, the rank adds the residual
    // to its slice and rounds ONCE, the BF16 slices are all-gathered.  (BF16-rounded partials put P
    // roundings in front of the sum: 1.1e-3 / 1.4e-3 from the unsplit result at 4 / 8 ranks, measured.)
    // An in-place residual needs no copy: a rank reads only its own slice of it before the gather.
    if (!comm->comm) return NVFP4_E_TP;          // a group without a live communicator (never created, or aborted)
    const size_t total = (size_t)M * H;
    if (!comm->bf16_partials && comm->f32_scratch && total * 4 <= comm->f32_bytes && (total % ((size_t)P * 8)) == 0) {
        int st = nvfp4_linear_f32(h, d.A, M, d.packed, d.scale, d.global_scale, H, d.K, comm->f32_scratch, s);
        if (st == NVFP4_OK) {
            const size_t cnt = total / P, off = (size_t)comm->rank * cnt;
            if (settle(comm, ncclReduceScatter(comm->f32_scratch, comm->f32_scratch + off, cnt, ncclFloat, ncclSum, comm->comm, s)))
                return NVFP4_E_TP;
            const long long n8 = (long long)(cnt / 8);
            int blocks = (int)((n8 + 255) / 256);
            if (blocks > 148 * 8) blocks = 148 * 8;
            finish_slice_kernel<<<blocks, 256, 0, s>>>(
                reinterpret_cast<const float4*>(comm->f32_scratch + off),
                d.residual ? reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(d.residual) + off) : nullptr,
                reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(d.C) + off), n8);
            if (cudaGetLastError() != cudaSuccess) return NVFP4_E_TP;
            if (settle(comm, ncclAllGather(static_cast<const __nv_bfloat16*>(d.C) + off, d.C, cnt, ncclBfloat16, comm->comm, s)))
                return NVFP4_E_TP;
            return NVFP4_OK;
        }
        if (st != NVFP4_E_LIMIT) return st;      // a shape without an FP32 epilogue: BF16 partials below
    }
    // BF16 partials.  They travel without the residual (a partial rounded to BF16 next to a residual ten
    // times its size would lose its low bits); it is added once, in FP32, after the sum.
    const void* res_src = d.residual;
    if (d.residual && d.residual == d.C) {   // in place: keep a copy of the residual while C carries the partial
        if (!res_copy) return NVFP4_E_NULL;
        if (cudaMemcpyAsync(res_copy, d.residual, (size_t)M * H * 2, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
            return NVFP4_E_TP;
        res_src = res_copy;
    }
    int st = nvfp4_linear(h, d.A, M, d.packed, d.scale, d.global_scale, H, d.K, nullptr, d.C, s);
    if (st) return st;
    if (settle(comm, ncclAllReduce(d.C, d.C, (size_t)M * H, ncclBfloat16, ncclSum, comm->comm, s)))
        return NVFP4_E_TP;
    if (res_src) {
        const long long n8 = (long long)M * H / 8;
        int blocks = (int)((n8 + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        add_residual_kernel<<<blocks, 256, 0, s>>>(static_cast<uint4*>(d.C), static_cast<const uint4*>(res_src), n8);
        if (cudaGetLastError() != cudaSuccess) return NVFP4_E_TP;
    }
    return NVFP4_OK;
}

}  // namespace tp
}  // namespace nvfp4

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
        // Non-blocking: the call returns at once and the set-up proceeds in the background; a rank that never
        // calls leaves the others polling until the deadline instead of blocked inside the library for good.
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.blocking = 0;
        const ncclResult_t r = ncclCommInitRankConfig(&c->comm, world, id, rank, &cfg);
        if (r != ncclSuccess && r != ncclInProgress) { delete c; return NVFP4_E_TP; }
        if (nvfp4::tp::settle(c, r) != NVFP4_OK) { delete c; return NVFP4_E_TP; }
    }
    *out = c;
    return NVFP4_OK;
}

int nvfp4_tp_comm_set_deadline_ms(nvfp4_tp_comm* c, int ms) {
    if (!c) return NVFP4_E_NULL;
    if (ms < 1) return NVFP4_E_OPTION;
    c->deadline_ms = ms;
    return NVFP4_OK;
}

int nvfp4_tp_comm_state(nvfp4_tp_comm* c, int* state) {
    if (!c || !state) return NVFP4_E_NULL;
    if (c->aborted) { *state = -1; return NVFP4_OK; }
    if (!c->comm) { *state = 0; return NVFP4_OK; }            // a group of one has no communicator to ask
    ncclResult_t r = ncclSuccess;
    if (ncclCommGetAsyncError(c->comm, &r) != ncclSuccess) { *state = -1; return NVFP4_OK; }
    *state = r == ncclSuccess ? 0 : (r == ncclInProgress ? 1 : -1);
    return NVFP4_OK;
}

int nvfp4_tp_comm_abort(nvfp4_tp_comm* c) {
    if (!c) return NVFP4_E_NULL;
    if (c->comm) ncclCommAbort(c->comm);
    c->comm = nullptr;
    c->aborted = true;
    return NVFP4_OK;
}

int nvfp4_tp_comm_set_bf16_partials(nvfp4_tp_comm* c, int on) {
    if (!c) return NVFP4_E_NULL;
    c->bf16_partials = on ? 1 : 0;
    return NVFP4_OK;
}

int nvfp4_tp_comm_destroy(nvfp4_tp_comm* c) {
    if (!c) return NVFP4_E_NULL;
    cudaFree(c->f32_scratch);
    if (c->comm) {
        // a non-blocking communicator is finalized first (that call, too, may come back as "in progress")
        if (nvfp4::tp::settle(c, ncclCommFinalize(c->comm)) == NVFP4_OK && c->comm) ncclCommDestroy(c->comm);
    }
    delete c;
    return NVFP4_OK;
}

int nvfp4_tp_exchange_destroy(nvfp4_tp_exchange* x) {
    if (!x) return NVFP4_E_NULL;
    for (int q = 0; q < NVFP4_TP_MAX_WORLD; ++q)
        if (x->peer[q] && x->peer[q] != x->xbuf) cudaIpcCloseMemHandle(x->peer[q]);
    cudaFree(x->xbuf);
    cudaFree(x->partial);
    delete x;
    return NVFP4_OK;
}

int nvfp4_tp_exchange_create(nvfp4_tp_comm* comm, int H, nvfp4_tp_exchange** out) {
    if (!comm || !out) return NVFP4_E_NULL;
    *out = nullptr;
    if (H <= 0 || (H % 256) != 0 || comm->world > NVFP4_TP_MAX_WORLD) return NVFP4_E_SHAPE;
    nvfp4_tp_exchange* x = new nvfp4_tp_exchange();
    x->comm = comm;
    x->H = H;
    const size_t bytes = buffer_bytes(comm->world, H);
    cudaError_t e = cudaMalloc((void**)&x->xbuf, bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&x->partial, (size_t)kFusedMaxM * H * 4);
    if (e == cudaSuccess) e = cudaMemset(x->xbuf, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();   // the zeroed buffer must be in place before a peer can push to it
    if (e != cudaSuccess) { nvfp4_tp_exchange_destroy(x); return (int)e; }
    *out = x;
    return NVFP4_OK;
}

int nvfp4_tp_exchange_handle(nvfp4_tp_exchange* x, void* out) {
    if (!x || !out) return NVFP4_E_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == NVFP4_TP_P2P_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t hd;
    if (cudaIpcGetMemHandle(&hd, x->xbuf) != cudaSuccess) return NVFP4_E_TP;
    std::memcpy(out, &hd, sizeof hd);
    return NVFP4_OK;
}

int nvfp4_tp_exchange_attach(nvfp4_tp_exchange* x, const void* handles) {
    if (!x) return NVFP4_E_NULL;
    if (x->attached) return NVFP4_E_TP;
    const int P = x->comm->world, r = x->comm->rank;
    if (P > 1 && !handles) return NVFP4_E_NULL;
    for (int q = 0; q < P; ++q) {
        if (q == r) { x->peer[q] = x->xbuf; continue; }
        cudaIpcMemHandle_t hd;
        std::memcpy(&hd, static_cast<const char*>(handles) + (size_t)q * NVFP4_TP_P2P_HANDLE_BYTES, sizeof hd);
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            for (int k = 0; k < q; ++k)
                if (k != r && x->peer[k]) { cudaIpcCloseMemHandle(x->peer[k]); x->peer[k] = nullptr; }
            return NVFP4_E_TP;
        }
        x->peer[q] = static_cast<unsigned char*>(ptr);
    }
    x->attached = true;
    return NVFP4_OK;
}

int nvfp4_tp_exchange_status(nvfp4_tp_exchange* x, unsigned int* status) {
    if (!x || !status) return NVFP4_E_NULL;
    if (cudaDeviceSynchronize() != cudaSuccess) return NVFP4_E_TP;
    return cudaMemcpy(status, x->xbuf + kXStatusOff, 4, cudaMemcpyDeviceToHost) == cudaSuccess ? NVFP4_OK : NVFP4_E_TP;
}

}  // extern "C"
