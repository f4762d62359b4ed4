// Tensor-parallel NVFP4 MLP: per-rank shards, two linears + SwiGLU from the core library, one
// NCCL all-reduce of the BF16 down-projection partials.  Host-side orchestration only; the
// kernels are the core library's.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstring>

#include "../../include/nvfp4_b200_tp.h"

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
};

namespace {

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
    delete m;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_create(nvfp4_handle* h, nvfp4_tp_comm* comm, int H, int I, const uint8_t* gup, const uint8_t* gus,
                        float gu_gs, const uint8_t* dnp, const uint8_t* dns, float dn_gs, int max_M,
                        nvfp4_tp_mlp** out) {
    if (!h || !comm || !gup || !gus || !dnp || !dns || !out) return NVFP4_E_NULL;
    *out = nullptr;
    const int P = comm->world, r = comm->rank;
    if (H <= 0 || I <= 0 || max_M <= 0 || (H % 256) != 0 || (I % (16 * P)) != 0) return NVFP4_E_SHAPE;
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
    st = nvfp4_swiglu_strided(m->h, gate, gate + (size_t)m->Ip * 2, M, m->Ip, 2LL * m->Ip, m->act, m->Kp, s);
    if (st) return st;
    if (P == 1) return nvfp4_linear(m->h, m->act, M, m->dn_packed, m->dn_scale, m->dn_gs, m->H, m->Kp, residual, out, s);
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

}  // extern "C"
