// Tensor-parallel NVFP4 MLP: per-rank shards, two linears + SwiGLU from the core library; the
// down projection is the row-split linear of tp_common.cu (sum of the partials over the ranks
// inside the GEMV kernel for up to 16 tokens, NCCL all-reduce otherwise).
#include <cuda_bf16.h>

#include <cstring>

#include "tp_internal.h"

struct nvfp4_tp_mlp {
    nvfp4_handle* h = nullptr;
    nvfp4_tp_comm* comm = nullptr;
    int H = 0, I = 0, Ip = 0, Kp = 0, max_M = 0;     // Ip = I / world, Kp = Ip rounded up to 256
    uint8_t *gu_packed = nullptr, *gu_scale = nullptr, *dn_packed = nullptr, *dn_scale = nullptr;
    float gu_gs = 1.0f, dn_gs = 1.0f;
    void *gate_up_out = nullptr, *act = nullptr;      // [max_M, 2*Ip], [max_M, Kp] (pad columns stay zero)
    void* res_copy = nullptr;                          // [max_M, H]: the residual of an in-place call
    nvfp4_tp_exchange* own_x = nullptr;                // the block's own peer exchange ...
    nvfp4_tp_exchange* x = nullptr;                    // ... or one shared with other blocks of the rank
    int fused = 1;
};

namespace {
constexpr int kSwigluInEpilogueMaxM = 16;  // the GEMV kernels (8 tokens per launch, or the wide one for 9..16)
}

extern "C" {

int nvfp4_tp_mlp_destroy(nvfp4_tp_mlp* m) {
    if (!m) return NVFP4_E_NULL;
    cudaFree(m->gu_packed); cudaFree(m->gu_scale); cudaFree(m->dn_packed); cudaFree(m->dn_scale);
    cudaFree(m->gate_up_out); cudaFree(m->act); cudaFree(m->res_copy);
    if (m->own_x) nvfp4_tp_exchange_destroy(m->own_x);
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
    if (e == cudaSuccess) e = cudaMemset(m->dn_packed, 0, (size_t)H * m->Kp / 2);   // zero codes and zero scales
    if (e == cudaSuccess) e = cudaMemset(m->dn_scale, 0, (size_t)H * m->Kp / 16);   // in the K padding
    if (e == cudaSuccess) e = cudaMemset(m->act, 0, (size_t)max_M * m->Kp * 2);     // pad activations stay zero
    // gate rows [r*Ip, (r+1)*Ip) and up rows I + [r*Ip, (r+1)*Ip) of the merged tensor, interleaved in
    // slabs of 16 rows (8 gate rows, their 8 up rows): a thread of the GEMV kernel then holds a gate
    // value next to its up value and the SwiGLU moves into the gate_up epilogue.  One strided copy
    // per half: blocks of 8 rows land 16 rows apart.
    const size_t prow = (size_t)H / 2, srow = (size_t)H / 16;
    const size_t slabs = (size_t)m->Ip / 8;
    if (e == cudaSuccess) e = cudaMemcpy2D(m->gu_packed, 16 * prow, gup + (size_t)r * m->Ip * prow, 8 * prow, 8 * prow, slabs, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(m->gu_packed + 8 * prow, 16 * prow, gup + ((size_t)I + (size_t)r * m->Ip) * prow, 8 * prow, 8 * prow, slabs, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(m->gu_scale, 16 * srow, gus + (size_t)r * m->Ip * srow, 8 * srow, 8 * srow, slabs, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(m->gu_scale + 8 * srow, 16 * srow, gus + ((size_t)I + (size_t)r * m->Ip) * srow, 8 * srow, 8 * srow, slabs, cudaMemcpyDeviceToDevice);
    // down columns [r*Ip, (r+1)*Ip) of every row, into rows of Kp elements.
    if (e == cudaSuccess) e = cudaMemcpy2D(m->dn_packed, (size_t)m->Kp / 2, dnp + (size_t)r * m->Ip / 2, (size_t)I / 2, (size_t)m->Ip / 2, H, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(m->dn_scale, (size_t)m->Kp / 16, dns + (size_t)r * m->Ip / 16, (size_t)I / 16, (size_t)m->Ip / 16, H, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { nvfp4_tp_mlp_destroy(m); return (int)e; }
    if (int st = nvfp4::tp::reserve_f32_partials(comm, max_M, H)) { nvfp4_tp_mlp_destroy(m); return st; }
    if (int st = nvfp4_tp_exchange_create(comm, H, &m->own_x)) { nvfp4_tp_mlp_destroy(m); return st; }
    m->x = m->own_x;
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
    nvfp4::tp::SameGemvScope same_gemv(m->h, m->comm, m->x, m->fused, M);
    nvfp4_linear_desc d{};
    d.M = M;
    d.packed = m->dn_packed; d.scale = m->dn_scale; d.global_scale = m->dn_gs; d.N = m->H; d.K = m->Kp;
    d.residual = residual; d.C = out;
    int st;
    if (M <= kSwigluInEpilogueMaxM) {
        // Up to 16 tokens the gate_up GEMV forms bf16(silu(gate) * up) in its epilogue (the shard's rows
        // are interleaved for that), so the MLP is two kernels and the [M, 2 I/P] tensor never exists.
        // (The tcgen05 GEMM has the same epilogue, but there the separate SwiGLU kernel is faster:
        // 4096 tokens 1.92 ms against 1.97 ms, the activation math then sits in the four epilogue warps.)
        // The down projection reads the [M, I/P] result in place; columns beyond I/P of its padded K
        // count as zero.
        nvfp4_linear_desc g{};
        g.A = X; g.M = M;
        g.packed = m->gu_packed; g.scale = m->gu_scale; g.global_scale = m->gu_gs; g.N = 2 * m->Ip; g.K = m->H;
        g.C = m->gate_up_out;
        g.swiglu_epilogue = 1;
        st = nvfp4_linear_ex(m->h, &g, s);
        if (st == NVFP4_OK) {
            d.A = m->gate_up_out;
            if (m->Kp != m->Ip) { d.a_row_stride = m->Ip; d.k_valid = m->Ip; }
            st = nvfp4::tp::rowsplit_linear(m->h, m->comm, m->x, m->fused, d, m->res_copy, s);
            if (st != NVFP4_E_LIMIT) return st;
            // the general kernels want plain [M, Kp] rows: copy (the pad columns of `act` stay zero)
            if (cudaMemcpy2DAsync(m->act, (size_t)m->Kp * 2, m->gate_up_out, (size_t)m->Ip * 2, (size_t)m->Ip * 2, M,
                                  cudaMemcpyDeviceToDevice, s) != cudaSuccess)
                return NVFP4_E_TP;
            d.A = m->act; d.a_row_stride = 0; d.k_valid = 0;
            return nvfp4::tp::rowsplit_linear(m->h, m->comm, m->x, m->fused, d, m->res_copy, s);
        }
        if (st != NVFP4_E_LIMIT) return st;      // a shape the GEMV kernel does not take: the general path below
    }
    st = nvfp4_linear(m->h, X, M, m->gu_packed, m->gu_scale, m->gu_gs, 2 * m->Ip, m->H, nullptr, m->gate_up_out, s);
    if (st) return st;
    st = nvfp4_swiglu_interleaved(m->h, m->gate_up_out, M, m->Ip, 2LL * m->Ip, m->act, m->Kp, s);
    if (st) return st;
    d.A = m->act;
    return nvfp4::tp::rowsplit_linear(m->h, m->comm, m->x, m->fused, d, m->res_copy, s);
}

int nvfp4_tp_mlp_p2p_handle(nvfp4_tp_mlp* m, void* out) {
    if (!m) return NVFP4_E_NULL;
    return nvfp4_tp_exchange_handle(m->own_x, out);
}

int nvfp4_tp_mlp_p2p_attach(nvfp4_tp_mlp* m, const void* handles) {
    if (!m) return NVFP4_E_NULL;
    return nvfp4_tp_exchange_attach(m->own_x, handles);
}

int nvfp4_tp_mlp_use_exchange(nvfp4_tp_mlp* m, nvfp4_tp_exchange* x) {
    if (!m) return NVFP4_E_NULL;
    if (x && (x->H != m->H || x->comm->world != m->comm->world || x->comm->rank != m->comm->rank)) return NVFP4_E_SHAPE;
    m->x = x ? x : m->own_x;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_set_fused(nvfp4_tp_mlp* m, int on) {
    if (!m) return NVFP4_E_NULL;
    m->fused = on < 0 || on > 2 ? 1 : on;
    return NVFP4_OK;
}

int nvfp4_tp_mlp_status(nvfp4_tp_mlp* m, unsigned int* status) {
    if (!m) return NVFP4_E_NULL;
    return nvfp4_tp_exchange_status(m->x, status);
}

}  // extern "C"
