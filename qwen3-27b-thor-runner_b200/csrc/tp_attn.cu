// Tensor-parallel attention projections: the merged QKV linear split by output rows (whole
// KV-head groups per rank, no exchange) and the output projection split by K columns, its
// partial sums added over the ranks by the row-split linear of tp_common.cu.  The attention
// itself (between the two calls) belongs to the caller: it works on this rank's heads only.
//
// Reference sequence (single GPU): src/engine/layer.cu:190-217 (merged FP4 QKV projection into
// q | k | v) and :404-409 (output projection, residual added by the caller's next fused
// add + norm).  Here the residual can ride in the output projection's epilogue.
//
// Split of the merged [q_rows + 2 kv_rows, H] tensor (q rows, then k rows, then v rows) over P
// ranks with n_kv KV heads: rank r owns q rows [r q_rows/P, (r+1) q_rows/P) -- the query heads
// of its KV heads, which are contiguous in grouped-query attention -- and
//   P <= n_kv: k and v rows of KV heads [r n_kv/P, (r+1) n_kv/P);
//   P >  n_kv: k and v rows of KV head r / (P / n_kv), replicated on P / n_kv ranks.
// The output projection [H, o_in] is cut into K columns [r o_in/P, (r+1) o_in/P), zero-padded to
// a multiple of 256 so that the scale rows stay 16-byte multiples.
#include <cuda_bf16.h>

#include "tp_internal.h"

struct nvfp4_tp_attn {
    nvfp4_handle* h = nullptr;
    nvfp4_tp_comm* comm = nullptr;
    int H = 0, q_local = 0, kv_local = 0, o_local = 0, Kp = 0, max_M = 0;
    uint8_t *qkv_packed = nullptr, *qkv_scale = nullptr, *o_packed = nullptr, *o_scale = nullptr;
    float qkv_gs = 1.0f, o_gs = 1.0f;
    void* act = nullptr;          // [max_M, Kp]: padded copy of the attention output where the GEMV kernel cannot read it in place
    void* res_copy = nullptr;     // [max_M, H]
    nvfp4_tp_exchange* x = nullptr;
    int fused = 1;
};

extern "C" {

int nvfp4_tp_attn_destroy(nvfp4_tp_attn* a) {
    if (!a) return NVFP4_E_NULL;
    cudaFree(a->qkv_packed); cudaFree(a->qkv_scale); cudaFree(a->o_packed); cudaFree(a->o_scale);
    cudaFree(a->act); cudaFree(a->res_copy);
    delete a;
    return NVFP4_OK;
}

int nvfp4_tp_attn_create(nvfp4_handle* h, nvfp4_tp_comm* comm, int H, int q_rows, int kv_rows, int n_kv_heads, int o_in,
                         const uint8_t* qkvp, const uint8_t* qkvs, float qkv_gs, const uint8_t* op, const uint8_t* os,
                         float o_gs, int max_M, nvfp4_tp_attn** out) {
    if (!h || !comm || !qkvp || !qkvs || !op || !os || !out) return NVFP4_E_NULL;
    *out = nullptr;
    const int P = comm->world, r = comm->rank;
    if (H <= 0 || q_rows <= 0 || kv_rows <= 0 || n_kv_heads <= 0 || o_in <= 0 || max_M <= 0) return NVFP4_E_SHAPE;
    if ((H % 256) != 0 || (q_rows % (8 * P)) != 0 || (kv_rows % n_kv_heads) != 0 || (o_in % (16 * P)) != 0 ||
        P > NVFP4_TP_MAX_WORLD)
        return NVFP4_E_SHAPE;
    if (P <= n_kv_heads ? (n_kv_heads % P) != 0 : (P % n_kv_heads) != 0) return NVFP4_E_SHAPE;
    const int head_rows = kv_rows / n_kv_heads;
    const int kv_local = P <= n_kv_heads ? kv_rows / P : head_rows;
    const int kv_first = P <= n_kv_heads ? r * kv_local : (r / (P / n_kv_heads)) * head_rows;
    if ((kv_local % 8) != 0) return NVFP4_E_SHAPE;
    nvfp4_tp_attn* a = new nvfp4_tp_attn();
    a->h = h; a->comm = comm; a->H = H; a->max_M = max_M;
    a->q_local = q_rows / P; a->kv_local = kv_local; a->o_local = o_in / P;
    a->Kp = (a->o_local + 255) / 256 * 256;
    a->qkv_gs = qkv_gs; a->o_gs = o_gs;
    const size_t rows = (size_t)a->q_local + 2 * (size_t)kv_local;
    const size_t prow = (size_t)H / 2, srow = (size_t)H / 16;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, bytes); };
    alloc((void**)&a->qkv_packed, rows * prow);
    alloc((void**)&a->qkv_scale, rows * srow);
    alloc((void**)&a->o_packed, (size_t)H * a->Kp / 2);
    alloc((void**)&a->o_scale, (size_t)H * a->Kp / 16);
    alloc(&a->act, (size_t)max_M * a->Kp * 2);
    alloc(&a->res_copy, (size_t)max_M * H * 2);
    if (e == cudaSuccess) e = cudaMemset(a->o_packed, 0, (size_t)H * a->Kp / 2);   // zero codes and zero scales
    if (e == cudaSuccess) e = cudaMemset(a->o_scale, 0, (size_t)H * a->Kp / 16);   // in the K padding
    if (e == cudaSuccess) e = cudaMemset(a->act, 0, (size_t)max_M * a->Kp * 2);
    // three contiguous row blocks of the merged tensor: q, k, v
    const size_t src_row[3] = {(size_t)r * a->q_local, (size_t)q_rows + kv_first, (size_t)q_rows + kv_rows + kv_first};
    const size_t n_rows[3] = {(size_t)a->q_local, (size_t)kv_local, (size_t)kv_local};
    size_t dst_row = 0;
    for (int b = 0; b < 3; ++b) {
        if (e == cudaSuccess) e = cudaMemcpy(a->qkv_packed + dst_row * prow, qkvp + src_row[b] * prow, n_rows[b] * prow, cudaMemcpyDeviceToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(a->qkv_scale + dst_row * srow, qkvs + src_row[b] * srow, n_rows[b] * srow, cudaMemcpyDeviceToDevice);
        dst_row += n_rows[b];
    }
    // output-projection columns [r o_local, (r+1) o_local) of every row, into rows of Kp elements
    if (e == cudaSuccess) e = cudaMemcpy2D(a->o_packed, (size_t)a->Kp / 2, op + (size_t)r * a->o_local / 2, (size_t)o_in / 2, (size_t)a->o_local / 2, H, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(a->o_scale, (size_t)a->Kp / 16, os + (size_t)r * a->o_local / 16, (size_t)o_in / 16, (size_t)a->o_local / 16, H, cudaMemcpyDeviceToDevice);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { nvfp4_tp_attn_destroy(a); return (int)e; }
    if (int st = nvfp4::tp::reserve_f32_partials(comm, max_M, H)) { nvfp4_tp_attn_destroy(a); return st; }
    *out = a;
    return NVFP4_OK;
}

int nvfp4_tp_attn_dims(nvfp4_tp_attn* a, int* q_local, int* kv_local, int* o_local) {
    if (!a) return NVFP4_E_NULL;
    if (q_local) *q_local = a->q_local;
    if (kv_local) *kv_local = a->kv_local;
    if (o_local) *o_local = a->o_local;
    return NVFP4_OK;
}

int nvfp4_tp_attn_shard_bytes(nvfp4_tp_attn* a, size_t* bytes) {
    if (!a || !bytes) return NVFP4_E_NULL;
    *bytes = ((size_t)a->q_local + 2 * (size_t)a->kv_local) * a->H * 9 / 16 + (size_t)a->H * a->Kp * 9 / 16;
    return NVFP4_OK;
}

int nvfp4_tp_attn_use_exchange(nvfp4_tp_attn* a, nvfp4_tp_exchange* x) {
    if (!a) return NVFP4_E_NULL;
    if (x && (x->H != a->H || x->comm->world != a->comm->world || x->comm->rank != a->comm->rank)) return NVFP4_E_SHAPE;
    a->x = x;
    return NVFP4_OK;
}

int nvfp4_tp_attn_set_fused(nvfp4_tp_attn* a, int on) {
    if (!a) return NVFP4_E_NULL;
    a->fused = on < 0 || on > 2 ? 1 : on;
    return NVFP4_OK;
}

int nvfp4_tp_attn_qkv(nvfp4_tp_attn* a, const void* X, int M, void* qkv_out, nvfp4_stream_t s) {
    if (!a || !X || !qkv_out) return NVFP4_E_NULL;
    if (M < 0 || M > a->max_M) return NVFP4_E_SHAPE;
    nvfp4::tp::SameGemvScope same_gemv(a->h, a->comm, a->x, a->fused, M);
    return nvfp4_linear(a->h, X, M, a->qkv_packed, a->qkv_scale, a->qkv_gs, a->q_local + 2 * a->kv_local, a->H, nullptr, qkv_out, s);
}

int nvfp4_tp_attn_out(nvfp4_tp_attn* a, const void* attn, long long row_stride, int M, const void* residual, void* out,
                      nvfp4_stream_t s) {
    if (!a || !attn || !out) return NVFP4_E_NULL;
    if (M < 0 || M > a->max_M || row_stride < 0 || (row_stride != 0 && row_stride < a->o_local)) return NVFP4_E_SHAPE;
    if (M == 0) return NVFP4_OK;
    if (row_stride == 0) row_stride = a->o_local;
    nvfp4::tp::SameGemvScope same_gemv(a->h, a->comm, a->x, a->fused, M);
    nvfp4_linear_desc d{};
    d.M = M;
    d.packed = a->o_packed; d.scale = a->o_scale; d.global_scale = a->o_gs; d.N = a->H; d.K = a->Kp;
    d.residual = residual; d.C = out;
    d.A = attn;
    if (row_stride == a->Kp && a->o_local == a->Kp)      // contiguous rows of the shard's own width: nothing to describe
        return nvfp4::tp::rowsplit_linear(a->h, a->comm, a->x, a->fused, d, a->res_copy, s);
    d.a_row_stride = row_stride;
    d.k_valid = a->o_local;
    int st = nvfp4::tp::rowsplit_linear(a->h, a->comm, a->x, a->fused, d, a->res_copy, s);
    if (st != NVFP4_E_LIMIT) return st;
    // the general kernels want plain [M, Kp] rows: copy (the pad columns of `act` stay zero)
    if (cudaMemcpy2DAsync(a->act, (size_t)a->Kp * 2, attn, (size_t)row_stride * 2, (size_t)a->o_local * 2, M,
                          cudaMemcpyDeviceToDevice, s) != cudaSuccess)
        return NVFP4_E_TP;
    d.A = a->act; d.a_row_stride = 0; d.k_valid = 0;
    return nvfp4::tp::rowsplit_linear(a->h, a->comm, a->x, a->fused, d, a->res_copy, s);
}

}  // extern "C"
