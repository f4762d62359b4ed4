/*
 * CPU oracle for the NVFP4 W4A16 linear layer.  TEST INFRASTRUCTURE ONLY:
 * the checker for the CUDA library and the timed CPU baseline.  See
 * nvfp4_oracle.h for the parity status and the reference lines followed.
 *
 * Build with IEEE semantics: -O2 -ffp-contract=off, never -ffast-math.
 */
#include "nvfp4_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* src/engine/dense_gemm_fp4_sm110.cu:24-27 (index 8 is +0.0f there too). */
static const float k_e2m1[16] = {
    0.0f,  0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f,
    0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

float nvfp4_oracle_e2m1(unsigned code) { return k_e2m1[code & 15u]; }

/* src/engine/dense_gemm_fp4_sm110.cu:30-41 */
float nvfp4_oracle_ue4m3(uint8_t v) {
    int exp = (v >> 3) & 0xF;
    int man = v & 0x7;
    if (exp == 0) return (float)man * 1.953125e-3f;
    float fval = 1.0f + (float)man * 0.125f;
    return ldexpf(fval, exp - 7);
}

uint16_t nvfp4_oracle_f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF; /* NaN, as __float2bfloat16 */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

float nvfp4_oracle_bf2f(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

uint8_t nvfp4_oracle_f2e4m3(float f) {
    float a = fabsf(f);
    if (!(a == a)) return 0x7E;
    if (a >= 448.0f) return 0x7E; /* 448 = 0x7E, the largest finite E4M3 */
    if (a < 0.015625f) {          /* below 2^-6: subnormal grid of 2^-9 */
        float q = a * 512.0f;
        float r = nearbyintf(q); /* default mode: ties to even */
        return (uint8_t)r;       /* r == 8 is 0x08 = 2^-6, the first normal */
    }
    int e;
    float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5,1) */
    float q = m * 16.0f;     /* [8,16) */
    float r = nearbyintf(q);
    if (r == 16.0f) { r = 8.0f; e += 1; }
    int exp = e - 1 + 7;
    int man = (int)r - 8;
    if (exp > 15 || (exp == 15 && man > 6)) return 0x7E;
    return (uint8_t)((exp << 3) | man);
}

/* src/engine/dense_gemm_fp4_sm110.cu:444-467; inv_gs computed on the host in
 * FP32 as at :554. */
void nvfp4_oracle_dequant_bf16(const uint8_t* packed, const uint8_t* scale,
                               float global_scale, int N, int K, uint16_t* out) {
    const float inv_gs = 1.0f / global_scale;
    const size_t kh = (size_t)K / 2, kg = (size_t)K / 16;
    for (int n = 0; n < N; ++n) {
        for (int k = 0; k < K; ++k) {
            uint8_t byte = packed[(size_t)n * kh + (size_t)k / 2];
            unsigned nib = (k & 1) ? (byte >> 4) & 0xFu : byte & 0xFu;
            float gs = nvfp4_oracle_ue4m3(scale[(size_t)n * kg + (size_t)k / 16]) * inv_gs;
            out[(size_t)n * K + k] = nvfp4_oracle_f2bf(k_e2m1[nib] * gs);
        }
    }
}

/* One output row, GEMV semantics (:96-141 for M=1, :192-240 batched): lane l of
 * a 32-lane warp takes groups l, l+32, ...; per group an FP32 dot of 16
 * products in byte order, then sum += group_dot * group_scale; lanes are
 * combined by the xor-butterfly (offsets 16,8,4,2,1). */
static float row_dot_gemv(const float* a, const uint8_t* w_row, const uint8_t* s_row,
                          float inv_gs, int K) {
    float lane[32];
    const int groups = K >> 4;
    for (int l = 0; l < 32; ++l) {
        float sum = 0.0f;
        for (int g = l; g < groups; g += 32) {
            float group_scale = nvfp4_oracle_ue4m3(s_row[g]) * inv_gs;
            const uint8_t* b = w_row + (size_t)g * 8;
            const float* ak = a + ((size_t)g << 4);
            float group_dot = 0.0f;
            for (int j = 0; j < 8; ++j) {
                float t = ak[2 * j] * k_e2m1[b[j] & 0xF] + ak[2 * j + 1] * k_e2m1[b[j] >> 4];
                group_dot += t;
            }
            sum += group_dot * group_scale;
        }
        lane[l] = sum;
    }
    for (int mask = 16; mask > 0; mask >>= 1) {
        float nxt[32];
        for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ mask];
        memcpy(lane, nxt, sizeof lane);
    }
    return lane[0];
}

/* One output row, GEMM semantics (:558-583): weights rounded to BF16 by the
 * dequant formula first, then an FP32 dot (the library's summation order is
 * not specified; sequential k here). */
static float row_dot_gemm(const float* a, const float* wq, int K) {
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) acc += a[k] * wq[k];
    return acc;
}

void nvfp4_oracle_linear_rows(const uint16_t* A, int M, const uint8_t* packed,
                              const uint8_t* scale, float global_scale, int N, int K,
                              const uint16_t* residual, uint16_t* C, int mode,
                              int n0, int n1) {
    if (mode == NVFP4_ORACLE_AUTO) mode = (M <= 8) ? NVFP4_ORACLE_GEMV : NVFP4_ORACLE_GEMM;
    const float inv_gs = 1.0f / global_scale;
    const size_t kh = (size_t)K / 2, kg = (size_t)K / 16;
    float* af = (float*)malloc((size_t)M * K * sizeof(float));
    float* wq = (float*)malloc((size_t)K * sizeof(float));
    for (size_t i = 0; i < (size_t)M * K; ++i) af[i] = nvfp4_oracle_bf2f(A[i]);
    for (int n = n0; n < n1; ++n) {
        const uint8_t* w_row = packed + (size_t)n * kh;
        const uint8_t* s_row = scale + (size_t)n * kg;
        if (mode == NVFP4_ORACLE_GEMM) {
            for (int k = 0; k < K; ++k) {
                uint8_t byte = w_row[k >> 1];
                unsigned nib = (k & 1) ? (byte >> 4) & 0xFu : byte & 0xFu;
                float gs = nvfp4_oracle_ue4m3(s_row[k >> 4]) * inv_gs;
                wq[k] = nvfp4_oracle_bf2f(nvfp4_oracle_f2bf(k_e2m1[nib] * gs));
            }
        }
        for (int m = 0; m < M; ++m) {
            const float* a = af + (size_t)m * K;
            float v = (mode == NVFP4_ORACLE_GEMM) ? row_dot_gemm(a, wq, K)
                                                  : row_dot_gemv(a, w_row, s_row, inv_gs, K);
            if (residual) v += nvfp4_oracle_bf2f(residual[(size_t)m * N + n]);
            C[(size_t)m * N + n] = nvfp4_oracle_f2bf(v);
        }
    }
    free(wq);
    free(af);
}

void nvfp4_oracle_linear(const uint16_t* A, int M, const uint8_t* packed,
                         const uint8_t* scale, float global_scale, int N, int K,
                         const uint16_t* residual, uint16_t* C, int mode) {
    nvfp4_oracle_linear_rows(A, M, packed, scale, global_scale, N, K, residual, C, mode, 0, N);
}

typedef struct {
    const uint16_t* A; int M; const uint8_t* packed; const uint8_t* scale; float gs;
    int N, K; const uint16_t* residual; uint16_t* C; int mode; int n0, n1;
} row_job;

static void* row_worker(void* p) {
    row_job* j = (row_job*)p;
    nvfp4_oracle_linear_rows(j->A, j->M, j->packed, j->scale, j->gs, j->N, j->K,
                             j->residual, j->C, j->mode, j->n0, j->n1);
    return NULL;
}

void nvfp4_oracle_linear_mt(const uint16_t* A, int M, const uint8_t* packed,
                            const uint8_t* scale, float global_scale, int N, int K,
                            const uint16_t* residual, uint16_t* C, int mode, int threads) {
    if (threads <= 1) {
        nvfp4_oracle_linear(A, M, packed, scale, global_scale, N, K, residual, C, mode);
        return;
    }
    if (mode == NVFP4_ORACLE_AUTO) mode = (M <= 8) ? NVFP4_ORACLE_GEMV : NVFP4_ORACLE_GEMM;
    if (threads > N) threads = N;
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    row_job* jobs = (row_job*)malloc(sizeof(row_job) * (size_t)threads);
    for (int t = 0; t < threads; ++t) {
        row_job j = {A, M, packed, scale, global_scale, N, K, residual, C, mode,
                     (int)((long long)N * t / threads), (int)((long long)N * (t + 1) / threads)};
        jobs[t] = j;
        pthread_create(&th[t], NULL, row_worker, &jobs[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(th[t], NULL);
    free(jobs);
    free(th);
}

/* src/engine/light_ops.cu:168-170 */
static float silu(float x) { return x / (1.0f + expf(-x)); }

void nvfp4_oracle_swiglu(const uint16_t* gate, const uint16_t* up, size_t n, uint16_t* out) {
    for (size_t i = 0; i < n; ++i) {
        float g = nvfp4_oracle_bf2f(gate[i]), u = nvfp4_oracle_bf2f(up[i]);
        out[i] = nvfp4_oracle_f2bf(silu(g) * u);
    }
}

void nvfp4_oracle_swiglu_merged(const uint16_t* merged, int T, int I, uint16_t* out) {
    for (int t = 0; t < T; ++t)
        nvfp4_oracle_swiglu(merged + (size_t)t * 2 * I, merged + (size_t)t * 2 * I + I,
                            (size_t)I, out + (size_t)t * I);
}

/* src/engine/dense_gemm.h:64-95 */
void nvfp4_oracle_dense_linear(const uint16_t* A, int M, const uint16_t* W, int N, int K,
                               const uint16_t* residual, uint16_t* C) {
    float* a = (float*)malloc((size_t)K * sizeof(float));
    for (int m = 0; m < M; ++m) {
        for (int k = 0; k < K; ++k) a[k] = nvfp4_oracle_bf2f(A[(size_t)m * K + k]);
        for (int n = 0; n < N; ++n) {
            const uint16_t* w = W + (size_t)n * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += a[k] * nvfp4_oracle_bf2f(w[k]);
            if (residual) acc += nvfp4_oracle_bf2f(residual[(size_t)m * N + n]);
            C[(size_t)m * N + n] = nvfp4_oracle_f2bf(acc);
        }
    }
    free(a);
}

/* The reference's BF16 GEMV for one token, in ITS summation order (src/engine/dense_gemm_sm110.cu:
 * gemv_kernel :544-604, gemv_kernel_scattered :682-735, the K-tiled variants :612-668 and their
 * "+ residual" twins :811-1033, dispatched by invoke_dense_gemv / _add :1140-1216).  One warp per
 * output row; lane l walks the 8-element chunks l, l+32, ... and adds, per pair of elements,
 * rn(a0*w0 + a1*w1) to its FP32 sum (products of two BF16 are exact in FP32, so fused or not the pair
 * sum is the same); elements beyond the last whole chunk go one by one to lane (k mod 32); the 32 sums
 * meet in an xor-shuffle tree (16, 8, 4, 2, 1); the residual is added in FP32 before the one rounding.
 * Every variant of the family keeps this order (the tile length is a multiple of 256). */
void nvfp4_oracle_dense_gemv_ref(const uint16_t* A, const uint16_t* W, int N, int K, const uint16_t* residual,
                                 uint16_t* C) {
    float* a = (float*)malloc((size_t)K * sizeof(float));
    for (int k = 0; k < K; ++k) a[k] = nvfp4_oracle_bf2f(A[k]);
    const int k8 = K / 8;
    for (int n = 0; n < N; ++n) {
        const uint16_t* w = W + (size_t)n * K;
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float sum = 0.0f;
            for (int i = l; i < k8; i += 32)
                for (int j = 0; j < 4; ++j) {
                    const int k = 8 * i + 2 * j;
                    const float pair = a[k] * nvfp4_oracle_bf2f(w[k]) + a[k + 1] * nvfp4_oracle_bf2f(w[k + 1]);
                    sum += pair;
                }
            for (int k = 8 * k8 + l; k < K; k += 32) sum += a[k] * nvfp4_oracle_bf2f(w[k]);
            lane[l] = sum;
        }
        for (int mask = 16; mask > 0; mask >>= 1) {
            float next[32];
            for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ mask];
            memcpy(lane, next, sizeof(lane));
        }
        float out = lane[0];
        if (residual) out = out + nvfp4_oracle_bf2f(residual[n]);
        C[n] = nvfp4_oracle_f2bf(out);
    }
    free(a);
}

/* src/engine/light_ops.cu:30-57 (blockReduceSum with 256 threads) over per-thread partial sums */
static float block_reduce_256(float* v) {
    float w[8];
    for (int wid = 0; wid < 8; ++wid) {
        float* l = v + 32 * wid;
        for (int off = 16; off > 0; off >>= 1)
            for (int lane = 0; lane + off < 32; ++lane) l[lane] += l[lane + off];   /* lane reads the old value of lane+off: ascending order keeps it old */
        w[wid] = l[0];
    }
    float l[32];
    for (int lane = 0; lane < 32; ++lane) l[lane] = lane < 8 ? w[lane] : 0.0f;
    for (int off = 16; off > 0; off >>= 1)
        for (int lane = 0; lane + off < 32; ++lane) l[lane] += l[lane + off];
    return l[0];
}

/* src/engine/light_ops.cu:65-106 and :270-318 */
void nvfp4_oracle_rmsnorm(const uint16_t* x, const uint16_t* bias, const uint16_t* weight, float eps,
                          int M, int K, uint16_t* out, uint16_t* residual_out) {
    float* r = (float*)malloc((size_t)K * sizeof(float));
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = x + (size_t)m * K;
        float part[256];
        for (int t = 0; t < 256; ++t) part[t] = 0.0f;
        for (int i = 0; i < K; ++i) {
            float v = nvfp4_oracle_bf2f(xr[i]);
            if (bias) v = v + nvfp4_oracle_bf2f(bias[(size_t)m * K + i]);
            r[i] = v;
        }
        for (int t = 0; t < 256; ++t)
            for (int i = t; i < K; i += 256) part[t] = fmaf(r[i], r[i], part[t]);
        const float sum_sq = block_reduce_256(part);
        const float inv_rms = 1.0f / sqrtf(sum_sq / (float)K + eps);
        for (int i = 0; i < K; ++i) {
            if (bias && residual_out) residual_out[(size_t)m * K + i] = nvfp4_oracle_f2bf(r[i]);
            const float w = nvfp4_oracle_bf2f(weight[i]);
            out[(size_t)m * K + i] = nvfp4_oracle_f2bf(r[i] * inv_rms * (1.0f + w));
        }
    }
    free(r);
}

void nvfp4_oracle_mlp(const uint16_t* X, int M, int H, int I,
                      const uint8_t* gu_packed, const uint8_t* gu_scale, float gu_gs,
                      const uint8_t* dn_packed, const uint8_t* dn_scale, float dn_gs,
                      const uint16_t* residual, uint16_t* out, int mode, int threads) {
    uint16_t* gu = (uint16_t*)malloc((size_t)M * 2 * I * 2);
    uint16_t* act = (uint16_t*)malloc((size_t)M * I * 2);
    nvfp4_oracle_linear_mt(X, M, gu_packed, gu_scale, gu_gs, 2 * I, H, NULL, gu, mode, threads);
    nvfp4_oracle_swiglu_merged(gu, M, I, act);
    nvfp4_oracle_linear_mt(act, M, dn_packed, dn_scale, dn_gs, H, I, residual, out, mode, threads);
    free(act);
    free(gu);
}

/* FP32 dot of one token row against columns [k0,k1) of one down-projection
 * row, with the semantics selected by `mode` restricted to that K slice. */
static float slice_dot(const float* a, const uint8_t* w_row, const uint8_t* s_row,
                       float inv_gs, int k0, int k1, int mode, float* wq) {
    if (mode == NVFP4_ORACLE_GEMM) {
        for (int k = k0; k < k1; ++k) {
            uint8_t byte = w_row[k >> 1];
            unsigned nib = (k & 1) ? (byte >> 4) & 0xFu : byte & 0xFu;
            float gs = nvfp4_oracle_ue4m3(s_row[k >> 4]) * inv_gs;
            wq[k - k0] = nvfp4_oracle_bf2f(nvfp4_oracle_f2bf(k_e2m1[nib] * gs));
        }
        return row_dot_gemm(a + k0, wq, k1 - k0);
    }
    return row_dot_gemv(a + k0, w_row + (k0 >> 1), s_row + (k0 >> 4), inv_gs, k1 - k0);
}

void nvfp4_oracle_tp_mlp(const uint16_t* X, int M, int H, int I, int P,
                         const uint8_t* gu_packed, const uint8_t* gu_scale, float gu_gs,
                         const uint8_t* dn_packed, const uint8_t* dn_scale, float dn_gs,
                         const uint16_t* residual, uint16_t* out, int mode,
                         int partial_bf16, int threads) {
    if (mode == NVFP4_ORACLE_AUTO) mode = (M <= 8) ? NVFP4_ORACLE_GEMV : NVFP4_ORACLE_GEMM;
    if (P == 1) partial_bf16 = 0; /* a single rank exchanges nothing: no intermediate rounding */
    /* Column-split gate/up never changes a single output value, so the full
     * gate_up linear + SwiGLU is computed once; only the down projection's K
     * split changes the arithmetic. */
    uint16_t* gu = (uint16_t*)malloc((size_t)M * 2 * I * 2);
    uint16_t* act = (uint16_t*)malloc((size_t)M * I * 2);
    nvfp4_oracle_linear_mt(X, M, gu_packed, gu_scale, gu_gs, 2 * I, H, NULL, gu, mode, threads);
    nvfp4_oracle_swiglu_merged(gu, M, I, act);
    float* af = (float*)malloc((size_t)M * I * sizeof(float));
    float* wq = (float*)malloc((size_t)I * sizeof(float));
    for (size_t i = 0; i < (size_t)M * I; ++i) af[i] = nvfp4_oracle_bf2f(act[i]);
    const float inv_gs = 1.0f / dn_gs;
    const int Ip = I / P;
    for (int n = 0; n < H; ++n) {
        const uint8_t* w_row = dn_packed + (size_t)n * (I / 2);
        const uint8_t* s_row = dn_scale + (size_t)n * (I / 16);
        for (int m = 0; m < M; ++m) {
            float total = 0.0f;
            for (int r = 0; r < P; ++r) {
                float part = slice_dot(af + (size_t)m * I, w_row, s_row, inv_gs,
                                       r * Ip, (r + 1) * Ip, mode, wq);
                if (partial_bf16) part = nvfp4_oracle_bf2f(nvfp4_oracle_f2bf(part));
                total += part;
            }
            if (residual) total += nvfp4_oracle_bf2f(residual[(size_t)m * H + n]);
            out[(size_t)m * H + n] = nvfp4_oracle_f2bf(total);
        }
    }
    free(wq);
    free(af);
    free(act);
    free(gu);
}

double nvfp4_oracle_rel_frobenius(const uint16_t* a, const uint16_t* b, size_t n) {
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < n; ++i) {
        double x = nvfp4_oracle_bf2f(a[i]), y = nvfp4_oracle_bf2f(b[i]);
        num += (x - y) * (x - y);
        den += y * y;
    }
    if (den == 0.0) return num == 0.0 ? 0.0 : INFINITY;
    return sqrt(num / den);
}
