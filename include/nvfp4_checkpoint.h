/*
 * nvfp4_checkpoint — host-side ingestion of NVFP4 ("compressed-tensors nvfp4-pack-quantized")
 * checkpoints for the nvfp4_b200 kernels: a safetensors reader, the row-concatenating merges the
 * reference performs at load time, the tensor-parallel shard rule, and a safetensors writer for
 * the offline shard tool.  Host memory only; no CUDA.  Library: libnvfp4_ckpt.so.
 *
 * Replaces, for the FP4 tensors, the reference's loader path:
 *   src/engine/safetensors.cpp:60-128   header parsing (8-byte length + JSON + raw data)
 *   src/engine/model.cpp:70-79          U8 / F8_E4M3 / F32 "*_global_scale" classification
 *   src/engine/model.cpp:213-232        <prefix>.weight_packed / .weight_scale /
 *                                       .weight_global_scale / .input_global_scale -> QuantizedWeight
 *   src/engine/model.cpp:296-350,456-514  QKV and gate+up merges: plain row concatenation of the
 *                                       packed and the scale tensors, global scale of the first part
 * The tensor-parallel shard rule has no reference counterpart (the reference is single-GPU); it
 * is the rule nvfp4_tp_mlp_create applies on the device (include/nvfp4_b200_tp.h).
 *
 * Every function returns 0 or a negative NVFP4_CKPT_E_* code.
 */
#ifndef NVFP4_CHECKPOINT_H
#define NVFP4_CHECKPOINT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_CKPT_OK 0
#define NVFP4_CKPT_E_NULL (-1)
#define NVFP4_CKPT_E_IO (-2)        /* cannot open / map / write the file */
#define NVFP4_CKPT_E_FORMAT (-3)    /* not a well-formed safetensors file */
#define NVFP4_CKPT_E_MISSING (-4)   /* no tensor of that name */
#define NVFP4_CKPT_E_TYPE (-5)      /* tensor present but of the wrong dtype or rank */
#define NVFP4_CKPT_E_SHAPE (-6)     /* shapes of packed / scale / parts do not agree */
#define NVFP4_CKPT_E_SCALE (-7)     /* parts of a merge carry different global scales */

typedef struct nvfp4_ckpt nvfp4_ckpt;

typedef struct nvfp4_ckpt_tensor {
    const void* data;     /* into the read-only mapping; valid until nvfp4_ckpt_close */
    size_t nbytes;
    char dtype[16];       /* as in the file: "U8", "F8_E4M3", "F32", "BF16", ... */
    int rank;
    long long shape[8];
} nvfp4_ckpt_tensor;

/* One quantised linear on the host, in the reference's layout (src/engine/layer.h:197-204):
 * packed [N, K/2] (low nibble = even k), scale [N, K/16] unsigned E4M3, W = e2m1 * ue4m3 / global_scale. */
typedef struct nvfp4_host_weight {
    const uint8_t* packed;
    const uint8_t* scale;
    float global_scale;
    float input_scale;    /* 0 when the checkpoint has none; unused by W4A16 */
    int N, K;
} nvfp4_host_weight;

int nvfp4_ckpt_open(const char* path, nvfp4_ckpt** out);
int nvfp4_ckpt_close(nvfp4_ckpt* c);
int nvfp4_ckpt_count(const nvfp4_ckpt* c);
const char* nvfp4_ckpt_name(const nvfp4_ckpt* c, int index);       /* NULL when out of range */
int nvfp4_ckpt_get(const nvfp4_ckpt* c, const char* name, nvfp4_ckpt_tensor* out);

/* <prefix>.weight_packed (U8, [N, K/2]), <prefix>.weight_scale (F8_E4M3 or U8, [N, K/16]),
 * <prefix>.weight_global_scale (F32, one element), optional <prefix>.input_global_scale. */
int nvfp4_ckpt_linear(const nvfp4_ckpt* c, const char* prefix, nvfp4_host_weight* out);

/* Row concatenation of n parts with equal K (QKV, gate+up): packed_out [sum N, K/2], scale_out
 * [sum N, K/16].  The parts must carry the same global scale (the reference silently takes the
 * first part's; a mismatch would dequantise the other parts wrongly, so it is an error here). */
int nvfp4_merge_rows(const nvfp4_host_weight* parts, int n, uint8_t* packed_out, uint8_t* scale_out,
                     nvfp4_host_weight* merged);
/* The same with the reference's rule as an option: take_first_scale != 0 accepts parts with different
 * global scales and gives the merged tensor the first part's (src/engine/model.cpp:329 for QKV, :492
 * for gate+up), so a checkpoint the reference loads is loaded the same way, wrong rows included. */
int nvfp4_merge_rows_ex(const nvfp4_host_weight* parts, int n, uint8_t* packed_out, uint8_t* scale_out,
                        nvfp4_host_weight* merged, int take_first_scale);

/* Merged gate/up [2I, H] (gate rows, then up rows) -> rows interleaved in slabs of 16: rows 16s..16s+7 =
 * gate rows 8s..8s+7, rows 16s+8..16s+15 = up rows 8s..8s+7.  That is the layout the swiglu_epilogue form
 * of nvfp4_linear_ex reads: a thread of the GEMV kernel then holds a gate value and its up value.
 * I % 8 == 0; works on a shard of nvfp4_tp_shard_gate_up as well. */
int nvfp4_interleave_gate_up(const nvfp4_host_weight* merged, uint8_t* packed_out, uint8_t* scale_out,
                             nvfp4_host_weight* out);

/* Tensor-parallel shards of the MLP, rank r of `world`:
 *   gate_up: merged [2I, H] -> gate rows and up rows [r*I/P, (r+1)*I/P), merged again [2I/P, H];
 *   down:    [H, I] -> K columns [r*I/P, (r+1)*I/P), K zero-padded (zero codes, zero scales) to a
 *            multiple of 256 so that scale rows stay 16-byte multiples.
 * I % (16 * world) == 0.  The *_bytes functions give the output sizes; *K_padded the shard's K. */
int nvfp4_tp_shard_gate_up(const nvfp4_host_weight* merged, int rank, int world, uint8_t* packed_out, uint8_t* scale_out,
                           nvfp4_host_weight* shard);
int nvfp4_tp_shard_down(const nvfp4_host_weight* down, int rank, int world, uint8_t* packed_out, uint8_t* scale_out,
                        nvfp4_host_weight* shard);
/* Attention side: merged QKV [q_rows + 2*kv_rows, H] (q rows, k rows, v rows) -> rank r's q rows
 * [r*q_rows/P, (r+1)*q_rows/P) and the k and v rows of its KV heads (n_kv_heads % P == 0), or of KV
 * head r / (P / n_kv_heads) when the ranks outnumber the KV heads (P % n_kv_heads == 0): shard
 * [q_rows/P + 2*kv_local, H].  The output projection [H, o_in] splits by K like the down projection
 * (nvfp4_tp_shard_down).  q_rows % (8 * world) == 0. */
int nvfp4_tp_shard_qkv(const nvfp4_host_weight* merged, int q_rows, int kv_rows, int n_kv_heads, int rank, int world,
                       uint8_t* packed_out, uint8_t* scale_out, nvfp4_host_weight* shard);
int nvfp4_tp_shard_qkv_rows(int q_rows, int kv_rows, int n_kv_heads, int world);   /* rows of a QKV shard, or < 0 */
int nvfp4_tp_shard_down_k(int I, int world);                       /* padded K of a down shard, or < 0 */

/* Minimal safetensors writer: n tensors, names[i], tensors[i] (data, nbytes, dtype, rank, shape). */
int nvfp4_ckpt_write(const char* path, const char* const* names, const nvfp4_ckpt_tensor* tensors, int n);

const char* nvfp4_ckpt_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif
