/*
 * nvfp4_b200_tp — tensor-parallel NVFP4 MLP and attention projections across the GPUs of one
 * node (one process per GPU).
 *
 * New work: the reference engine is single-GPU (its link line carries no communication
 * library).  The block reproduces the reference's MLP sequence (run_mlp,
 * src/engine/layer.cu:62-110: merged gate/up linear -> SwiGLU -> down linear + residual) with
 * the Megatron split: gate/up by output rows (no exchange), down by K columns, ONE sum
 * all-reduce of the [M, H] down-projection partials: NCCL (BF16) in general, a fused
 * push-and-sum kernel over peer memory (FP32, rank order) for up to 16 tokens.
 * Rank r owns gate rows and up rows [r*I/P, (r+1)*I/P) and down columns [r*I/P, (r+1)*I/P);
 * a shard is a pure slice of the reference layout (no re-quantisation); the down shard's K is
 * zero-padded to a multiple of 256 so that its scale rows stay 16-byte multiples, and the block's
 * own copy of the gate/up shard has its rows interleaved in slabs of 16 (8 gate rows, their 8 up
 * rows) so that up to 16 tokens get their SwiGLU in the gate_up kernel's epilogue.
 * Library: libnvfp4_b200_tp.so (needs libnvfp4_b200.so and libnccl.so.2).
 */
#ifndef NVFP4_B200_TP_H
#define NVFP4_B200_TP_H

#include "nvfp4_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nvfp4_tp_comm nvfp4_tp_comm;
typedef struct nvfp4_tp_mlp nvfp4_tp_mlp;
typedef struct nvfp4_tp_attn nvfp4_tp_attn;
typedef struct nvfp4_tp_exchange nvfp4_tp_exchange;

#define NVFP4_TP_UNIQUE_ID_BYTES 128
#define NVFP4_TP_P2P_HANDLE_BYTES 64
#define NVFP4_TP_MAX_WORLD 8

/* Rank 0 makes the id (ncclGetUniqueId) and ships the 128 bytes to the other ranks by any
 * means (the benchmark uses a torch.distributed broadcast). */
int nvfp4_tp_unique_id(void* out_128_bytes);
/* Collective over all ranks: ncclCommInitRankConfig on the current device with a NON-BLOCKING
 * communicator.  Every library call on it (the set-up itself, the collectives of the forward
 * calls, the finalize in destroy) may come back "in progress"; the library then polls
 * ncclCommGetAsyncError until the call settles or the deadline (default 30 s) has passed.  After
 * an error or the deadline it aborts the communicator (ncclCommAbort) and returns NVFP4_E_TP, as
 * does every later call that needs it.  So a rank that never shows up costs the others the
 * deadline, not a process stuck inside the library.  (The reference's analogue, for its one GPU:
 * sync_stream_with_timeout, src/engine/engine.cpp:38-61.)  world == 1 needs no id. */
int nvfp4_tp_comm_create(const void* unique_id_128_bytes, int rank, int world, nvfp4_tp_comm** out);
int nvfp4_tp_comm_destroy(nvfp4_tp_comm* comm);
int nvfp4_tp_comm_set_deadline_ms(nvfp4_tp_comm* comm, int milliseconds);
/* For a caller's watchdog.  state: 0 = idle or healthy, 1 = a call is in progress, -1 = failed or aborted. */
int nvfp4_tp_comm_state(nvfp4_tp_comm* comm, int* state);
/* Gives the communicator up without waiting for the peers (ncclCommAbort); the blocks built on it return
 * NVFP4_E_TP from then on wherever they would need it. */
int nvfp4_tp_comm_abort(nvfp4_tp_comm* comm);
/* How the partial sums travel where the library collective adds them (more than 16 tokens, or no
 * attached exchange).  Default (0): unrounded FP32 partials -- ncclReduceScatter(FP32), the residual
 * added and the result rounded once on each rank's slice, ncclAllGather(BF16): within 1e-3 of the
 * unsplit layer at any group size.  1: the partials are rounded to BF16 first and summed by one
 * ncclAllReduce(BF16), half the bytes on the wire but one rounding per rank in front of the sum
 * (about 1.1e-3 / 1.4e-3 from the unsplit layer at 4 / 8 ranks).  Same value on every rank. */
int nvfp4_tp_comm_set_bf16_partials(nvfp4_tp_comm* comm, int on);

/* Builds this rank's shards from the FULL device-resident tensors (gate_up [2I, H] merged gate
 * rows then up rows, down [H, I]) and allocates the intermediate buffers for up to max_M
 * tokens.  The full tensors may be freed afterwards.  H % 256 == 0, I % (16 * world) == 0. */
int nvfp4_tp_mlp_create(nvfp4_handle* h, nvfp4_tp_comm* comm, int H, int I,
                        const uint8_t* gate_up_packed, const uint8_t* gate_up_scale, float gate_up_global_scale,
                        const uint8_t* down_packed, const uint8_t* down_scale, float down_global_scale,
                        int max_M, nvfp4_tp_mlp** out);
int nvfp4_tp_mlp_destroy(nvfp4_tp_mlp* mlp);

/* out[M,H] = down( swiglu( gate_up(X) ) ) (+ residual), identical on every rank after the
 * all-reduce.  X, residual, out: BF16 device pointers, replicated on every rank; residual may
 * be NULL and may alias out.  Asynchronous on `stream`. */
int nvfp4_tp_mlp_forward(nvfp4_tp_mlp* mlp, const void* X_bf16, int M, const void* residual_bf16_or_null,
                         void* out_bf16, nvfp4_stream_t stream);

/* Fused reduction for M <= 16 (the decode regime) in place of the library collective: every
 * rank exports the 64-byte handle of its exchange buffer (cudaIpcGetMemHandle), the host ships
 * all of them to every rank (rank order, world x 64 bytes; any transport), every rank attaches
 * (cudaIpcOpenMemHandle; needs peer access, i.e. NVLink or PCIe P2P between the GPUs).  After
 * that nvfp4_tp_mlp_forward's down projection pushes its FP32 sums to all peers with plain
 * stores, waits (bounded: about a second, then the status word below becomes non-zero and that
 * part of `out` is left unwritten) for theirs and adds them in rank order in FP32 with the
 * residual, all in one kernel.  world == 1 may attach with NULL.
 * nvfp4_tp_mlp_set_fused(mlp, 0) returns to the NCCL path; 1 (default once attached) fuses the
 * push and the reduction into the down-projection kernel itself (nvfp4_linear_reduce_peers);
 * 2 runs them as a separate kernel behind an FP32 down projection.  All ranks must make the same
 * sequence of forward calls (same M), as with any collective. */
int nvfp4_tp_mlp_p2p_handle(nvfp4_tp_mlp* mlp, void* out_64_bytes);
int nvfp4_tp_mlp_p2p_attach(nvfp4_tp_mlp* mlp, const void* handles_world_x_64_bytes);
int nvfp4_tp_mlp_set_fused(nvfp4_tp_mlp* mlp, int on);
/* Synchronises the device and reads the exchange kernel's sticky status (0 = every wait was met). */
int nvfp4_tp_mlp_status(nvfp4_tp_mlp* mlp, unsigned int* status);

/* Bytes this rank streams per forward (its weight shards incl. padding). */
int nvfp4_tp_mlp_shard_bytes(nvfp4_tp_mlp* mlp, size_t* bytes);

/* The peer exchange as an object of its own: one per rank serves every block whose output is
 * [M, H] (the MLP blocks and the attention blocks of all layers), as long as all ranks call the
 * blocks in the same order -- the two slot sets alternate per reduction, whichever block runs
 * it.  handle / attach / status as for nvfp4_tp_mlp_p2p_* above (collective: every rank attaches
 * the handles of all ranks, in rank order).  The exchange must outlive the blocks that use it. */
int nvfp4_tp_exchange_create(nvfp4_tp_comm* comm, int H, nvfp4_tp_exchange** out);
int nvfp4_tp_exchange_destroy(nvfp4_tp_exchange* x);
int nvfp4_tp_exchange_handle(nvfp4_tp_exchange* x, void* out_64_bytes);
int nvfp4_tp_exchange_attach(nvfp4_tp_exchange* x, const void* handles_world_x_64_bytes);
int nvfp4_tp_exchange_status(nvfp4_tp_exchange* x, unsigned int* status);
/* The MLP block reduces through `x` instead of its own exchange (NULL: back to its own). */
int nvfp4_tp_mlp_use_exchange(nvfp4_tp_mlp* mlp, nvfp4_tp_exchange* x);

/* Attention-side projections as a tensor-parallel block.  New work like the MLP block; the
 * single-GPU sequence it splits is src/engine/layer.cu:190-217 (merged FP4 QKV projection) and
 * :404-409 (output projection).  The merged QKV tensor [q_rows + 2*kv_rows, H] (q rows, k rows,
 * v rows) is split by output rows in whole KV-head groups: rank r owns q rows
 * [r*q_rows/P, (r+1)*q_rows/P) and the k and v rows of its KV heads (n_kv_heads % P == 0), or,
 * with more ranks than KV heads (P % n_kv_heads == 0), of KV head r / (P / n_kv_heads).  The
 * output projection [H, o_in] is split by K columns [r*o_in/P, (r+1)*o_in/P); its partial sums
 * are added over the ranks exactly as the MLP's down projection (inside the GEMV kernel for
 * M <= 16 once nvfp4_tp_attn_use_exchange gave it an attached exchange, NCCL otherwise).
 * Built from the FULL device-resident tensors, which may be freed afterwards.
 * H % 256 == 0, q_rows % (8*P) == 0, o_in % (16*P) == 0. */
int nvfp4_tp_attn_create(nvfp4_handle* h, nvfp4_tp_comm* comm, int H, int q_rows, int kv_rows, int n_kv_heads, int o_in,
                         const uint8_t* qkv_packed, const uint8_t* qkv_scale, float qkv_global_scale,
                         const uint8_t* o_packed, const uint8_t* o_scale, float o_global_scale,
                         int max_M, nvfp4_tp_attn** out);
int nvfp4_tp_attn_destroy(nvfp4_tp_attn* attn);
/* This rank's widths: q rows, k rows (= v rows), output-projection input columns. */
int nvfp4_tp_attn_dims(nvfp4_tp_attn* attn, int* q_local, int* kv_local, int* o_local);
int nvfp4_tp_attn_shard_bytes(nvfp4_tp_attn* attn, size_t* bytes);
int nvfp4_tp_attn_use_exchange(nvfp4_tp_attn* attn, nvfp4_tp_exchange* x);
int nvfp4_tp_attn_set_fused(nvfp4_tp_attn* attn, int mode);   /* 0, 1, 2 as nvfp4_tp_mlp_set_fused */
/* qkv_out[M, q_local + 2*kv_local] = X[M,H] * shard^T: this rank's q | k | v, no exchange. */
int nvfp4_tp_attn_qkv(nvfp4_tp_attn* attn, const void* X_bf16, int M, void* qkv_out_bf16, nvfp4_stream_t stream);
/* out[M,H] = sum over ranks of attn_r[M, o_local] * o_shard_r^T (+ residual), identical on every
 * rank.  attn rows are row_stride elements apart (0 = o_local; a multiple of 8): the attention
 * output may be read in place from a wider buffer.  residual may be NULL and may alias out. */
int nvfp4_tp_attn_out(nvfp4_tp_attn* attn, const void* attn_bf16, long long row_stride, int M,
                      const void* residual_bf16_or_null, void* out_bf16, nvfp4_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
