/*
 * nvfp4_b200_tp — tensor-parallel NVFP4 MLP across the GPUs of one node (one process per GPU).
 *
 * New work: the reference engine is single-GPU (its link line carries no communication
 * library).  The block reproduces the reference's MLP sequence (run_mlp,
 * src/engine/layer.cu:62-110: merged gate/up linear -> SwiGLU -> down linear + residual) with
 * the Megatron split: gate/up by output rows (no exchange), down by K columns, ONE sum
 * all-reduce of the [M, H] down-projection partials: NCCL (BF16) in general, a fused
 * push-and-sum kernel over peer memory (FP32, rank order) for up to 16 tokens.
 * Rank r owns gate rows and up rows [r*I/P, (r+1)*I/P) and down columns [r*I/P, (r+1)*I/P);
 * a shard is a pure slice of the reference layout (no re-quantisation); the down shard's K is
 * zero-padded to a multiple of 256 so that its scale rows stay 16-byte multiples.
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

#define NVFP4_TP_UNIQUE_ID_BYTES 128
#define NVFP4_TP_P2P_HANDLE_BYTES 64
#define NVFP4_TP_MAX_WORLD 8

/* Rank 0 makes the id (ncclGetUniqueId) and ships the 128 bytes to the other ranks by any
 * means (the benchmark uses a torch.distributed broadcast). */
int nvfp4_tp_unique_id(void* out_128_bytes);
/* Collective over all ranks: ncclCommInitRank on the current device.  world == 1 needs no id. */
int nvfp4_tp_comm_create(const void* unique_id_128_bytes, int rank, int world, nvfp4_tp_comm** out);
int nvfp4_tp_comm_destroy(nvfp4_tp_comm* comm);

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

#ifdef __cplusplus
}
#endif
#endif
