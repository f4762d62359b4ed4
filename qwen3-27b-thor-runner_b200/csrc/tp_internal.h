// Shared between the tensor-parallel blocks (tp_common.cu, tp_mlp.cu, tp_attn.cu): the
// communicator, the peer-exchange object of the fused small-M reduction, and the row-split linear
// (K columns split over the ranks, partial sums added over the group) both blocks end with.
#pragma once
#include <cuda_runtime.h>
#include <nccl.h>

#include "../../include/nvfp4_b200_tp.h"
#include "exchange_layout.h"

struct nvfp4_tp_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    // NCCL path of the row-split linear: FP32 partial sums [M, H] of the largest block created on this
    // communicator (reduce-scattered in FP32, finished per slice, all-gathered as BF16); with
    // bf16_partials the older form, one all-reduce of BF16-rounded partials, is used instead.
    float* f32_scratch = nullptr;
    size_t f32_bytes = 0;
    int bf16_partials = 0;
    // The communicator is non-blocking: a call may come back as "in progress", and the caller polls the
    // communicator's asynchronous state until it settles or this many milliseconds have passed; then the
    // communicator is aborted and every later call on it fails.
    int deadline_ms = 30000;
    bool aborted = false;
};

// One rank's end of the peer exchange.  xbuf: this rank's buffer; peer[q]: rank q's buffer as
// mapped into this process (peer[rank] == xbuf).  One exchange serves any number of blocks with
// the same output width H, as long as every rank calls them in the same order.
struct nvfp4_tp_exchange {
    nvfp4_tp_comm* comm = nullptr;
    int H = 0;
    unsigned char* xbuf = nullptr;
    unsigned char* peer[NVFP4_TP_MAX_WORLD] = {};
    float* partial = nullptr;          // [16, H] FP32: this rank's partial for the stand-alone exchange kernel
    bool attached = false;
};

namespace nvfp4 {
namespace tp {

constexpr int kFusedMaxM = xchg::kMaxTokens;

// Settles the result of an NCCL call on the non-blocking communicator: NVFP4_OK, or NVFP4_E_TP after an
// error or after the deadline (the communicator is aborted then).
int settle(nvfp4_tp_comm* comm, ncclResult_t r);

// Where the row-split linear sums over the group inside the mma.sync GEMV (mode 1, up to 16 tokens), the block's
// other linears take that GEMV too: a step that alternates between it and the NVFP4 tensor-core GEMV with its
// pre-pass is slower than either alone (2 GPUs, 64-layer token-step: 3.51 ms mixed, 3.09 ms mma.sync only).
// Sets the handle's "decode_impl" to 2 for the scope, if it was on automatic.
struct SameGemvScope {
    nvfp4_handle* h;
    bool on;
    SameGemvScope(nvfp4_handle* handle, const nvfp4_tp_comm* comm, const nvfp4_tp_exchange* x, int mode, int M)
        : h(handle), on(false) {
        int impl = 0;
        if (comm && comm->world > 1 && mode == 1 && x && x->attached && M <= kFusedMaxM &&
            nvfp4_get_option(h, "decode_impl", &impl) == NVFP4_OK && impl == 0)
            on = nvfp4_set_option(h, "decode_impl", 2) == NVFP4_OK;
    }
    ~SameGemvScope() {
        if (on) nvfp4_set_option(h, "decode_impl", 0);
    }
};

// Room for [max_M, H] FP32 partial sums on the communicator (grown at block-creation time, never in a forward).
int reserve_f32_partials(nvfp4_tp_comm* comm, int max_M, int H);

// C[M,H] = sum over ranks of A_r[M,K_r] * W_r[H,K_r]^T (+ residual), identical on every rank.
// `d` describes this rank's share (A, shard, residual, C; optionally the strided / SwiGLU /
// k_valid forms of nvfp4_linear_ex).  mode: 0 = NCCL (FP32 partials: reduce-scatter, residual and the
// one rounding on the rank's slice, all-gather; or, with comm->bf16_partials, one all-reduce of
// BF16-rounded partials), 1 = reduction inside the GEMV kernel,
// 2 = FP32 GEMV + stand-alone exchange kernel; 1 and 2 need an attached exchange and M <= 16.
// Returns NVFP4_E_LIMIT when `d` uses nvfp4_linear_ex options and the fused path cannot take
// it: the caller then materialises plain [M, K] activations and calls again.
// res_copy: [max_M, H] BF16 scratch for an in-place residual on the NCCL path.
int rowsplit_linear(nvfp4_handle* h, nvfp4_tp_comm* comm, nvfp4_tp_exchange* x, int mode, const nvfp4_linear_desc& d,
                    void* res_copy, cudaStream_t s);

}  // namespace tp
}  // namespace nvfp4
