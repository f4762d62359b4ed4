"""CUDA-graph replay of single library calls whose row tiles are split over CTAs.

A captured graph replays its kernel parameters unchanged, so whatever tags the cross-CTA
hand-offs (split-tile partial pairs, stream-K flags) must not come from the host: the kernels
take it from a counter in their scratch.  Each case captures ONE call, then replays it many
times while the activation buffer is overwritten in place with new seeded values before every
replay; every replay must give the bits of an eager call on the same inputs (partials are added
in a fixed order) and sit within 1e-3 of the oracle on a sample of weight rows.  The reference
engine captures its decode step the same way (src/benchmark.cpp:777-810).
"""
import ctypes

import numpy as np
import pytest

import nvfp4
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu
TOL = 1e-3
REPLAYS = 200
N_INPUTS = 8


def _capture(torch, fn):
    """Warm up on a side stream, then capture one call of fn(stream) into a graph."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn(s)
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        fn(torch.cuda.current_stream())
    return g


def _replay_case(torch, M, K, n_out, call, oracle_fn, cols, status_fn, tol=TOL, replays=REPLAYS):
    """call(dA, dC, stream) launches the entry point under test on [M,K] activations and an
    [M,n_out] output; oracle_fn(A) gives the expected bits of output columns `cols`."""
    inputs = [util.make_bf16((M, K), seed=9000 + i, std=[1.0, 0.3, 4.0][i % 3]) for i in range(N_INPUTS)]
    staged = [util.to_dev(a) for a in inputs]
    want = [oracle_fn(a) for a in inputs]
    dA = torch.zeros((M, K), dtype=torch.int16, device="cuda")
    dC = torch.zeros((M, n_out), dtype=torch.int16, device="cuda")
    pick = lambda t: np.ascontiguousarray(util.to_host_u16(t)[:, cols])
    eager = []
    for i, a in enumerate(staged):
        dA.copy_(a)
        dC.fill_(0x7FC0)                      # NaN canary: an output nobody wrote shows up
        call(dA, dC, torch.cuda.current_stream())
        torch.cuda.synchronize()
        eager.append(dC.clone())
        assert ob.rel_frobenius(pick(dC), want[i]) <= tol, ("eager", i)
    g = _capture(torch, lambda s: call(dA, dC, s))
    bad = []
    for r in range(replays):
        i = (r * 3 + 1) % N_INPUTS
        dA.copy_(staged[i])                   # new activations in the same buffer: the graph's parameters stay as captured
        dC.fill_(0x7FC0)
        g.replay()
        if not torch.equal(dC, eager[i]):
            bad.append(r)
        if r % 50 == 0:
            torch.cuda.synchronize()
            assert ob.rel_frobenius(pick(dC), want[i]) <= tol, ("replay", r)
    torch.cuda.synchronize()
    assert not bad, f"{len(bad)} of {replays} replays differ from the eager call, first at {bad[:5]}"
    assert status_fn() == 0


def _sample_rows(N, seed, count=96):
    return np.sort(np.random.default_rng(seed).choice(N, min(N, count), replace=False))


@pytest.mark.parametrize("M,N,K", [
    (4, 5120, 17408),     # down projection: every row tile shared by 3-4 CTAs, middle contributors publish at their very end
    (1, 1024, 2048),      # two half-units per CTA: owners look for their contributors at once
    (8, 640, 5120),       # few row tiles over all CTAs
    (12, 5120, 17408),    # 10..16 tokens: activations streamed through the ring
    (16, 1024, 2048),
    (40, 1000, 17408),    # few-token tcgen05 kernel, every tile split along k
    (64, 5120, 4352),
    (300, 15360, 3840),   # prefill kernel: a whole wave of tiles + tiles split along k
    (130, 512, 5120),     # prefill kernel, every tile split
])
def test_graph_replay_linear(handle, M, N, K):
    _graph_replay_linear(handle, M, N, K)


@pytest.mark.parametrize("M,N,K", [
    (4, 5120, 17408),     # the mma.sync GEMV (pairs cleared after use): the kernel of the group reduction and of chains
    (1, 1024, 2048),
    (8, 640, 5120),
    (12, 5120, 17408),    # its wide variant (tag from the device-side counter)
    (16, 1024, 2048),
])
def test_graph_replay_linear_mma_sync_kernels(handle, M, N, K):
    handle.set_option("decode_impl", 2)
    try:
        _graph_replay_linear(handle, M, N, K)
    finally:
        handle.set_option("decode_impl", 0)


def _graph_replay_linear(handle, M, N, K):
    import torch
    packed, scale = util.make_weight(N, K, seed=M + N, sigma=0.14 if M > 16 else 0.02)
    dp, ds = util.to_dev(packed), util.to_dev(scale)
    rows = _sample_rows(N, N)
    sp, ss = np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scale[rows])
    mode = ob.GEMV if M <= 16 else ob.GEMM
    _replay_case(torch, M, K, N,
                 lambda dA, dC, s: handle.linear(dA, M, dp, ds, 1.0, N, K, dC, stream=s),
                 lambda A: ob.linear(A, sp, ss, 1.0, mode=mode, threads=8), rows, handle.device_status)


@pytest.mark.parametrize("M,N,K", [(4, 2048, 8192), (130, 512, 5120)])
def test_graph_replay_linear_bf16(handle, M, N, K):
    """BF16 weights: the GEMV skeleton (split row tiles) and the tcgen05 GEMM (split tiles)."""
    import torch
    W = util.make_bf16((N, K), seed=N, std=0.05)
    dW = util.to_dev(W)
    rows = _sample_rows(N, N + 1)
    Ws = np.ascontiguousarray(W[rows])
    _replay_case(torch, M, K, N,
                 lambda dA, dC, s: handle.linear_bf16(dA, M, dW, N, K, dC, stream=s),
                 lambda A: ob.dense_linear(A, Ws), rows, handle.device_status)


def test_graph_replay_noalloc():
    """The allocation-free GEMV: its fixed scratch array carries the same counter."""
    import torch
    lib = nvfp4.load()
    M, N, K = 4, 5120, 17408
    packed, scale = util.make_weight(N, K, seed=77)
    dp, ds = util.to_dev(packed), util.to_dev(scale)
    rows = _sample_rows(N, 5)
    sp, ss = np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scale[rows])

    def call(dA, dC, s):
        st = lib.nvfp4_linear_decode_noalloc(dA.data_ptr(), M, dp.data_ptr(), ds.data_ptr(), 1.0, N, K, None,
                                             dC.data_ptr(), s.cuda_stream)
        assert st == 0, lib.nvfp4_status_string(st).decode()

    def status():
        v = ctypes.c_uint(1)
        assert lib.nvfp4_noalloc_status(ctypes.byref(v), 0) == 0
        return v.value

    _replay_case(torch, M, K, N, call, lambda A: ob.linear(A, sp, ss, 1.0, mode=ob.GEMV, threads=8), rows, status)


def test_graph_replay_decode_step_of_two_linears(handle):
    """gate_up with the SwiGLU epilogue, then down with the residual, captured together (the decode
    MLP as the tensor-parallel block of one rank issues it): the second launch reads what the
    first wrote, both split their row tiles."""
    import torch
    import nvfp4_tp
    M, H, I = 2, 1024, 2304
    gu_p, gu_s = util.make_weight(2 * I, H, seed=41)
    dn_p, dn_s = util.make_weight(H, I, seed=42)
    order = nvfp4_tp.interleave_rows(I)
    d_gu_p, d_gu_s = util.to_dev(np.ascontiguousarray(gu_p[order])), util.to_dev(np.ascontiguousarray(gu_s[order]))
    d_dn_p, d_dn_s = util.to_dev(dn_p), util.to_dev(dn_s)
    R = util.make_bf16((M, H), seed=43)
    dR = util.to_dev(R)
    act = torch.zeros((M, I), dtype=torch.int16, device="cuda")

    def call(dA, dC, s):
        handle.linear_ex(dA, M, d_gu_p, d_gu_s, 1.0, 2 * I, H, act, swiglu_epilogue=True, stream=s)
        handle.linear(act, M, d_dn_p, d_dn_s, 1.0, H, I, dC, residual=dR, stream=s)

    cols = np.arange(H)
    _replay_case(torch, M, H, H, call, lambda A: ob.mlp(A, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R), cols,
                 handle.device_status, tol=2e-3)
