"""BF16-weight linear (lm_head, projections that stay BF16 in a quantised checkpoint): the GEMV
kernel for up to 16 tokens against the CPU oracle, through the C ABI.  FP32 accumulation of exact
BF16 products: the only difference allowed is the summation order (relative Frobenius <= 1e-3,
the tolerance of the quantised path)."""
import os
import sys

import numpy as np
import pytest

import nvfp4
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu

TOL = 1e-3


def run(h, A, W, residual=None):
    import torch
    M, K = A.shape
    N = W.shape[0]
    dC = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")   # NaN canary
    dR = None
    if residual is not None:
        dC.copy_(util.to_dev(residual))
        dR = dC                                                         # in place
    h.linear_bf16(util.to_dev(A), M, util.to_dev(W), N, K, dC, residual=dR)
    torch.cuda.synchronize()
    return util.to_host_u16(dC)


@pytest.mark.parametrize("M,N,K,res", [
    (1, 128, 128, False),          # one unit
    (1, 300, 1024, True),          # N not a multiple of the 128-row tile
    (3, 5120, 5120, False),        # row tiles split over the CTAs
    (8, 20000, 256, True),         # many row tiles, two units each
    (5, 128, 17408, True),         # one row tile over all CTAs: many contributors
    (13, 1000, 2560, True),        # two launches of the 8-token kernel
    (16, 640, 640, False),
])
def test_dense_gemv_vs_oracle(handle, M, N, K, res):
    W = util.make_bf16((N, K), seed=N + K, std=0.05)
    A = util.make_bf16((M, K), seed=M + 1)
    R = util.make_bf16((M, N), seed=N + 2) if res else None
    l0 = handle.launch_count()
    got = run(handle, A, W, residual=R)
    assert handle.launch_count() - l0 == (1 if M <= 8 else 2)
    assert np.array_equal(got, run(handle, A, W, residual=R))          # fixed summation order
    want = ob.dense_linear(A, W, residual=R)
    assert ob.rel_frobenius(got, want) <= TOL
    assert handle.device_status() == 0


def test_dense_lm_head_shape_sample(handle):
    """A slice of the lm_head's width at the model's K, one token: every output against float64."""
    N, K = 24832, 5120
    W = util.make_bf16((N, K), seed=5, std=0.02)
    A = util.make_bf16((1, K), seed=6)
    got = ob.bf16_to_f32(run(handle, A, W)).astype(np.float64)
    want = ob.bf16_to_f32(A).astype(np.float64) @ ob.bf16_to_f32(W).astype(np.float64).T
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 3e-3   # BF16 output rounding


@pytest.mark.parametrize("M,N,K,res", [
    (17, 256, 256, False),         # one tile, one stage
    (24, 256, 512, True),
    (128, 1000, 1024, True),       # N not a multiple of the 256-row tile
    (300, 2048, 1280, False),      # three token tiles: a pair and a single
    (1000, 640, 5120, True),       # few tiles, deep K: split along k over the CTAs
    (130, 40000, 256, True),       # more tiles than CTAs: whole waves of pairs + a split remainder
])
def test_dense_gemm_vs_oracle(handle, M, N, K, res):
    """More than 16 tokens: the tcgen05 GEMM with the BF16 weight blocks loaded straight into the
    operand buffers."""
    W = util.make_bf16((N, K), seed=N + K + 1, std=0.05)
    A = util.make_bf16((M, K), seed=M + 3)
    R = util.make_bf16((M, N), seed=N + 4) if res else None
    l0 = handle.launch_count()
    got = run(handle, A, W, residual=R)
    assert handle.launch_count() - l0 == 1
    assert np.array_equal(got, run(handle, A, W, residual=R))          # fixed summation order
    assert ob.rel_frobenius(got, ob.dense_linear(A, W, residual=R)) <= TOL
    assert handle.device_status() == 0


def test_dense_fallback_shapes(handle):
    """K not a multiple of 256 beyond 16 tokens: the plain CUDA-core GEMM."""
    M, N, K = 24, 256, 384
    W = util.make_bf16((N, K), seed=7, std=0.05)
    A = util.make_bf16((M, K), seed=8)
    R = util.make_bf16((M, N), seed=9)
    got = run(handle, A, W, residual=R)
    assert ob.rel_frobenius(got, ob.dense_linear(A, W, residual=R)) <= TOL


def test_dense_argument_errors(handle):
    import torch
    A = torch.zeros((1, 128), dtype=torch.int16, device="cuda")
    W = torch.zeros((128, 128), dtype=torch.int16, device="cuda")
    C = torch.zeros((1, 128), dtype=torch.int16, device="cuda")
    with pytest.raises(nvfp4.Nvfp4Error):
        handle.linear_bf16(A, 1, W, 128, 124, C)            # K % 8
    with pytest.raises(nvfp4.Nvfp4Error):
        handle.linear_bf16(A, 1, W, 128, 128, A)            # output over the input


DENSE_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_b200_dense.npz")


@pytest.mark.skipif(not os.path.exists(DENSE_GOLDEN), reason="golden file not generated")
def test_dense_gemv_against_committed_reference_outputs(handle):
    """The BF16 GEMV against what the reference's own invoke_dense_gemv / _add kernels stored on a B200
    (src/engine/dense_gemm_sm110.cu:1140-1216)."""
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_reference_dense_golden as g
    gold = np.load(DENSE_GOLDEN)
    for name, c in g.cases().items():
        got = run(handle, c["A"], c["W"], residual=c["residual"])
        assert ob.rel_frobenius(got, gold[name]) <= TOL, name


@pytest.mark.skipif(not ob.ref_dense_available(), reason="oracle/_ref/libref_dense.so not built")
def test_dense_gemv_side_by_side_with_reference_kernels(handle):
    """The reference's BF16 GEMV and ours on the same device buffers, model-sized K."""
    import torch
    dense = ob.load_ref().dense
    st = torch.cuda.current_stream().cuda_stream
    for (N, K, res) in [(5120, 5120, False), (2048, 6144, True), (1024, 17408, True)]:
        W, A = util.make_bf16((N, K), seed=N + 3, std=0.05), util.make_bf16((1, K), seed=K + 4)
        R = util.make_bf16((1, N), seed=N + 5) if res else None
        dA, dW = util.to_dev(A), util.to_dev(W)
        o_ref = torch.zeros(1, N, dtype=torch.int16, device="cuda")
        if res:
            dense.ref_dense_gemv_add(dA.data_ptr(), dW.data_ptr(), o_ref.data_ptr(), util.to_dev(R).data_ptr(), N, K, st)
        else:
            dense.ref_dense_gemv(dA.data_ptr(), dW.data_ptr(), o_ref.data_ptr(), N, K, st)
        torch.cuda.synchronize()
        ref_bits = util.to_host_u16(o_ref)
        assert np.array_equal(ref_bits, ob.dense_gemv_ref(A, W, residual=R)), (N, K)      # the restatement, once more
        assert ob.rel_frobenius(run(handle, A, W, residual=R), ref_bits) <= TOL, (N, K)
