"""The GEMV on the NVFP4 tensor-core path (tcgen05.mma kind::mxf4nvf4; up to 16 tokens): weights go from
HBM to the tensor core untouched, the BF16 activations are expanded into five or six NVFP4 term rows per
token.  Checked against the CPU oracle (relative Frobenius <= 1e-3, the bar of every linear), against
the mma.sync GEMV on the same inputs, for exactness where the expansion is exact, and under
CUDA-graph replay."""
import numpy as np
import pytest

import nvfp4
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu
TOL = 1e-3


def run(h, A, packed, scale, gs, residual=None, native=True):
    import torch
    M, K = A.shape
    N = packed.shape[0]
    dC = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
    dR = None
    if residual is not None:
        dC.copy_(util.to_dev(residual))
        dR = dC
    h.set_option("decode_impl", 3 if native else 2)
    try:
        l0 = h.launch_count()
        h.linear(util.to_dev(A), M, util.to_dev(packed), util.to_dev(scale), gs, N, K, dC, residual=dR)
        launches = h.launch_count() - l0
    finally:
        h.set_option("decode_impl", 0)
    torch.cuda.synchronize()
    return util.to_host_u16(dC), launches


@pytest.mark.parametrize("M,N,K,res", [
    (1, 128, 256, False),          # one half-unit
    (1, 5120, 5120, False),        # the single-GEMV configuration of the benchmark
    (2, 300, 1024, True),          # N not a multiple of the 128-row tile
    (3, 2048, 5120, True),
    (4, 1024, 17408, True),        # deep K: row tiles split over many CTAs
    (5, 640, 5120, False),         # few row tiles over all CTAs
    (8, 4352, 5120, True),         # 48 MMA columns, two groups of activation scales
    (9, 1000, 2048, True),
    (7, 20000, 512, False),        # many row tiles, two half-units each
    (10, 640, 5120, True),         # six terms in 64 columns
    (12, 1000, 2048, True),        # 64 columns, five terms
    (13, 2048, 1024, False),       # 80 columns: the 128-column accumulators, three groups of activation scales
    (16, 4352, 5120, True),        # the largest token count of the kernel
    (16, 5120, 17408, True),       # ... on the deep shape of the benchmark
])
def test_fp4_gemv_vs_oracle(handle, M, N, K, res):
    packed, scale = util.make_weight(N, K, seed=N + K)
    A = util.make_bf16((M, K), seed=M + 3)
    R = util.make_bf16((M, N), seed=M + 4) if res else None
    got, launches = run(handle, A, packed, scale, 1.0, residual=R)
    assert launches in (1, 2)                                   # (the activation pre-pass +) the tensor-core GEMV
    want = ob.linear(A, packed, scale, 1.0, residual=R, mode=ob.GEMV, threads=8)
    assert ob.rel_frobenius(got, want) <= TOL
    again, _ = run(handle, A, packed, scale, 1.0, residual=R)
    assert np.array_equal(got, again)                           # fixed summation order
    other, _ = run(handle, A, packed, scale, 1.0, residual=R, native=False)
    assert ob.rel_frobenius(got, other) <= 5e-4                 # the mma.sync GEMV on the same inputs
    assert handle.device_status() == 0


def test_fp4_gemv_fuzz(handle):
    """Random shapes, global scales, weight and activation magnitudes (outliers included), residual."""
    rng = np.random.default_rng(77)
    worst = 0.0
    for it in range(120):
        K = int(rng.integers(1, 28)) * 256
        N = int(rng.integers(1, 700)) if it % 6 else int(rng.integers(700, 6000))
        M = int(rng.integers(1, 17))
        gs = float(rng.choice([1.0, 0.37, 7.25, 2688.0]))
        packed, scale = util.make_weight(N, K, seed=it, sigma=float(rng.choice([0.02, 0.14, 1.0])))
        A = util.make_bf16((M, K), seed=1000 + it, std=float(rng.choice([0.01, 1.0, 30.0])))
        if it % 4 == 0:                                         # a few elements a thousand times the rest
            A = A.copy()
            idx = rng.integers(0, K, 3)
            A[rng.integers(0, M), idx] = ob.f32_to_bf16(np.array([900.0, -1500.0, 640.0], np.float32) * float(rng.choice([0.01, 1.0])))
        R = util.make_bf16((M, N), seed=2000 + it) if it % 3 else None
        got, launches = run(handle, A, packed, scale, gs, residual=R)
        assert launches in (1, 2)
        err = ob.rel_frobenius(got, ob.linear(A, packed, scale, gs, residual=R, mode=ob.GEMV, threads=4))
        assert err <= TOL, (it, M, N, K, gs, err)
        worst = max(worst, err)
    print(f"worst relative Frobenius error {worst:.2e}")
    assert handle.device_status() == 0


def test_fp4_one_hot_and_power_of_two_activations_are_exact(handle):
    """A = e_k returns the dequantised column bit for bit; doubling the activations doubles every output;
    zero activations return the residual."""
    import torch
    N, K = 300, 1024
    packed, scale = util.make_weight(N, K, seed=77, sigma=0.14)
    wq = ob.dequant(packed, scale, 1.0)
    canon = lambda x: np.where((x & 0x7FFF) == 0, 0, x)
    for k in (0, 1, 15, 16, 333, 1023):
        A = np.zeros((1, K), np.uint16)
        A[0, k] = 0x3F80
        got, _ = run(handle, A, packed, scale, 1.0)
        assert np.array_equal(canon(got[0]), canon(wq[:, k])), k
    A = util.make_bf16((4, K), seed=5)
    a1, _ = run(handle, A, packed, scale, 1.0)
    a2, _ = run(handle, (A + 0x0080).astype(np.uint16), packed, scale, 1.0)
    nz = (a1 & 0x7FFF) != 0
    assert np.array_equal(a2[nz], (a1[nz] + 0x0080).astype(np.uint16))
    R = util.make_bf16((4, N), seed=6)
    z, _ = run(handle, np.zeros((4, K), np.uint16), packed, scale, 1.0, residual=R)
    assert np.array_equal(z, R)


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (2, 300, 6144), (5, 1000, 2048), (12, 640, 1024)])
def test_fp4_non_finite_activations_poison_their_token_only(handle, M, N, K):
    """An infinity or a NaN in a token makes that token's outputs NaN (the pre-pass has no finite expansion for it);
    the other tokens come out as if it were not there."""
    packed, scale = util.make_weight(N, K, seed=N)
    A = util.make_bf16((M, K), seed=M + 31)
    clean, _ = run(handle, A, packed, scale, 1.0)
    for bad_bits in (0x7F80, 0xFF80, 0x7FC0):             # +inf, -inf, NaN
        B = A.copy()
        B[M - 1, K // 3] = bad_bits
        got, _ = run(handle, B, packed, scale, 1.0)
        is_nan = ((got & 0x7F80) == 0x7F80) & ((got & 0x007F) != 0)
        assert is_nan[M - 1].all()
        assert np.array_equal(got[:M - 1], clean[:M - 1])
    assert handle.device_status() == 0


def test_fp4_scale_codes(handle):
    """Every scale code the format's finite range holds (0x00 .. 0x7E, and the same with bit 7 set, which
    the format ignores) in one weight.  0x7F / 0xFF are NaN to the tensor core and are left out: no finite
    FP8 E4M3 scale encodes to them."""
    N, K = 128, 2048
    rng = np.random.default_rng(9)
    packed = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    scale = rng.integers(0, 127, (N, K // 16), dtype=np.uint8) | (rng.integers(0, 2, (N, K // 16), dtype=np.uint8) << 7)
    A = util.make_bf16((3, K), seed=4)
    got, launches = run(handle, A, packed, scale, 1.0)
    assert launches == 2
    assert ob.rel_frobenius(got, ob.linear(A, packed, scale, 1.0, mode=ob.GEMV)) <= TOL


@pytest.mark.parametrize("M,N,K", [(1, 5120, 6144), (2, 640, 17408), (1, 300, 256), (2, 2048, 1024), (1, 7168, 5120)])
def test_fp4_own_expansion_equals_prepass(handle, M, N, K):
    """One or two tokens: the GEMV that expands its activations itself (no pre-pass launch) gives the bits of
    the pre-pass followed by the GEMV -- same terms, same sums -- also through a row stride and a K padded
    beyond the tensor."""
    import torch
    packed, scale = util.make_weight(N, K, seed=N + 3 * K)
    A = util.make_bf16((M, K), seed=M + 11, std=2.0)
    R = util.make_bf16((M, N), seed=M + 12)
    own, l1 = run(handle, A, packed, scale, 1.3, residual=R)
    handle.set_option("fp4_own_quant", 0)
    try:
        pre, l2 = run(handle, A, packed, scale, 1.3, residual=R)
    finally:
        handle.set_option("fp4_own_quant", 1)
    assert (l1, l2) == (1, 2)                              # shapes whose CTAs hold at most 8 chunks x tokens
    assert np.array_equal(own, pre)
    assert ob.rel_frobenius(own, ob.linear(A, packed, scale, 1.3, residual=R, mode=ob.GEMV, threads=8)) <= TOL
    if K >= 512:
        # the activations as the left part of wider rows, the last 256 columns of K beyond the tensor
        kv = K - 256
        wide = util.make_bf16((M, K + 64), seed=M + 13)
        Az = wide[:, :K].copy()
        Az[:, kv:] = 0
        want = ob.linear(Az, packed, scale, 1.0, mode=ob.GEMV, threads=8)
        dW, dp, ds = util.to_dev(wide), util.to_dev(packed), util.to_dev(scale)
        outs = []
        for own_on in (1, 0):
            handle.set_option("fp4_own_quant", own_on)
            handle.set_option("decode_impl", 3)
            try:
                dC = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
                handle.linear_ex(dW, M, dp, ds, 1.0, N, K, dC, a_row_stride=K + 64, k_valid=kv)
                torch.cuda.synchronize()
                outs.append(util.to_host_u16(dC))
            finally:
                handle.set_option("fp4_own_quant", 1)
                handle.set_option("decode_impl", 0)
        assert np.array_equal(outs[0], outs[1])
        assert ob.rel_frobenius(outs[0], want) <= TOL
    assert handle.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 17408, 5120), (1, 300, 1024), (2, 4096, 2048), (4, 1000, 5120), (8, 640, 17408)])
def test_fp4_dual_is_one_launch(handle, M, N, K):
    """Two weights of one shape on the same activations (the reference's dual GEMV, gate and up projection of one
    token): one pre-pass and ONE GEMV launch whose row tiles run over both weights."""
    import torch
    p1, s1 = util.make_weight(N, K, seed=N + 1)
    p2, s2 = util.make_weight(N, K, seed=N + 2, sigma=0.05)
    A = util.make_bf16((M, K), seed=M + 21)
    dA, dp1, ds1, dp2, ds2 = map(util.to_dev, (A, p1, s1, p2, s2))
    c1 = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
    c2 = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
    l0 = handle.launch_count()
    handle.linear_dual(dA, M, dp1, ds1, 1.0, dp2, ds2, 2.5, N, K, c1, c2)
    launches = handle.launch_count() - l0
    torch.cuda.synchronize()
    assert launches <= 2
    g1, g2 = util.to_host_u16(c1), util.to_host_u16(c2)
    assert ob.rel_frobenius(g1, ob.linear(A, p1, s1, 1.0, mode=ob.GEMV, threads=8)) <= TOL
    assert ob.rel_frobenius(g2, ob.linear(A, p2, s2, 2.5, mode=ob.GEMV, threads=8)) <= TOL
    single1, _ = run(handle, A, p1, s1, 1.0)
    single2, _ = run(handle, A, p2, s2, 2.5)
    # the single calls split their row tiles over the CTAs at other places: same products, another summation order
    assert ob.rel_frobenius(g1, single1) <= 2e-4 and ob.rel_frobenius(g2, single2) <= 2e-4
    assert handle.device_status() == 0


def test_fp4_graph_replay(handle):
    """One captured call (pre-pass + GEMV), replayed with new activations in the same buffer."""
    import torch
    M, N, K = 4, 5120, 17408
    packed, scale = util.make_weight(N, K, seed=3)
    dp, ds = util.to_dev(packed), util.to_dev(scale)
    inputs = [util.to_dev(util.make_bf16((M, K), seed=40 + i, std=[1.0, 0.3, 4.0][i % 3])) for i in range(6)]
    dA = torch.zeros((M, K), dtype=torch.int16, device="cuda")
    dC = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    eager = []
    for a in inputs:
        dA.copy_(a)
        handle.linear(dA, M, dp, ds, 1.0, N, K, dC)
        torch.cuda.synchronize()
        eager.append(dC.clone())
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        handle.linear(dA, M, dp, ds, 1.0, N, K, dC, stream=torch.cuda.current_stream())
    bad = []
    for r in range(200):
        i = (r * 5 + 1) % len(inputs)
        dA.copy_(inputs[i])
        dC.fill_(0x7FC0)
        g.replay()
        if not torch.equal(dC, eager[i]):
            bad.append(r)
    torch.cuda.synchronize()
    assert not bad, f"{len(bad)} replays differ, first at {bad[:5]}"
    assert handle.device_status() == 0
