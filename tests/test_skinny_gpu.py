"""Few-token kernel (dequantised weights in tensor memory, tokens on the N side of tcgen05.mma):
parity with the CPU oracle for 1 <= M <= 128, through the C ABI.  The arithmetic is the
reference's small-M kernel (src/engine/dense_gemm_fp4_sm110.cu:96-233): FP32 block scales,
FP32 accumulation, residual added before the only rounding."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu

TOL = 1e-3   # relative Frobenius error against the oracle


@pytest.fixture()
def skinny(handle):
    handle.set_option("skinny_min_m", 1)
    handle.set_option("skinny_max_m", 128)
    handle.set_option("wide_gemv", 0)
    yield handle
    handle.set_option("wide_gemv", 1)
    handle.set_option("skinny_min_m", 9)
    handle.set_option("skinny_max_m", 64)


def run(h, A, packed, scale, gs, residual=None):
    import torch
    M, K = A.shape
    N = packed.shape[0]
    dA, dp, ds = util.to_dev(A), util.to_dev(packed), util.to_dev(scale)
    dC = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")   # NaN canary
    dR = None
    if residual is not None:
        dC.copy_(util.to_dev(residual))
        dR = dC                                                         # in place, as the reference's down projection
    h.linear(dA, M, dp, ds, gs, N, K, dC, residual=dR)
    torch.cuda.synchronize()
    return util.to_host_u16(dC)


@pytest.mark.parametrize("M,N,K,res", [
    (1, 128, 256, False),        # one tile, one stage
    (1, 256, 512, True),
    (3, 300, 1024, True),        # N not a multiple of the 128-row tile
    (8, 5120, 4352, False),      # 40 row tiles split by k over all SMs
    (16, 1000, 2560, True),
    (17, 64, 256, False),        # fewer rows than one tile
    (40, 20000, 512, True),      # 157 row tiles: one whole wave + split remainder
    (64, 2048, 5120, False),
    (100, 640, 1280, True),
    (128, 384, 768, True),
])
def test_skinny_vs_oracle(skinny, M, N, K, res):
    import oracle_binding as ob
    packed, scale = util.make_weight(N, K, seed=M + N, sigma=0.14)
    A = util.make_bf16((M, K), seed=M + 1)
    R = util.make_bf16((M, N), seed=N + 2) if res else None
    got = run(skinny, A, packed, scale, 1.0, residual=R)
    again = run(skinny, A, packed, scale, 1.0, residual=R)
    assert np.array_equal(got, again)                       # fixed summation order
    want = ob.linear(A, packed, scale, 1.0, residual=R, mode=ob.GEMV, threads=8)
    assert ob.rel_frobenius(got, want) <= TOL
    assert skinny.device_status() == 0


def test_skinny_global_scale_and_extreme_values(skinny):
    """global_scale != 1, block scales over the whole UE4M3 range (denormals, 448), large and
    tiny BF16 activations: the per-token power-of-two scale of the FP16 copy is exact and undone
    in FP32."""
    import oracle_binding as ob
    M, N, K = 5, 256, 1024
    rng = np.random.default_rng(7)
    packed = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    scale = rng.integers(0, 127, size=(N, K // 16), dtype=np.uint8)
    A = util.make_bf16((M, K), seed=9)
    Af = ob.bf16_to_f32(A)
    Af[0] *= 1e4
    Af[1] *= 1e-6
    A = ob.f32_to_bf16(Af)
    got = run(skinny, A, packed, scale, 37.5)
    want = ob.linear(A, packed, scale, 37.5, mode=ob.GEMV, threads=4)
    assert ob.rel_frobenius(got, want) <= TOL


def test_skinny_matches_gemv_kernel(skinny):
    """Same inputs through the mma.sync GEMV kernel and through this one: both accumulate exact
    products in FP32, so they differ only by summation order."""
    import oracle_binding as ob
    M, N, K = 4, 1024, 5120
    packed, scale = util.make_weight(N, K, seed=21)
    A = util.make_bf16((M, K), seed=22)
    a = run(skinny, A, packed, scale, 1.0)
    skinny.set_option("skinny_min_m", 17)
    b = run(skinny, A, packed, scale, 1.0)
    assert ob.rel_frobenius(a, b) <= 2e-4


# ---------------------------------------------------------------- wide GEMV: 9..16 tokens in one launch

@pytest.mark.parametrize("M,N,K,res", [
    (9, 128, 256, False),         # one row tile, one half-unit
    (12, 300, 1024, True),        # N not a multiple of the 128-row tile
    (16, 5120, 4352, True),       # 40 row tiles split by k over all SMs (odd number of half-units per tile)
    (16, 20000, 512, False),      # many row tiles, two half-units each
    (11, 1000, 17408, True),      # deep K
])
def test_wide_gemv_vs_oracle(handle, M, N, K, res):
    import oracle_binding as ob
    assert handle.get_option("wide_gemv") == 1
    packed, scale = util.make_weight(N, K, seed=M + N, sigma=0.14)
    A = util.make_bf16((M, K), seed=M + 1)
    R = util.make_bf16((M, N), seed=N + 2) if res else None
    l0 = handle.launch_count()
    got = run(handle, A, packed, scale, 1.7, residual=R)
    assert handle.launch_count() - l0 == 2                  # the activation pre-pass + ONE GEMV launch
    again = run(handle, A, packed, scale, 1.7, residual=R)
    assert np.array_equal(got, again)                       # fixed summation order
    want = ob.linear(A, packed, scale, 1.7, residual=R, mode=ob.GEMV, threads=8)
    assert ob.rel_frobenius(got, want) <= TOL
    handle.set_option("wide_gemv", 0)                       # the same through two launches of the 8-token kernel
    handle.set_option("skinny_min_m", 129)
    try:
        two = run(handle, A, packed, scale, 1.7, residual=R)
    finally:
        handle.set_option("wide_gemv", 1)
        handle.set_option("skinny_min_m", 9)
    assert ob.rel_frobenius(got, two) <= 2e-4
    assert handle.device_status() == 0
