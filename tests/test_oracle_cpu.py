"""CPU tests of the oracle: the format decoders against independent numpy restatements,
the structural facts of the reference formula, and the golden vectors produced by the
reference's own kernels on a B200 (tests/golden/reference_b200.npz)."""
import os
import sys

import numpy as np
import pytest

import oracle_binding as ob
import util

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_b200.npz")
E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def test_e2m1_table():
    lib = ob.load()
    for c in range(16):
        v = lib.nvfp4_oracle_e2m1(c)
        want = E2M1[c & 7] * (-1.0 if c & 8 else 1.0)
        assert v == want
    # code 8 is +0.0, not -0.0 (reference table, dense_gemm_fp4_sm110.cu:24-27)
    assert np.signbit(np.float32(lib.nvfp4_oracle_e2m1(8))) == False  # noqa: E712


def test_ue4m3_all_codes():
    lib = ob.load()
    for b in range(256):
        e, m = (b >> 3) & 0xF, b & 7
        want = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        assert lib.nvfp4_oracle_ue4m3(b) == np.float32(want)
    assert lib.nvfp4_oracle_ue4m3(0x7F) == 480.0 and lib.nvfp4_oracle_ue4m3(0xFF) == 480.0
    assert lib.nvfp4_oracle_ue4m3(0x80) == 0.0   # sign bit ignored


def test_e4m3_encoder_roundtrip_and_rne():
    lib = ob.load()
    for b in range(0x7F):   # every finite code decodes and re-encodes to itself
        assert lib.nvfp4_oracle_f2e4m3(lib.nvfp4_oracle_ue4m3(b)) == b
    # midpoints go to the even code
    for b in range(0x7E):
        lo, hi = lib.nvfp4_oracle_ue4m3(b), lib.nvfp4_oracle_ue4m3(b + 1)
        mid = (np.float64(lo) + np.float64(hi)) / 2
        got = lib.nvfp4_oracle_f2e4m3(float(mid))
        assert got == (b if b % 2 == 0 else b + 1)
    assert lib.nvfp4_oracle_f2e4m3(1e9) == 0x7E and lib.nvfp4_oracle_f2e4m3(448.0) == 0x7E


def test_e4m3_encoder_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)
    x = np.abs(rng.normal(0, 0.02, 4096)).astype(np.float32) / 6
    x = np.concatenate([x, np.abs(rng.normal(0, 3.0, 4096)).astype(np.float32)])
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(ob.encode_e4m3(x), want)
    assert np.array_equal(ob.encode_e4m3_scalar(x[::7]), want[::7])
    edge = np.array([0.0, 2.0 ** -10, 2.0 ** -9, 0.015625, 0.0146484375, 447.0, 448.0, 464.0, 1e6], np.float32)
    assert np.array_equal(ob.encode_e4m3(edge), ob.encode_e4m3_scalar(edge))


def test_bf16_rounding_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, 100000).astype(np.float32)
    x[:8] = [0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, -1e-40]
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ob.f32_to_bf16(x), want)
    lib = ob.load()
    got = np.array([lib.nvfp4_oracle_f2bf(float(v)) for v in x[:2000]], np.uint16)
    assert np.array_equal(got, want[:2000])


def dequant_table_case(gs):
    """N=256 rows (row n uses scale code n), K=16 (element k uses nibble code k)."""
    packed = np.tile(np.array([(2 * j) | ((2 * j + 1) << 4) for j in range(8)], np.uint8), (256, 1))
    scale = np.arange(256, dtype=np.uint8).reshape(256, 1)
    return packed, scale, gs


@pytest.mark.parametrize("gs", [1.0, 1.7, 2688.0])
def test_dequant_exhaustive_table(gs):
    packed, scale, gs = dequant_table_case(gs)
    out = ob.dequant(packed, scale, gs)
    inv = np.float32(1.0) / np.float32(gs)
    for n in range(256):
        e, m = (n >> 3) & 0xF, n & 7
        s = np.float32(m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))
        g = np.float32(s * inv)
        for k in range(16):
            lut = np.float32(E2M1[k & 7] * (-1.0 if (k & 8 and k & 7) else 1.0))
            want = ob.f32_to_bf16(np.array([lut * g], np.float32))[0]
            assert out[n, k] == want, (n, k)
    # negative code x zero scale is -0; code 8 stays +0
    assert out[0, 9] == 0x8000 and out[0, 8] == 0x0000 and out[200, 8] == 0x0000


def test_nibble_order_and_scale_index():
    N, K = 3, 64
    for k in range(K):
        packed = np.zeros((N, K // 2), np.uint8)
        scale = np.full((N, K // 16), 0x38, np.uint8)   # 1.0
        scale[1, k // 16] = 0x40                        # 2.0 only in the block that holds k
        packed[1, k // 2] = 0x2 << (4 * (k & 1))        # code 2 = 1.0; low nibble = even k
        A = np.zeros((1, K), np.uint16)
        A[0, k] = 0x4040                                # 3.0
        C = ob.linear(A, packed, scale, 1.0)
        assert ob.bf16_to_f32(C)[0].tolist() == [0.0, 6.0, 0.0], k


def test_linear_modes_against_float64():
    N, K, M = 48, 512, 5
    packed, scale = util.make_weight(N, K, seed=11)
    A = util.make_bf16((M, K), seed=12)
    R = util.make_bf16((M, N), seed=13)
    for gs in (1.0, 3.3):
        wq = ob.bf16_to_f32(ob.dequant(packed, scale, gs)).astype(np.float64)
        exact = ob.bf16_to_f32(A).astype(np.float64) @ wq.T + ob.bf16_to_f32(R)
        want = ob.f32_to_bf16(exact.astype(np.float32))
        for mode in (ob.GEMV, ob.GEMM):
            C = ob.linear(A, packed, scale, gs, residual=R, mode=mode)
            tol = 1e-3 if gs == 1.0 or mode == ob.GEMM else 2e-3
            assert ob.rel_frobenius(C, want) < tol
        # with gs == 1 every dequantised weight is exact in BF16, so both modes see the same operands
        if gs == 1.0:
            a = ob.linear(A, packed, scale, gs, mode=ob.GEMV)
            b = ob.linear(A, packed, scale, gs, mode=ob.GEMM)
            assert ob.rel_frobenius(a, b) < 1e-3


def test_residual_alias_and_threads():
    N, K, M = 40, 256, 3
    packed, scale = util.make_weight(N, K, seed=21)
    A = util.make_bf16((M, K), seed=22)
    R = util.make_bf16((M, N), seed=23)
    want = ob.linear(A, packed, scale, 1.0, residual=R)
    buf = R.copy()
    lib = ob.load()
    lib.nvfp4_oracle_linear_mt(A, M, packed, scale, 1.0, N, K, buf.ctypes.data, buf, 0, 1)   # C aliases residual
    assert np.array_equal(buf, want)
    assert np.array_equal(ob.linear(A, packed, scale, 1.0, residual=R, threads=4), want)


def test_swiglu_against_torch_fp32():
    torch = pytest.importorskip("torch")
    T, I = 3, 136
    merged = util.make_bf16((T, 2 * I), seed=31, std=2.0)
    out = ob.swiglu_merged(merged)
    x = torch.from_numpy(ob.bf16_to_f32(merged))
    g, u = x[:, :I], x[:, I:]
    want = (g / (1 + torch.exp(-g)) * u).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert util.bf16_ulp_diff(out, want) <= 1
    assert np.array_equal(ob.swiglu(np.ascontiguousarray(merged[:, :I]), np.ascontiguousarray(merged[:, I:])), out)


def test_mlp_and_tp_oracle_consistency():
    M, H, I = 3, 128, 256
    gu_p, gu_s = util.make_weight(2 * I, H, seed=41)
    dn_p, dn_s = util.make_weight(H, I, seed=42)
    X = util.make_bf16((M, H), seed=43)
    R = util.make_bf16((M, H), seed=44)
    full = ob.mlp(X, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R)
    # P = 1 must reproduce the unpartitioned MLP bit for bit
    assert np.array_equal(ob.tp_mlp(X, 1, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R), full)
    for P in (2, 4, 8):
        fp32 = ob.tp_mlp(X, P, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R, partial_bf16=False)
        bf16 = ob.tp_mlp(X, P, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R, partial_bf16=True)
        assert ob.rel_frobenius(fp32, full) < 1e-3
        assert ob.rel_frobenius(bf16, full) < 1e-2


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden file not generated yet")
def test_oracle_against_reference_golden():
    """Outputs of the reference engine's own kernels on a B200 (make_reference_golden.py)."""
    import make_reference_golden as mg
    g = np.load(GOLDEN)
    canon = lambda x: np.where((x & 0x7FFF) == 0, 0, x)
    for name, case in mg.cases().items():
        want = g[name]
        got = mg.oracle_output(case)
        M = case["A"].shape[0] if "A" in case else 0
        if case["kind"] == "dequant":
            # bit-exact; the identity-GEMM readout of the table turns -0 into +0
            assert np.array_equal(canon(got), canon(want)), name
        elif case["kind"] in ("dual", "swiglu") or M <= 8:
            # the reference's GEMV kernels are deterministic: the oracle reproduces them bit for bit
            assert np.array_equal(got, want), name
        elif case["residual"] is None:
            assert ob.rel_frobenius(got, want) <= 1e-3, name
        else:
            # M > 8 with a residual goes through the reference's library GEMM with beta = 1, whose
            # result sits one extra BF16 rounding away from the FP32-accumulate formula (measured
            # 1.15e-3 on this case; the oracle matches the float64 evaluation exactly).
            assert ob.rel_frobenius(got, want) <= 3e-3, name


# ---------------------------------------------------------------- RMSNorm

def test_rmsnorm_oracle_against_float64():
    M, K = 4, 5120
    x, w, b = util.make_bf16((M, K), seed=1, std=1.5), util.make_bf16((K,), seed=2, std=0.3), util.make_bf16((M, K), seed=3)
    xf, wf = ob.bf16_to_f32(x).astype(np.float64), ob.bf16_to_f32(w).astype(np.float64)
    want = ob.f32_to_bf16((xf / np.sqrt((xf ** 2).mean(1, keepdims=True) + 1e-6) * (1 + wf)).astype(np.float32))
    got = ob.rmsnorm(x, w, 1e-6)
    assert util.bf16_ulp_diff(got, want) <= 1 and (got != want).mean() < 0.02
    s = xf + ob.bf16_to_f32(b)
    want = ob.f32_to_bf16((s / np.sqrt((s ** 2).mean(1, keepdims=True) + 1e-6) * (1 + wf)).astype(np.float32))
    got, res = ob.rmsnorm(x, w, 1e-6, bias=b)
    assert np.array_equal(res, ob.f32_to_bf16(s.astype(np.float32)))
    assert util.bf16_ulp_diff(got, want) <= 1 and (got != want).mean() < 0.02


NORM_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_b200_rmsnorm.npz")


@pytest.mark.skipif(not os.path.exists(NORM_GOLDEN), reason="golden file not generated")
def test_rmsnorm_oracle_against_committed_reference_outputs():
    """The oracle against what the reference's own kernels stored on a B200: the updated residual
    bit for bit, the normalised rows up to the last bit of a few elements (the reference is
    compiled with fast-math rsqrt and division)."""
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_reference_rmsnorm_golden as g
    gold = np.load(NORM_GOLDEN)
    for name, c in g.cases().items():
        norm, res = g.oracle_output(c)
        if c["add"]:
            assert np.array_equal(res, gold[name + "_residual"]), name
        assert util.bf16_ulp_diff(norm, gold[name]) <= 1, name
        assert (norm != gold[name]).mean() <= 0.02, name


def test_dense_linear_oracle_against_float64():
    M, N, K = 3, 200, 768
    A, W, R = util.make_bf16((M, K), seed=31), util.make_bf16((N, K), seed=32, std=0.05), util.make_bf16((M, N), seed=33)
    want = ob.bf16_to_f32(A).astype(np.float64) @ ob.bf16_to_f32(W).astype(np.float64).T + ob.bf16_to_f32(R)
    got = ob.dense_linear(A, W, residual=R)
    assert util.bf16_ulp_diff(got, ob.f32_to_bf16(want.astype(np.float32))) <= 1


DENSE_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_b200_dense.npz")


@pytest.mark.skipif(not os.path.exists(DENSE_GOLDEN), reason="golden file not generated")
def test_dense_gemv_restatement_reproduces_the_reference_kernels_bit_for_bit():
    """The oracle's statement of the reference's BF16 GEMV order against what the reference's own
    kernels (plain, scattered and K-tiled, with and without the residual) stored on a B200."""
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_reference_dense_golden as g
    gold = np.load(DENSE_GOLDEN)
    for name, c in g.cases().items():
        assert np.array_equal(g.oracle_output(c), gold[name]), name
        # the generic FP32 dot in k order is the same sum in another order: last-bit differences only
        assert ob.rel_frobenius(ob.dense_linear(c["A"], c["W"], residual=c["residual"]), gold[name]) <= 3e-4, name
