"""The activation expansion of the NVFP4 tensor-core GEMV (act_fp4.cu), restated in numpy and checked on the CPU:
a BF16 token times a power of two c is split, per 16-element block, into T terms q_t * s_t (q_t an E2M1 value,
s_t a power of two an unsigned E4M3 byte holds) whose sum reproduces it up to s_0 / 4096 (five terms) or
s_0 / 32768 (six), or 2^-11 where a block's terms have reached the smallest scale (2^-20 of the token's largest
element).  This pins the error bound the kernel's accuracy claim rests on; the GPU tests pin the kernel."""
import numpy as np
import pytest

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def round_e2m1(x):
    """cvt.rn.satfinite.e2m1x2.f32: nearest E2M1 value, ties to the even code, saturating at +-6."""
    a = np.minimum(np.abs(x), 6.0).astype(np.float32)
    idx = np.searchsorted(E2M1, a, side="left")                 # first grid value >= a
    idx = np.clip(idx, 1, 7)
    lo, hi = E2M1[idx - 1], E2M1[idx]
    take_hi = (a - lo > hi - a) | ((a - lo == hi - a) & (idx % 2 == 0))     # tie: the even code (index) wins
    q = np.where(take_hi, hi, lo)
    return np.sign(x).astype(np.float32) * q


def expand(x, terms):
    """x: float32 [K] (a BF16 token, K % 16 == 0).  Returns (terms as float32 [T, K], c, s0 per block)."""
    amax = np.abs(x).max()
    e = np.floor(np.log2(amax)) if amax > 0 else 0.0
    c = np.float32(2.0 ** (9 - e))                              # largest magnitude into [2^9, 2^10)
    r = (x * c).astype(np.float32).reshape(-1, 16)
    bmax = np.abs(r).max(axis=1)
    p0 = np.where(bmax > 0, np.ceil(np.log2(np.maximum(bmax, 1e-30) / 6.0)), -9).astype(np.int32)
    p0 = np.clip(p0, -9, 8)
    out = []
    for t in range(terms):
        p = np.maximum(p0 - (0 if t == 0 else 2 + 3 * (t - 1)), -9)
        s = (2.0 ** p).astype(np.float32)[:, None]
        q = round_e2m1(r / s)
        out.append((q * s).reshape(-1))
        r = (r - q * s).astype(np.float32)                      # exact: powers of two and short mantissas
    return np.stack(out), c, (2.0 ** p0).astype(np.float32), r.reshape(-1)


def bf16(x):
    u = np.asarray(x, np.float32).view(np.uint32)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.view(np.float32)


@pytest.mark.parametrize("terms,bound", [(5, 1.0 / 4096), (6, 1.0 / 32768)])
@pytest.mark.parametrize("kind", ["normal", "outliers", "tiny_blocks", "one_hot"])
def test_remainder_bound(terms, bound, kind):
    rng = np.random.default_rng(len(kind) * 10 + terms)
    K = 2048
    x = bf16(rng.standard_normal(K).astype(np.float32) * 3.0)
    if kind == "outliers":
        x[rng.integers(0, K, 4)] = bf16(np.float32([900.0, -1500.0, 640.0, 2.0e4]))
    if kind == "tiny_blocks":
        x[256:768] = bf16(x[256:768] * np.float32(2.0 ** -12))
    if kind == "one_hot":
        x[:] = 0.0
        x[333] = 1.0
    t, c, s0, rem = expand(x, terms)
    s0_el = np.repeat(s0, 16)
    # ... or a quarter of the smallest scale, 2^-11, where a block's later terms have reached it: after the token scaling
    # that is 2^-20 (1e-6) of the token's largest element
    assert np.all(np.abs(rem) <= np.maximum(s0_el * np.float32(bound), np.float32(2.0 ** -11)) * (1 + 1e-6))
    assert np.abs(x * c).max() >= 512.0
    # every scale is a power of two unsigned E4M3 represents (2^-9 .. 2^8), every term value is exact in FP32
    assert s0.min() >= 2.0 ** -9 and s0.max() <= 2.0 ** 8
    back = t.sum(axis=0, dtype=np.float32) + rem
    assert np.array_equal(back, (x * c).astype(np.float32))      # the split loses nothing but the stated remainder
    if kind == "one_hot":
        assert np.all(rem == 0)
    # relative to the block's largest element: five terms 8e-5, six 1e-5 (s0 < max / 3), unless the 2^-11 floor applies
    blk = np.abs((x * c).reshape(-1, 16)).max(axis=1)
    rmax = np.abs(rem.reshape(-1, 16)).max(axis=1)
    assert np.all((rmax <= blk * np.float32(bound / 3) * (1 + 1e-6)) | (rmax <= 2.0 ** -11))


def test_e2m1_rounding_ties_to_even():
    x = np.float32([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -5.0, 0.2, 0.3])
    want = np.float32([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0, -4.0, 0.0, 0.5])
    assert np.array_equal(np.abs(round_e2m1(x)), np.abs(want))
