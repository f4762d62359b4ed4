"""The benchmark's own shapes against the oracle at full size.

Decode sweep: fused gate/up 34816 x 5120 and down 5120 x 17408 at 1, 2, 4, 8 and 16 tokens, every
output column of a seeded sample of weight rows.  Prefill: the same two weights at 64, 256, 2048
and 8192 tokens, a seeded sample of token rows x a seeded sample of weight rows (the oracle needs
seconds for that; the whole product would take it hours).  Inputs follow the benchmark's
distributions: uniform E2M1 codes, block scale = E4M3(max|w|/6) with w ~ N(0, 0.02), global scale 1,
activations ~ N(0,1) in BF16.  Tolerance: relative Frobenius error <= 1e-3 on the sample.
"""
import functools

import numpy as np
import pytest

import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu
TOL = 1e-3
SHAPES = {"gate_up": (34816, 5120), "down": (5120, 17408)}


@functools.lru_cache(maxsize=2)
def _weight(name):
    """Host copy and device copy of one full-size weight (generated once per shape)."""
    N, K = SHAPES[name]
    packed, scale = util.make_weight(N, K, seed=N)
    return packed, scale, util.to_dev(packed), util.to_dev(scale)


@pytest.mark.parametrize("name", ["gate_up", "down"])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_decode_sweep_shapes_sampled_rows(handle, name, M):
    import torch
    N, K = SHAPES[name]
    packed, scale, dp, ds = _weight(name)
    seed = 100 * M + N
    rows = np.sort(np.random.default_rng(seed).choice(N, 96, replace=False))
    A = util.make_bf16((M, K), seed=seed)
    R = util.make_bf16((M, N), seed=seed + 1)
    dC = util.to_dev(R)
    handle.linear(util.to_dev(A), M, dp, ds, 1.0, N, K, dC, residual=dC)
    torch.cuda.synchronize()
    got = np.ascontiguousarray(util.to_host_u16(dC)[:, rows])
    want = ob.linear(A, np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scale[rows]), 1.0,
                     residual=np.ascontiguousarray(R[:, rows]), mode=ob.GEMV, threads=8)
    err = ob.rel_frobenius(got, want)
    assert err <= TOL, (name, M, seed, err)
    assert handle.device_status() == 0


@pytest.mark.parametrize("name", ["gate_up", "down"])
@pytest.mark.parametrize("M", [64, 256, 2048, 8192])
def test_prefill_shapes_sampled_tokens_and_rows(big_handle, name, M):
    import torch
    N, K = SHAPES[name]
    packed, scale, dp, ds = _weight(name)
    seed = 7 * M + N
    rng = np.random.default_rng(seed)
    toks = np.sort(rng.choice(M, 64, replace=False))
    rows = np.sort(rng.choice(N, 256, replace=False))
    # activations are drawn on the device (8192 x 17408 normals take numpy a while); the sampled token rows
    # come back to the host for the oracle
    g = torch.Generator(device="cuda").manual_seed(seed)
    dA = torch.randn((M, K), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    dC = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    big_handle.linear(dA, M, dp, ds, 1.0, N, K, dC)
    torch.cuda.synchronize()
    t_idx = torch.from_numpy(toks).cuda()
    r_idx = torch.from_numpy(rows).cuda()
    A_s = util.to_host_u16(dA[t_idx].contiguous().view(torch.int16))
    got = util.to_host_u16(dC[t_idx][:, r_idx].contiguous().view(torch.int16))
    want = ob.linear(A_s, np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scale[rows]), 1.0, mode=ob.GEMM,
                     threads=8)
    err = ob.rel_frobenius(got, want)
    assert err <= TOL, (name, M, seed, err)
    assert big_handle.device_status() == 0
    # nothing outside the sample is left unwritten or non-finite
    assert bool(torch.isfinite(dC.float()).all())
