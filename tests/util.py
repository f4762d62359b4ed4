"""Seeded synthetic inputs in the reference's NVFP4 layout, shared by tests, golden
generation and the benchmark's parity spot-checks.  numpy only."""
import numpy as np

import oracle_binding as ob


def make_weight(N, K, seed, sigma=0.02):
    """packed uint8 [N,K/2] with every nibble uniform over the 16 codes; scale uint8
    [N,K/16] = E4M3(max|w|/6), w ~ N(0, sigma), 16 draws per block."""
    rng = np.random.default_rng([seed, N, K, 1])
    packed = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    w = rng.normal(0.0, sigma, size=(N, K // 16, 16)).astype(np.float32)
    s = np.abs(w).max(axis=-1) / np.float32(6.0)
    scale = ob.encode_e4m3(s)
    return packed, scale


def make_bf16(shape, seed, std=1.0):
    rng = np.random.default_rng([seed, 2] + list(shape))
    return ob.f32_to_bf16(rng.normal(0.0, std, size=shape).astype(np.float32))


def to_dev(arr):
    """numpy -> CUDA tensor of the same bytes (uint16 BF16 bits travel as int16)."""
    import torch
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.view(np.int16)).cuda()
    return torch.from_numpy(arr).cuda()


def to_host_u16(t):
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bf16_ulp_diff(a, b):
    """Max distance in BF16 ulps between two bit arrays (sign-magnitude aware)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return int(np.abs(key(a) - key(b)).max()) if a.size else 0


def pad_cols(a, cols):
    """[M, c] -> [M, cols] with zero columns appended (BF16 bits: zero is +0.0)."""
    out = np.zeros((a.shape[0], cols), a.dtype)
    out[:, :a.shape[1]] = a
    return out
