"""CPU tests of the tensor-parallel MLP's host-side logic: the sharding rule, the K padding and
the one-all-reduce composition, run as two gloo ranks with the CPU oracle standing in for the
per-rank kernels, against the partition-aware oracle."""
import os
import socket

import numpy as np
import pytest

import nvfp4_tp
import oracle_binding as ob
import util


def test_shards_tile_the_full_weight():
    H, I, P = 256, 512, 4
    gu_p, gu_s = util.make_weight(2 * I, H, seed=1)
    dn_p, dn_s = util.make_weight(H, I, seed=2)
    gates, ups, cols = [], [], []
    for r in range(P):
        p, s = nvfp4_tp.shard_gate_up(gu_p, gu_s, r, P)
        assert p.shape == (2 * I // P, H // 2) and s.shape == (2 * I // P, H // 16)
        gates.append(p[:I // P]); ups.append(p[I // P:])
        dp, ds = nvfp4_tp.shard_down(dn_p, dn_s, r, P)
        assert dp.shape[1] * 2 % 256 == 0 and ds.shape[1] * 16 == dp.shape[1] * 2
        cols.append(dp[:, :I // P // 2])
        assert not dp[:, I // P // 2:].any() and not ds[:, I // P // 16:].any()
    assert np.array_equal(np.concatenate(gates + ups), gu_p)
    assert np.array_equal(np.concatenate(cols, axis=1), dn_p)


def test_padding_contributes_nothing():
    H, I = 256, 2176   # I/P = 272 at P = 8 is not a multiple of 256: padded to 512
    dn_p, dn_s = util.make_weight(H, I, seed=3)
    A = util.make_bf16((3, I), seed=4)
    for P in (8,):
        ip = I // P
        for r in (0, 5):
            p, s = nvfp4_tp.shard_down(dn_p, dn_s, r, P)
            a = nvfp4_tp.pad_activation(np.ascontiguousarray(A[:, r * ip:(r + 1) * ip]), p.shape[1] * 2)
            got = ob.linear(a, p, s, 1.0, mode=ob.GEMV)
            want = ob.linear(np.ascontiguousarray(A[:, r * ip:(r + 1) * ip]),
                             np.ascontiguousarray(dn_p[:, r * ip // 2:(r + 1) * ip // 2]),
                             np.ascontiguousarray(dn_s[:, r * ip // 16:(r + 1) * ip // 16]), 1.0, mode=ob.GEMV)
            assert ob.rel_frobenius(got, want) < 1e-6


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_qkv_split_follows_the_kv_heads(world):
    """Every q row lands on exactly one rank; every KV head on one rank, or, with more ranks than
    KV heads, on world / n_kv ranks -- and always on the rank that holds its query heads."""
    q_rows, kv_rows, n_kv = 6144, 512, 2
    head = kv_rows // n_kv
    q_per_kv = q_rows // n_kv
    seen_q = np.zeros(q_rows, int)
    seen_kv = np.zeros(kv_rows, int)
    for r in range(world):
        rows = nvfp4_tp.qkv_rows(q_rows, kv_rows, n_kv, r, world)
        q = rows[rows < q_rows]
        k = rows[(rows >= q_rows) & (rows < q_rows + kv_rows)] - q_rows
        v = rows[rows >= q_rows + kv_rows] - q_rows - kv_rows
        assert np.array_equal(k, v) and len(q) == q_rows // world
        seen_q[q] += 1
        seen_kv[k] += 1
        # the KV heads of this rank's query rows are the KV heads it holds
        assert set(q // q_per_kv) == set(k // head)
    assert (seen_q == 1).all()
    assert (seen_kv == max(1, world // n_kv)).all()


def test_attention_projections_split_matches_unsplit():
    """Column-split QKV + row-split output projection with the oracle as the kernel: the shards'
    outputs are slices of the unsplit projection, and the partial sums add up to the unsplit
    output projection (FP32 partials: the fused path's arithmetic)."""
    M, H, world = 3, 256, 4
    q_rows, kv_rows, n_kv, o_in = 1024, 128, 2, 1024
    qkv_p, qkv_s = util.make_weight(q_rows + 2 * kv_rows, H, seed=21)
    o_p, o_s = util.make_weight(H, o_in, seed=22)
    X = util.make_bf16((M, H), seed=23)
    full = ob.linear(X, qkv_p, qkv_s, 1.0)
    attn_full = np.ascontiguousarray(full[:, :q_rows])          # stub attention: the q columns
    want = ob.bf16_to_f32(ob.linear(attn_full, o_p, o_s, 1.0))
    total = np.zeros((M, H), np.float64)
    for r in range(world):
        p, s = nvfp4_tp.shard_qkv(qkv_p, qkv_s, q_rows, kv_rows, n_kv, r, world)
        mine = ob.linear(X, p, s, 1.0)
        assert np.array_equal(mine, full[:, nvfp4_tp.qkv_rows(q_rows, kv_rows, n_kv, r, world)])
        ol = o_in // world
        dp, ds = nvfp4_tp.shard_down(o_p, o_s, r, world)        # the output projection splits like the down projection
        a = nvfp4_tp.pad_activation(np.ascontiguousarray(mine[:, :ol]), dp.shape[1] * 2)
        total += ob.bf16_to_f32(ob.linear(a, dp, ds, 1.0)).astype(np.float64)
    # each partial carries one BF16 rounding here (the oracle's output type); the fused kernel keeps FP32
    assert np.linalg.norm(total - want) / np.linalg.norm(want) < 5e-3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, H, I = 3, 256, 512
        gu_p, gu_s = util.make_weight(2 * I, H, seed=11)
        dn_p, dn_s = util.make_weight(H, I, seed=12)
        X = util.make_bf16((M, H), seed=13)
        R = util.make_bf16((M, H), seed=14)
        # what nvfp4_tp_mlp_forward does on one rank, with the oracle as the kernel
        p, s = nvfp4_tp.shard_gate_up(gu_p, gu_s, rank, world)
        gate_up = ob.linear(X, p, s, 1.0)
        act = ob.swiglu_merged(gate_up)
        dp, ds = nvfp4_tp.shard_down(dn_p, dn_s, rank, world)
        part = ob.linear(nvfp4_tp.pad_activation(act, dp.shape[1] * 2), dp, ds, 1.0)
        t = torch.from_numpy(ob.bf16_to_f32(part).copy())
        dist.all_reduce(t)                     # one sum all-reduce of the [M, H] BF16 partials
        summed = ob.bf16_to_f32(ob.f32_to_bf16(t.numpy()))              # the collective delivers BF16
        got = ob.f32_to_bf16(summed + ob.bf16_to_f32(R))                # residual added once, after the sum
        q.put((rank, got))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_gloo_matches_partition_aware_oracle(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    M, H, I = 3, 256, 512
    gu_p, gu_s = util.make_weight(2 * I, H, seed=11)
    dn_p, dn_s = util.make_weight(H, I, seed=12)
    X = util.make_bf16((M, H), seed=13)
    R = util.make_bf16((M, H), seed=14)
    assert np.array_equal(outs[0], outs[1])    # every rank ends with the same tensor
    full = ob.mlp(X, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R)
    aware = ob.tp_mlp(X, world, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R, partial_bf16=True)
    # BF16 partials: close to the partition-aware oracle, a BF16 rounding away from the unsplit MLP
    assert ob.rel_frobenius(outs[0], aware) < 5e-3
    assert ob.rel_frobenius(outs[0], full) < 1e-2


def _rank_main_fp32(rank, world, port, q):
    """The NCCL path of the row-split linear as the library runs it above 16 tokens, with gloo and numpy in
    place of NCCL and the kernels: unrounded FP32 partial sums, summed over the ranks, each rank finishes ITS
    slice (residual, one rounding), the BF16 slices are gathered."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, H, I = 24, 256, 512
        gu_p, gu_s = util.make_weight(2 * I, H, seed=11)
        dn_p, dn_s = util.make_weight(H, I, seed=12)
        X = util.make_bf16((M, H), seed=13)
        R = util.make_bf16((M, H), seed=14)
        p, s = nvfp4_tp.shard_gate_up(gu_p, gu_s, rank, world)
        act = ob.swiglu_merged(ob.linear(X, p, s, 1.0))
        dp, ds = nvfp4_tp.shard_down(dn_p, dn_s, rank, world)
        a32 = ob.bf16_to_f32(nvfp4_tp.pad_activation(act, dp.shape[1] * 2))
        w32 = ob.bf16_to_f32(ob.dequant(dp, ds, 1.0))                  # exact: 2 + 4 significant bits
        part = torch.from_numpy((a32 @ w32.T).astype(np.float32))      # unrounded FP32 partial [M, H]
        dist.all_reduce(part)                                          # reduce-scatter: the sum, of which a rank keeps its slice
        cnt = M * H // world
        mine = part.reshape(-1)[rank * cnt:(rank + 1) * cnt].numpy()
        res = ob.bf16_to_f32(R).reshape(-1)[rank * cnt:(rank + 1) * cnt]
        piece = torch.from_numpy(ob.f32_to_bf16(mine + res).astype(np.int32))
        pieces = [torch.empty_like(piece) for _ in range(world)]
        dist.all_gather(pieces, piece)                                 # all-gather of the finished BF16 slices
        got = np.concatenate([t.numpy() for t in pieces]).astype(np.uint16).reshape(M, H)
        q.put((rank, got))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_fp32_partials_stay_within_the_linear_tolerance():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main_fp32, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    M, H, I = 24, 256, 512
    gu_p, gu_s = util.make_weight(2 * I, H, seed=11)
    dn_p, dn_s = util.make_weight(H, I, seed=12)
    X, R = util.make_bf16((M, H), seed=13), util.make_bf16((M, H), seed=14)
    assert np.array_equal(outs[0], outs[1])
    full = ob.mlp(X, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R)
    assert ob.rel_frobenius(outs[0], full) <= 1e-3                     # one rounding, as the unsplit layer
    bf16_form = ob.tp_mlp(X, world, gu_p, gu_s, 1.0, dn_p, dn_s, 1.0, residual=R, partial_bf16=True)
    assert ob.rel_frobenius(bf16_form, full) > ob.rel_frobenius(outs[0], full)     # what BF16-rounded partials cost


def _attn_rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, H, q_rows, kv_rows, n_kv, o_in = 3, 256, 512, 128, 2, 512
        qkv_p, qkv_s = util.make_weight(q_rows + 2 * kv_rows, H, seed=41)
        o_p, o_s = util.make_weight(H, o_in, seed=42)
        X, R = util.make_bf16((M, H), seed=43), util.make_bf16((M, H), seed=44)
        # what nvfp4_tp_attn_qkv / nvfp4_tp_attn_out do on one rank, with the oracle as the kernel
        p, s = nvfp4_tp.shard_qkv(qkv_p, qkv_s, q_rows, kv_rows, n_kv, rank, world)
        qkv = ob.linear(X, p, s, 1.0)
        ol = o_in // world
        attn = np.ascontiguousarray(qkv[:, :ol])               # stub attention: this rank's q columns
        dp, ds = nvfp4_tp.shard_down(o_p, o_s, rank, world)
        part = ob.linear(nvfp4_tp.pad_activation(attn, dp.shape[1] * 2), dp, ds, 1.0)
        t = torch.from_numpy(ob.bf16_to_f32(part).copy())
        dist.all_reduce(t)                                     # one sum all-reduce of the [M, H] partials
        got = ob.f32_to_bf16(ob.bf16_to_f32(ob.f32_to_bf16(t.numpy())) + ob.bf16_to_f32(R))
        q.put((rank, qkv, got))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_attention_block():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_attn_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {r: (a, b) for r, a, b in (q.get(timeout=120) for _ in range(world))}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    M, H, q_rows, kv_rows, n_kv, o_in = 3, 256, 512, 128, 2, 512
    qkv_p, qkv_s = util.make_weight(q_rows + 2 * kv_rows, H, seed=41)
    o_p, o_s = util.make_weight(H, o_in, seed=42)
    X, R = util.make_bf16((M, H), seed=43), util.make_bf16((M, H), seed=44)
    full = ob.linear(X, qkv_p, qkv_s, 1.0)
    for r in range(world):                                     # every rank's q | k | v = rows of the unsplit projection
        assert np.array_equal(res[r][0], full[:, nvfp4_tp.qkv_rows(q_rows, kv_rows, n_kv, r, world)])
    assert np.array_equal(res[0][1], res[1][1])                # every rank ends with the same tensor
    want = ob.linear(np.ascontiguousarray(full[:, :q_rows]), o_p, o_s, 1.0, residual=R)
    assert ob.rel_frobenius(res[0][1], want) < 1e-2            # BF16 partials: a rounding away from the unsplit projection
