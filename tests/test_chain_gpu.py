"""nvfp4_chain: several linears (up to 8 tokens each) run in order by ONE launch of the GEMV kernel, with a
grid-wide barrier in device memory between them.  Checked against the same linears issued one by one
(same kernel, same summation order: identical bits), against the CPU oracle, and under CUDA-graph
replay with changing inputs.  The layer-shaped case is the reference's decode sequence around the MLP
(src/engine/layer.cu:404-409 output projection + residual, :47-110 norm, gate_up, SwiGLU, down + residual)."""
import numpy as np
import pytest

import nvfp4
import nvfp4_tp
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _dev_weight(N, K, seed):
    p, s = util.make_weight(N, K, seed=seed)
    return p, s, util.to_dev(p), util.to_dev(s)


@pytest.mark.parametrize("M", [1, 3, 8])
def test_chain_of_independent_linears_equals_single_calls(handle, M):
    """Shapes whose row tiles are split over CTAs, whole, or fewer than the CTAs: every linear of the chain
    gives the bits of nvfp4_linear on the same inputs (the 8-token kernel in both cases)."""
    import torch
    shapes = [(5120, 2048), (640, 5120), (128, 256), (1000, 1024), (2304, 17408), (5120, 2048)]
    handle.set_option("skinny_min_m", 129)
    handle.set_option("decode_impl", 2)          # the single calls through the chain's own kernel, the mma.sync GEMV
    try:
        lin, want = [], []
        for i, (N, K) in enumerate(shapes):
            p, s, dp, ds = _dev_weight(N, K, seed=10 + i)
            A = util.make_bf16((M, K), seed=20 + i)
            R = util.make_bf16((M, N), seed=30 + i) if i % 2 else None
            dA = util.to_dev(A)
            single = util.to_dev(R) if R is not None else torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
            handle.linear(dA, M, dp, ds, 1.5, N, K, single, residual=single if R is not None else None)
            C = util.to_dev(R) if R is not None else torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
            lin.append(dict(A=dA, M=M, packed=dp, scale=ds, global_scale=1.5, N=N, K=K, C=C, residual=C if R is not None else None))
            want.append((single, ob.linear(A, p, s, 1.5, residual=R, mode=ob.GEMV, threads=8)))
        chain = nvfp4.Chain(handle, lin)
        try:
            chain.run()
            torch.cuda.synchronize()
            for l, (single, oracle) in zip(lin, want):
                assert torch.equal(l["C"], single), (l["N"], l["K"])
                assert ob.rel_frobenius(util.to_host_u16(l["C"]), oracle) <= TOL
        finally:
            chain.close()
    finally:
        handle.set_option("skinny_min_m", 9)
        handle.set_option("decode_impl", 0)
    assert handle.device_status() == 0


def _layer(handle, torch, M, H, I, O, seed):
    """Buffers and descriptors of: hid2 = hid + attn * Wo^T ; act = swiglu(rmsnorm(hid2) * Wgu^T) ; out = hid2 + act * Wdn^T."""
    o_p, o_s, d_o_p, d_o_s = _dev_weight(H, O, seed)
    gu_p, gu_s = util.make_weight(2 * I, H, seed=seed + 1)
    order = nvfp4_tp.interleave_rows(I)
    d_gu_p, d_gu_s = util.to_dev(np.ascontiguousarray(gu_p[order])), util.to_dev(np.ascontiguousarray(gu_s[order]))
    dn_p, dn_s, d_dn_p, d_dn_s = _dev_weight(H, I, seed + 2)
    w = util.make_bf16((H,), seed=seed + 3, std=0.3)
    bufs = dict(attn=torch.zeros((M, O), dtype=torch.int16, device="cuda"), hid=torch.zeros((M, H), dtype=torch.int16, device="cuda"),
                hid2=torch.zeros((M, H), dtype=torch.int16, device="cuda"), act=torch.zeros((M, I), dtype=torch.int16, device="cuda"),
                out=torch.zeros((M, H), dtype=torch.int16, device="cuda"), w=util.to_dev(w))
    descs = [dict(A=bufs["attn"], M=M, packed=d_o_p, scale=d_o_s, N=H, K=O, C=bufs["hid2"], residual=bufs["hid"]),
             dict(A=bufs["hid2"], M=M, packed=d_gu_p, scale=d_gu_s, N=2 * I, K=H, C=bufs["act"], norm_weight=bufs["w"], norm_eps=1e-6,
                  swiglu_epilogue=True),
             dict(A=bufs["act"], M=M, packed=d_dn_p, scale=d_dn_s, N=H, K=I, C=bufs["out"], residual=bufs["hid2"])]
    host = dict(o=(o_p, o_s), gu=(gu_p, gu_s), dn=(dn_p, dn_s), w=w)
    return bufs, descs, host


def _layer_oracle(host, attn, hid):
    hid2 = ob.linear(attn, *host["o"], 1.0, residual=hid, mode=ob.GEMV, threads=8)
    act = ob.swiglu_merged(ob.linear(ob.rmsnorm(hid2, host["w"], 1e-6), *host["gu"], 1.0, mode=ob.GEMV, threads=8))
    return ob.linear(act, *host["dn"], 1.0, residual=hid2, mode=ob.GEMV, threads=8)


@pytest.mark.parametrize("M", [1, 4])
def test_chain_decode_layer_sequence(handle, M):
    """Each linear reads what the previous one wrote: the chain against the same three calls issued one by
    one (identical bits) and against the oracle's sequence."""
    import torch
    H, I, O = 1024, 2304, 1536
    bufs, descs, host = _layer(handle, torch, M, H, I, O, seed=50)
    attn, hid = util.make_bf16((M, O), seed=60), util.make_bf16((M, H), seed=61)
    bufs["attn"].copy_(util.to_dev(attn))
    bufs["hid"].copy_(util.to_dev(hid))
    handle.set_option("decode_impl", 2)                        # one by one, through the chain's own kernel
    try:
        for d in descs:
            handle.linear_ex(d["A"], M, d["packed"], d["scale"], 1.0, d["N"], d["K"], d["C"], residual=d.get("residual"),
                             norm_weight=d.get("norm_weight"), norm_eps=d.get("norm_eps", 0.0), swiglu_epilogue=d.get("swiglu_epilogue", False))
    finally:
        handle.set_option("decode_impl", 0)
    torch.cuda.synchronize()
    single = bufs["out"].clone()
    for k in ("hid2", "act", "out"):
        bufs[k].fill_(0x7FC0)
    chain = nvfp4.Chain(handle, descs)
    try:
        chain.run()
        torch.cuda.synchronize()
        assert torch.equal(bufs["out"], single)
        assert ob.rel_frobenius(util.to_host_u16(bufs["out"]), _layer_oracle(host, attn, hid)) <= 2e-3     # SwiGLU amplifies last-bit differences
    finally:
        chain.close()
    assert handle.device_status() == 0


def test_chain_graph_replay_with_new_inputs(handle):
    """A captured chain replayed 200 times, the input buffers overwritten before every replay: every replay
    equals the eager run on the same inputs (barrier counter and split-tile tags live in device memory)."""
    import torch
    M, H, I, O = 2, 1024, 2304, 1536
    bufs, descs, host = _layer(handle, torch, M, H, I, O, seed=70)
    chain = nvfp4.Chain(handle, descs)
    try:
        inputs = [(util.to_dev(util.make_bf16((M, O), seed=80 + i, std=[1.0, 0.3, 3.0][i % 3])),
                   util.to_dev(util.make_bf16((M, H), seed=90 + i))) for i in range(6)]
        eager = []
        for a, h0 in inputs:
            bufs["attn"].copy_(a)
            bufs["hid"].copy_(h0)
            chain.run()
            torch.cuda.synchronize()
            eager.append(bufs["out"].clone())
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            chain.run(s)
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            chain.run(torch.cuda.current_stream())
        bad = []
        for r in range(200):
            i = (r * 5 + 1) % len(inputs)
            bufs["attn"].copy_(inputs[i][0])
            bufs["hid"].copy_(inputs[i][1])
            bufs["out"].fill_(0x7FC0)
            g.replay()
            if not torch.equal(bufs["out"], eager[i]):
                bad.append(r)
        torch.cuda.synchronize()
        assert not bad, f"{len(bad)} replays differ, first at {bad[:5]}"
    finally:
        chain.close()
    assert handle.device_status() == 0


def test_chain_of_many_layers(handle):
    """Twelve layers back to back in one launch (36 linears): the residual stream runs through all of them."""
    import torch
    M, H, I, O, L = 2, 512, 768, 512, 12
    layers = [_layer(handle, torch, M, H, I, O, seed=100 + 10 * l) for l in range(L)]
    descs = []
    for l, (bufs, d, host) in enumerate(layers):
        if l > 0:                                                  # the layer's input stream is the previous layer's output
            d[0]["residual"] = layers[l - 1][0]["out"]
        descs += d
    attn = [util.make_bf16((M, O), seed=200 + l, std=0.5) for l in range(L)]
    hid = util.make_bf16((M, H), seed=300)
    for l in range(L):
        layers[l][0]["attn"].copy_(util.to_dev(attn[l]))
    layers[0][0]["hid"].copy_(util.to_dev(hid))
    chain = nvfp4.Chain(handle, descs)
    try:
        chain.run()
        torch.cuda.synchronize()
        want = hid
        for l in range(L):
            want = _layer_oracle(layers[l][2], attn[l], want)
        assert ob.rel_frobenius(util.to_host_u16(layers[-1][0]["out"]), want) <= 5e-3      # twelve layers of compounding last-bit differences
        first = layers[-1][0]["out"].clone()
        chain.run()
        torch.cuda.synchronize()
        assert torch.equal(layers[-1][0]["out"], first)
    finally:
        chain.close()
    assert handle.device_status() == 0


def test_chain_refuses_what_the_kernel_does_not_take(handle):
    import torch
    p, s, dp, ds = _dev_weight(256, 512, seed=1)
    A = torch.zeros((9, 512), dtype=torch.int16, device="cuda")
    C = torch.zeros((9, 256), dtype=torch.int16, device="cuda")
    with pytest.raises(nvfp4.Nvfp4Error) as e:
        nvfp4.Chain(handle, [dict(A=A, M=9, packed=dp, scale=ds, N=256, K=512, C=C)])      # more than 8 tokens
    assert e.value.status == -10
    p2, s2, dp2, ds2 = _dev_weight(256, 48, seed=2)
    with pytest.raises(nvfp4.Nvfp4Error) as e:
        nvfp4.Chain(handle, [dict(A=A, M=1, packed=dp2, scale=ds2, N=256, K=48, C=C)])     # K not a multiple of 256
    assert e.value.status == -10
