"""Secondary measurements of bench.py: the end-to-end host-buffer path, the prefill sweep,
the 64-layer weight stream and the reference engine's own kernels on the same GPU."""
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))


def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def e2e(h, shapes, rot, args, torch, alg_bytes, decode_ms):
    """The decode sweep through nvfp4_linear_host: activations start in pinned HOST memory and
    outputs end there; every call copies H2D, launches, gets its outputs into host memory (a copy back, or
    the kernels' own stores into the pinned buffer) and synchronises."""
    hin, hout = {}, {}
    for name in rot:
        N, K = shapes[name]
        for M in decode_ms:
            hin[(name, M)] = torch.randn((M, K)).to(torch.bfloat16).pin_memory()
            hout[(name, M)] = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream()

    def step():
        for M in decode_ms:
            for name in ("gate_up", "down"):
                N, K = shapes[name]
                p, s = rot[name].next()
                h.linear_host(hin[(name, M)], M, p, s, 1.0, N, K, hout[(name, M)], stream=stream)

    for _ in range(3):
        step()
    e0, e1 = _events(torch)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    step_bytes = sum(alg_bytes(*shapes[n], M) for n in rot for M in decode_ms)
    h2d = sum(hin[k].numel() * 2 for k in hin)
    d2h = sum(hout[k].numel() * 2 for k in hout)
    return {"value": round(step_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(ms, 4),
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "api": "nvfp4_linear_host (pinned host activations copied in; the outputs end in pinned host memory, written "
                   "there by the kernels themselves over PCIe -- no residual in this sweep -- and are complete when the call "
                   "returns; weights device-resident)"}


def prefill(h, shapes, rot, peaks, torch, small=False, ms_list=(64, 256, 2048, 8192)):
    """configs[2]: M in {64,256,2048,8192} on the two MLP shapes; TFLOP/s = 2*M*N*K / time."""
    dev = torch.device("cuda:0")
    fast = True
    out = []
    for name in ("gate_up", "down"):
        N, K = shapes[name]
        for M in ms_list:
            A = torch.randn((M, K), device=dev).to(torch.bfloat16)
            C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            p, s = rot[name].next()
            st = h.linear(A, M, p, s, 1.0, N, K, C, check=False)
            if st != 0:
                out.append({"shape": name, "M": M, "error": int(st)})
                continue
            torch.cuda.synchronize()
            # one launch tells how long this path takes; slow (debug) paths are measured once only
            e0, e1 = _events(torch)
            e0.record()
            h.linear(A, M, *rot[name].next(), 1.0, N, K, C)
            e1.record()
            torch.cuda.synchronize()
            t1 = e0.elapsed_time(e1)
            iters = 1 if t1 > 200 else max(3, min(20, int(200 / max(t1, 1e-3))))
            # `iters` calls captured in one CUDA graph: the small-M launches are shorter than the
            # host's time to issue them
            import bench
            ms = bench.time_region(lambda: h.linear(A, M, *rot[name].next(), 1.0, N, K, C, check=False), iters, torch,
                                   graph=(t1 <= 200))
            tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            # the same calls with the leftover tiles kept whole (no split along K), for comparison
            h.set_option("prefill_stream_k", 0)
            ms_whole = bench.time_region(lambda: h.linear(A, M, *rot[name].next(), 1.0, N, K, C, check=False), iters,
                                         torch, graph=(t1 <= 200))
            h.set_option("prefill_stream_k", 1)
            out.append({"shape": name, "M": M, "ms": round(ms, 4), "TFLOPs": round(tf, 1),
                        "ms_whole_tiles_only": round(ms_whole, 4),
                        "frac_of_measured_bf16_burst": round(tf / peaks["bf16_tflops"], 4),
                        "frac_of_measured_bf16_sustained": round(tf / peaks["bf16_tflops_sustained"], 4),
                        "frac_of_2250_nominal": round(tf / 2250.0, 4)})
            if ms > 2000:
                fast = False
            del A, C
            if not fast:
                break
    return out


def layer_stream(h, SHAPES, peaks, torch, alg_bytes, layers=64):
    """configs[3]: 64 layers x {qkv, o, gate_up, down}, every tensor distinct (12.08 GB of weights),
    M in {1,2,4}: time per token-step of all 256 linears and sustained GB/s."""
    import bench
    dev = torch.device("cuda:0")
    names = ("qkv", "o", "gate_up", "down")
    ws = []
    for l in range(layers):
        ws.append({n: bench.device_weight(*SHAPES[n], seed=1000 + 4 * l + i, dev=dev) for i, n in enumerate(names)})
    res = []
    for M in (1, 2, 4):
        acts = {n: bench.device_acts(M, SHAPES[n][1], seed=M, dev=dev) for n in names}
        outs = {n: torch.empty((M, SHAPES[n][0]), dtype=torch.bfloat16, device=dev) for n in names}

        def token_step():
            for l in range(layers):
                for n in names:
                    N, K = SHAPES[n]
                    p, s = ws[l][n]
                    h.linear(acts[n], M, p, s, 1.0, N, K, outs[n])

        token_step()
        ms = bench.time_region(token_step, 3, torch, graph=True)
        nbytes = layers * sum(alg_bytes(*SHAPES[n], M) for n in names)
        gbs = nbytes / (ms * 1e-3) / 1e9
        row = {"M": M, "ms_per_token_step": round(ms, 4), "GBps": round(gbs, 1),
               "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4), "frac_of_8TBps": round(gbs / 8000.0, 4),
               "launch_mode": "CUDA-graph replay of 3 token-steps (768 launches)"}
        # the same 256 linears as ONE launch: nvfp4_chain (grid-wide barrier between linears, the loader
        # streaming the next linear's weights across it)
        import nvfp4
        chain = nvfp4.Chain(h, [dict(A=acts[n], M=M, packed=ws[l][n][0], scale=ws[l][n][1], N=SHAPES[n][0], K=SHAPES[n][1], C=outs[n])
                                for l in range(layers) for n in names])
        chain.run()
        torch.cuda.synchronize()
        ms_c = bench.time_region(chain.run, 3, torch, graph=True)
        chain.close()
        gbs_c = nbytes / (ms_c * 1e-3) / 1e9
        row.update({"chain_ms_per_token_step": round(ms_c, 4), "chain_GBps": round(gbs_c, 1),
                    "chain_frac_of_measured_hbm": round(gbs_c / peaks["hbm_gbs"], 4),
                    "chain_launch_mode": "one nvfp4_chain launch per token-step (256 linears), CUDA-graph replay of 3"})
        res.append(row)
    del ws
    torch.cuda.empty_cache()
    return res


def mlp_block(h, shapes, rot, torch, tokens=(1, 2, 4, 8)):
    """One decode MLP block of a layer, src/engine/layer.cu:47-110: RMSNorm -> gate_up -> SwiGLU -> down
    + residual, as four launches (the reference's sequence), with the norm formed in the gate_up
    GEMV's staging and, up to four tokens, the SwiGLU in the down GEMV's (two launches), and with the
    SwiGLU in the gate_up GEMV's epilogue (gate/up rows interleaved at load time; two launches).
    CUDA-graph timed; the weights rotate over copies larger than L2."""
    import bench
    dev = torch.device("cuda:0")
    (N1, K1), (N2, K2) = shapes["gate_up"], shapes["down"]
    I = N1 // 2
    w = bench.device_acts(1, K1, seed=77, dev=dev).reshape(-1)
    out = []
    for M in tokens:
        X = bench.device_acts(M, K1, seed=M, dev=dev)
        Xn = torch.empty_like(X)
        gu = torch.empty((M, N1), dtype=torch.bfloat16, device=dev)
        act = torch.empty((M, I), dtype=torch.bfloat16, device=dev)
        Y = torch.empty((M, N2), dtype=torch.bfloat16, device=dev)

        def separate():
            p1, s1 = rot["gate_up"].next()
            p2, s2 = rot["down"].next()
            h.rmsnorm(X, w, 1e-6, M, K1, Xn)
            h.linear(Xn, M, p1, s1, 1.0, N1, K1, gu)
            h.swiglu(gu, None, M, I, act)
            h.linear(act, M, p2, s2, 1.0, N2, K2, Y, residual=X)

        def fused():
            p1, s1 = rot["gate_up"].next()
            p2, s2 = rot["down"].next()
            h.linear_ex(X, M, p1, s1, 1.0, N1, K1, gu, norm_weight=w, norm_eps=1e-6)
            if M <= 4:
                h.linear_ex(gu, M, p2, s2, 1.0, N2, K2, Y, residual=X, swiglu_up=gu[:, I:], a_row_stride=2 * I)
            else:
                h.swiglu(gu, None, M, I, act)
                h.linear(act, M, p2, s2, 1.0, N2, K2, Y, residual=X)

        def fused_epilogue():
            # gate/up rows interleaved at load time: SwiGLU in the gate_up epilogue, two launches for any M <= 8
            p1, s1 = rot["gate_up"].next()          # timing only: the row order does not change the work
            p2, s2 = rot["down"].next()
            h.linear_ex(X, M, p1, s1, 1.0, N1, K1, act, norm_weight=w, norm_eps=1e-6, swiglu_epilogue=True)
            h.linear(act, M, p2, s2, 1.0, N2, K2, Y, residual=X)

        # the same two linears as one launch (nvfp4_chain), one chain per pairing of the rotating weight copies
        import nvfp4
        nch = max(rot["gate_up"].n, rot["down"].n)
        chains = [nvfp4.Chain(h, [dict(A=X, M=M, packed=rot["gate_up"].w[i % rot["gate_up"].n][0], scale=rot["gate_up"].w[i % rot["gate_up"].n][1],
                                       N=N1, K=K1, C=act, norm_weight=w, norm_eps=1e-6, swiglu_epilogue=True),
                                  dict(A=act, M=M, packed=rot["down"].w[i % rot["down"].n][0], scale=rot["down"].w[i % rot["down"].n][1],
                                       N=N2, K=K2, C=Y, residual=X)]) for i in range(nch)]
        state = {"i": 0}

        def chained():
            state["i"] = (state["i"] + 1) % nch
            chains[state["i"]].run()

        row = {"M": M}
        for name, fn in (("ms_four_launches", separate), ("ms_fused_prologues", fused),
                         ("ms_norm_prologue_swiglu_epilogue", fused_epilogue), ("ms_chain_one_launch", chained)):
            fn(); fn()
            row[name] = round(bench.time_region(fn, 6, torch, graph=True), 5)
        for c in chains:
            c.close()
        out.append(row)
    return out


def dense_bf16(h, peaks, torch, tokens=(1, 4, 8), gemm_tokens=(256, 2048)):
    """BF16-weight GEMV (the tensors a quantised checkpoint keeps in BF16): the lm_head [248320, 5120]
    (2.54 GB, far larger than L2) and a 5120 x 5120 projection rotating over copies larger than L2.
    CUDA-graph timed; GB/s counts weight + activation + output bytes."""
    import bench
    dev = torch.device("cuda:0")
    out = []
    for name, N, K, copies in (("lm_head", 248320, 5120, 1), ("proj_5120", 5120, 5120, 6)):
        ws = [(torch.randn((N, K), device=dev, generator=torch.Generator(device=dev).manual_seed(40 + i)) * 0.02).to(torch.bfloat16)
              for i in range(copies)]
        for M in tokens:
            A = bench.device_acts(M, K, seed=M, dev=dev)
            C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            st = {"i": 0}

            def go():
                st["i"] = (st["i"] + 1) % copies
                h.linear_bf16(A, M, ws[st["i"]], N, K, C)

            go(); go()
            ms = bench.time_region(go, 6, torch, graph=True)
            nbytes = 2 * N * K + 2 * M * K + 2 * M * N
            gbs = nbytes / (ms * 1e-3) / 1e9
            out.append({"shape": name, "N": N, "K": K, "M": M, "us": round(ms * 1e3, 2), "GBps": round(gbs, 1),
                        "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4)})
        if name == "proj_5120":
            for M in gemm_tokens:          # the tcgen05 GEMM on the same weights
                A = bench.device_acts(M, K, seed=M, dev=dev)
                C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
                st = {"i": 0}

                def go():
                    st["i"] = (st["i"] + 1) % copies
                    h.linear_bf16(A, M, ws[st["i"]], N, K, C)

                go(); go()
                ms = bench.time_region(go, 6, torch, graph=True)
                tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
                out.append({"shape": name, "N": N, "K": K, "M": M, "us": round(ms * 1e3, 2), "TFLOPs": round(tf, 1),
                            "frac_of_measured_bf16_burst": round(tf / peaks["bf16_tflops"], 4)})
        del ws
        torch.cuda.empty_cache()
    return out


def reference_kernels(shapes, rot, acts, outs, torch, alg_bytes, decode_ms):
    """The reference engine's kernels (its own source compiled for sm_100a into oracle/_ref) on the
    same device buffers: what the reference would do on this GPU, beside ours."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_binding as ob
    if not ob.ref_available():
        return {"unavailable": "oracle/_ref/libref_fp4.so not built"}
    ref = ob.load_ref()
    st = torch.cuda.current_stream().cuda_stream
    out = []
    for name in ("gate_up", "down"):
        N, K = shapes[name]
        for M in decode_ms:
            A, C = acts[(name, M)], outs[(name, M)]

            def go():
                p, s = rot[name].next()
                ref.ref_fp4_gemm(A.data_ptr(), p.data_ptr(), s.data_ptr(), 1.0, N, K, C.data_ptr(), M, st)

            go(); go()
            e0, e1 = _events(torch)
            torch.cuda.synchronize()
            e0.record()
            iters = 5
            for _ in range(iters):
                go()
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / iters * 1e-3
            out.append({"shape": name, "M": M, "us": round(t * 1e6, 2),
                        "GBps": round(alg_bytes(N, K, M) / t / 1e9, 1)})
    return out
