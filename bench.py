#!/usr/bin/env python
"""Benchmark of the NVFP4 W4A16 linear layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sections a,b]

One JSON line on stdout (rank 0).  The headline workload is the decode batch sweep of the
27B-class MLP shapes: one "step" is, for each M in {1,2,4,8,16}, the fused gate/up linear
(K=5120, N=34816) followed by the down linear (K=17408, N=5120) -- ten launches of the
dequant-GEMV.  `value` is algorithmic bytes per step / device time per step, weights and
activations resident in HBM; weights rotate over several distinct copies larger than L2.
With N > 1 GPUs the same sweep runs as the tensor-parallel MLP (gate/up column-split, SwiGLU,
down row-split, one all-reduce), total work fixed ("strong").

`--impl reference` times the CPU restatement of the reference's algorithm (the oracle port,
all host threads) on a bounded sample of the same workload: the reference engine has no CPU
implementation of this path and its kernels are built for Jetson Thor only.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "qwen3-27b-thor-runner_b200"), os.path.join(ROOT, "oracle"),
           os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOAD = "configs[1]: decode sweep M in {1,2,4,8,16}, gate_up 34816x5120 + down 5120x17408"
H, I = 5120, 17408
SHAPES = {"gate_up": (2 * I, H), "down": (H, I), "qkv": (7168, 5120), "o": (5120, 6144)}   # name -> (N, K)
DECODE_MS = (1, 2, 4, 8, 16)
# dram__bytes_read.sum + dram__bytes_write.sum of one gate_up call at M = 1 (algorithmic: 100.35 MB), from one
# ncu capture per kernel: the NVFP4 tensor-core GEMV with its pre-pass, and the mma.sync GEMV
NCU_TRAFFIC_GATE_UP_M1 = {"fp4": 106466560, "mma": 106047744}
L2_BYTES = 126 << 20


def alg_bytes(N, K, M, residual=False):
    return N * K // 2 + N * K // 16 + 2 * M * K + 2 * M * N * (2 if residual else 1)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """nvidia-smi clock / throttle-reason sampling during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.split(",") for r in open(self.f.name).read().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.f.name)
        sm, reasons = [], set()
        for r in rows:
            r = [x.strip() for x in r]
            try:
                sm.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


# ----------------------------------------------------------------------------- synthetic data (device)

def device_weight(N, K, seed, dev):
    """Nibbles uniform over the 16 codes; block scale = E4M3(max|w|/6), w ~ N(0, 0.02) x16 (sigma 0.02)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=g)
    scale = torch.empty((N, K // 16), dtype=torch.uint8, device=dev)
    rows = max(1, (64 << 20) // (K * 4))
    for r0 in range(0, N, rows):
        r1 = min(N, r0 + rows)
        w = torch.randn((r1 - r0, K // 16, 16), device=dev, generator=g) * 0.02
        s = w.abs().amax(dim=-1) / 6.0
        scale[r0:r1] = s.to(torch.float8_e4m3fn).view(torch.uint8)
    return packed, scale


def device_acts(M, K, seed, dev):
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)


# ----------------------------------------------------------------------------- CPU baseline (oracle port)

_CPU_DATA = {}   # synthetic host tensors of the CPU baseline, generated once


def cpu_baseline_sweep(seconds_hint=15.0):
    """Times the oracle (scalar C port of the reference algorithm) on the host cores: the decode
    sweep M in {1,2,4,8,16} over both MLP shapes (all rows), rows split over all threads, repeated
    until about `seconds_hint` seconds of CPU work (threads x wall time) have been spent."""
    import numpy as np
    import oracle_binding as ob
    import util
    threads = os.cpu_count() or 1
    data = _CPU_DATA
    for name in ("gate_up", "down"):
        if name in data:
            continue
        N, K = SHAPES[name]
        packed, scale = util.make_weight(N, K, seed=0)
        data[name] = (packed, scale, {M: util.make_bf16((M, K), seed=M) for M in DECODE_MS})
    nbytes, t_total, reps = 0, 0.0, 0
    while reps == 0 or (t_total * threads < seconds_hint and reps < 50):
        for name in ("gate_up", "down"):
            N, K = SHAPES[name]
            packed, scale, acts = data[name]
            for M in DECODE_MS:
                t0 = time.perf_counter()
                ob.linear(acts[M], packed, scale, 1.0, mode=ob.GEMV, threads=threads)
                t_total += time.perf_counter() - t0
                nbytes += alg_bytes(N, K, M)
        reps += 1
    return dict(value=nbytes / t_total / 1e9, unit="GB/s", cores=threads, kind="port",
                sample=f"{reps} x decode sweep M in {{1,2,4,8,16}} on gate_up 34816x5120 + down 5120x17408 (all rows), "
                       f"{t_total:.1f} s wall on {threads} threads = {t_total * threads:.0f} s of CPU work"), t_total


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    per = max(4.0, min(20.0, 150.0 / (steps + args.warmup)))   # CPU-seconds per step: the whole run stays in minutes
    for _ in range(args.warmup):
        cpu_baseline_sweep(1.0)
    vals, tt = [], 0.0
    for _ in range(steps):
        cb, t = cpu_baseline_sweep(per)
        vals.append(cb["value"])
        tt += t
    cb["value"] = sum(vals) / len(vals)
    line = {"impl": "reference", "metric": "decode_gemv_hbm_gbs", "value": cb["value"], "unit": "GB/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * tt / steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x nvfp4 -> fp32 acc",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "arm": "CPU oracle port of the reference algorithm, all rows of both shapes, all host threads"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------- our arm

def sweep_parity(h, shapes, rot, acts, outs, torch, n_rows=64):
    """Relative Frobenius error of every timed (shape, M) of the sweep against the CPU oracle on a seeded
    sample of weight rows: the timed kernels on the timed buffers, launched once more and read back."""
    import numpy as np
    import oracle_binding as ob
    import util
    out, worst = [], 0.0
    for name in rot:
        N, K = shapes[name]
        p, s = rot[name].w[0]
        rows = np.sort(np.random.default_rng(N).choice(N, min(N, n_rows), replace=False))
        r_idx = torch.from_numpy(rows).to(p.device)
        hp, hs = p[r_idx].cpu().numpy(), s[r_idx].cpu().numpy()
        for M in DECODE_MS:
            A, C = acts[(name, M)], outs[(name, M)]
            C.zero_()
            h.linear(A, M, p, s, 1.0, N, K, C)
            torch.cuda.synchronize()
            got = util.to_host_u16(C[:, r_idx].contiguous().view(torch.int16))
            want = ob.linear(util.to_host_u16(A.view(torch.int16)), np.ascontiguousarray(hp), np.ascontiguousarray(hs), 1.0,
                             mode=ob.GEMV, threads=8)
            err = float(ob.rel_frobenius(got, want))
            worst = max(worst, err)
            out.append({"shape": name, "M": M, "rel_frobenius": round(err, 7)})
    return {"checked": f"{n_rows} sampled weight rows per shape, all tokens, vs the CPU oracle (FP32 accumulate, one rounding)",
            "tolerance": 1e-3, "worst": round(worst, 7), "ok": worst <= 1e-3, "rows": out, "device_status": h.device_status()}


def config0(h, peaks, torch, dev, use_graph, steps):
    """configs[0]: one GEMV, M = 1, K = N = 5120 (14.7 MB of weights): time over rotating copies and the
    whole output against the CPU oracle."""
    import numpy as np
    import oracle_binding as ob
    import util
    N = K = 5120
    rot = Rotating(N, K, dev, seed=50)
    A = device_acts(1, K, seed=0, dev=dev)
    C = torch.empty((1, N), dtype=torch.bfloat16, device=dev)

    def go():
        p, s = rot.next()
        h.linear(A, 1, p, s, 1.0, N, K, C, stream=torch.cuda.current_stream())

    for _ in range(3):
        go()
    st = {}
    time_region(go, max(steps, 20), torch, graph=use_graph, stats=st)
    p, s = rot.w[0]
    h.linear(A, 1, p, s, 1.0, N, K, C)
    torch.cuda.synchronize()
    want = ob.linear(util.to_host_u16(A.view(torch.int16)), p.cpu().numpy(), s.cpu().numpy(), 1.0, mode=ob.GEMV, threads=8)
    err = float(ob.rel_frobenius(util.to_host_u16(C.view(torch.int16)), want))
    gbs = alg_bytes(N, K, 1) / (st["median_ms"] * 1e-3) / 1e9
    return {"workload": "configs[0]: M=1, K=5120, N=5120", "us": round(st["median_ms"] * 1e3, 2), "us_min": round(st["min_ms"] * 1e3, 2),
            "replays": st["replays"], "cv": round(st["cv"], 4), "GBps": round(gbs, 1),
            "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4), "rel_frobenius_vs_oracle": round(err, 7),
            "copies": rot.n}


class Rotating:
    """Distinct device copies of one weight, used round-robin so that no launch finds its
    weights in L2 (total footprint >= 2 x L2)."""

    def __init__(self, N, K, dev, seed):
        per = N * K // 2 + N * K // 16
        self.n = max(2, -(-2 * L2_BYTES // per) + 1)
        self.w = [device_weight(N, K, seed + i, dev) for i in range(self.n)]
        self.i = 0

    def next(self):
        self.i = (self.i + 1) % self.n
        return self.w[self.i]


def time_region(fn, steps, torch, graph=True, replays=50, stats=None, budget_s=0.4, exact_replays=None):
    """Device time per call of fn (ms).  graph=True: `steps` calls are captured into one CUDA graph (the
    library's launches are capturable: no allocation, no synchronisation) and the graph is replayed
    `replays` times (fewer when one replay is long: the timed replays together stay near budget_s, at
    least 5), each replay between its own pair of events; the MEDIAN replay is reported, so the figure is
    free of host launch overhead and of a single outlier.  `stats`, when given, receives the number of
    timed replays, their median, minimum and coefficient of variation (per call, ms).  graph=False: the
    calls are issued on the stream between one pair of events.
    exact_replays: replay exactly that many times, whatever one replay takes.  Ranks whose calls contain
    a collective or wait for each other's kernels MUST pass it: a count derived from a rank's own clock
    can differ between the ranks, and the rank that replays once more waits for peers that have stopped."""
    if graph:
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for _ in range(steps):
                    fn()
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            first = e0.elapsed_time(e1)
            n = int(max(5, min(replays, budget_s * 1e3 / max(first, 1e-3)))) if exact_replays is None else int(exact_replays)
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
            for a, b in ev:
                a.record()
                g.replay()
                b.record()
        torch.cuda.synchronize()
        t = sorted(a.elapsed_time(b) / steps for a, b in ev)
        med = t[len(t) // 2]
        if stats is not None:
            mean = sum(t) / len(t)
            var = sum((x - mean) ** 2 for x in t) / len(t)
            stats.update({"replays": len(t), "median_ms": med, "min_ms": t[0], "cv": (var ** 0.5) / mean if mean else 0.0})
        return med
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if stats is not None:
        stats.update({"replays": 1, "median_ms": ms, "min_ms": ms, "cv": 0.0})
    return ms   # ms per step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sections", default="decode,parity,config0,prefill,stream,mlp,dense,e2e,cpu,refkernel,tp",
                    help="extra measurements to add to the JSON line")
    ap.add_argument("--small", action="store_true", help="shrunk shapes (profiler captures, smoke runs)")
    ap.add_argument("--prefill-ms", default="64,256,2048,8192", help="token counts of the prefill section")
    ap.add_argument("--decode-ms", default="", help="token counts of the decode sweep (default: the five of configs[1]); "
                                                    "a single value gives a profiler a known launch")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="kernel-selection option set on the handle (nvfp4_set_option), e.g. skinny_min_m=1")
    ap.add_argument("--no-graph", action="store_true", help="time stream launches instead of a CUDA-graph replay")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.decode_ms:
        globals()["DECODE_MS"] = tuple(int(x) for x in args.decode_ms.split(","))
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import nvfp4

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 or args.gpus > 1:
        import bench_tp
        return bench_tp.main(args, world, rank, local_rank)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    sections = set(args.sections.split(","))
    peaks = load_peaks()
    shapes = dict(SHAPES)
    if args.small:
        shapes = {"gate_up": (34816 // 4, 5120), "down": (5120, 17408 // 4), "qkv": (7168, 5120), "o": (5120, 6144)}
    h = nvfp4.Handle(0, 1 << 30)
    for kv in args.option:
        name, _, val = kv.partition("=")
        h.set_option(name, int(val))
    stream = torch.cuda.current_stream()

    rot = {name: Rotating(*shapes[name], dev, seed=10 * i) for i, name in enumerate(("gate_up", "down"))}
    acts = {(name, M): device_acts(M, shapes[name][1], seed=M, dev=dev) for name in rot for M in DECODE_MS}
    outs = {(name, M): torch.empty((M, shapes[name][0]), dtype=torch.bfloat16, device=dev)
            for name in rot for M in DECODE_MS}

    def launch(name, M):
        N, K = shapes[name]
        p, s = rot[name].next()
        h.linear(acts[(name, M)], M, p, s, 1.0, N, K, outs[(name, M)], stream=torch.cuda.current_stream())

    def step():
        for M in DECODE_MS:
            launch("gate_up", M)
            launch("down", M)

    step_bytes = sum(alg_bytes(*shapes[n], M) for n in rot for M in DECODE_MS)
    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(0)
    sampler.start()
    use_graph = not args.no_graph
    l0 = h.launch_count()
    value_stats = {}
    ms = time_region(step, args.steps, torch, graph=use_graph, stats=value_stats)
    launches = (h.launch_count() - l0)   # kernels launched by the K steps (= kernels in ONE timed replay)
    # Second pass, same launches regrouped: for every (shape, M) the `steps` launches of the timed
    # region run back to back between one event pair (weights still rotate), which gives the
    # kernel's average launch duration without an event gap between launches.
    per = {}
    for M in DECODE_MS:
        for name in ("gate_up", "down"):
            launch(name, M)
            st = {}
            time_region(lambda: launch(name, M), args.steps, torch, graph=use_graph, stats=st)
            per[(name, M)] = st
    clocks = sampler.stop()
    value = step_bytes / (ms * 1e-3) / 1e9

    sweep = []
    for (name, M), st in sorted(per.items()):
        t = st["median_ms"] * 1e-3
        gbs = alg_bytes(*shapes[name], M) / t / 1e9
        sweep.append({"shape": name, "M": M, "us": round(t * 1e6, 2), "us_min": round(st["min_ms"] * 1e3, 2),
                      "replays": st["replays"], "cv": round(st["cv"], 4),
                      "GBps": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4),
                      "frac_of_8TBps": round(gbs / 8000.0, 4)})
    # Dominant kernel: the GEMV kernel on gate_up.  Token counts above 9 go through another kernel
    # (see decode_sweep), so the roofline object averages the launches of M <= 8.
    gu = [x for x in sweep if x["shape"] == "gate_up" and x["M"] <= 8] or [x for x in sweep if x["shape"] == "gate_up"]
    ach = sum(alg_bytes(*shapes["gate_up"], x["M"]) for x in gu) / sum(x["us"] * 1e-6 for x in gu) / 1e9
    fp4 = h.get_option("fp4_native") == 1 and h.get_option("decode_impl") in (0, 3)
    roofline = {"bound": "hbm",
                "kernel": ("decode GEMV on the NVFP4 tensor-core path (decode_fp4_kernel; its launch time includes the activation "
                           "pre-pass act_to_fp4_kernel in front of it)" if fp4 else "decode GEMV (decode_mma_kernel)")
                          + ", gate_up 34816x5120, mean over its calls at M in " + str([x["M"] for x in gu]),
                "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "peak_source": peaks["source"],
                "unit": "GB/s", "frac": round(ach / peaks["hbm_gbs"], 4),
                "traffic": None if args.small else NCU_TRAFFIC_GATE_UP_M1["fp4" if fp4 else "mma"]}
    line = {"metric": "decode_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x nvfp4 -> fp32 acc", "data": "synthetic",
            "config": {"workload": WORKLOAD
                                   + (" (SMALL shapes)" if args.small else "")
                                   + (f" (M restricted to {list(DECODE_MS)})" if args.decode_ms else ""),
                       "l2": f"weights rotate over {rot['gate_up'].n}/{rot['down'].n} distinct copies (> 2 x L2)",
                       "global_scale": 1.0, "scale_sigma": 0.02, "seed": 0,
                       "timing": (f"median of {value_stats.get('replays')} CUDA-graph replays of the K steps" if use_graph
                                  else "K steps of stream launches"),
                       "decode_impl": h.get_option("decode_impl"), "prefill_impl": h.get_option("prefill_impl"),
                       "options": args.option},
            "roofline": roofline, "clocks": clocks, "gpu_launches": int(launches), "decode_sweep": sweep,
            "consistency": {"timed_replays": value_stats.get("replays"), "ms_per_step_min": round(value_stats.get("min_ms", ms), 5),
                            "cv": round(value_stats.get("cv", 0.0), 4)}}
    if "parity" in sections:
        line["parity"] = sweep_parity(h, shapes, rot, acts, outs, torch)
    if "config0" in sections and not args.small:
        line["config0"] = config0(h, peaks, torch, dev, use_graph, args.steps)

    if "e2e" in sections:
        import bench_sections
        line["e2e"] = bench_sections.e2e(h, shapes, rot, args, torch, alg_bytes, DECODE_MS)
    if "prefill" in sections:
        import bench_sections
        line["prefill"] = bench_sections.prefill(h, shapes, rot, peaks, torch, small=args.small,
                                                  ms_list=tuple(int(x) for x in args.prefill_ms.split(",")))
    if "stream" in sections and not args.small:
        import bench_sections
        line["layer_stream"] = bench_sections.layer_stream(h, SHAPES, peaks, torch, alg_bytes)
    if "mlp" in sections and not args.small:
        import bench_sections
        line["mlp_block"] = bench_sections.mlp_block(h, shapes, rot, torch)
    if "dense" in sections and not args.small:
        import bench_sections
        line["dense_bf16_gemv"] = bench_sections.dense_bf16(h, peaks, torch)
    if "refkernel" in sections:
        import bench_sections
        line["reference_kernels_on_this_gpu"] = bench_sections.reference_kernels(shapes, rot, acts, outs, torch,
                                                                                 alg_bytes, DECODE_MS)
    if "tp" in sections and not args.small:
        # configs[4] at one GPU: the MLP block (gate_up -> SwiGLU -> down), the base of the 2/4/8-GPU runs
        import bench_tp
        import nvfp4_tp
        comm1 = nvfp4_tp.Comm(None, 0, 1)

        def make_one(max_M):
            out = []
            for c in range(3 if max_M <= 256 else 2):
                gp, gs = device_weight(2 * I, H, seed=100 + 2 * c, dev=dev)
                dp, ds = device_weight(H, I, seed=101 + 2 * c, dev=dev)
                out.append(nvfp4_tp.TpMlp(h, comm1, H, I, gp, gs, 1.0, dp, ds, 1.0, max_M))
            return out

        line["tp_mlp"] = bench_tp.run_tp_mlp_table(torch, None, make_one, H, dev, 1, args.steps)
        line["tp_layer_stream"] = bench_tp.run_tp_layer_stream(torch, None, h, comm1, dev, 1)
        comm1.close()
    if "cpu" in sections:
        line["cpu_baseline"], _ = cpu_baseline_sweep(15.0)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
