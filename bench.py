#!/usr/bin/env python
"""MoE-layer throughput benchmark (the role of the reference's bench.c harness).

Workload (`config.workload`): decode through a stack of 40 DISTINCT MoE layers
(256 routed + 1 shared MXFP4 experts each, D = 2048, FF = 512, top-8), so that
every step streams fresh expert weights from HBM (about 40 x 97 MB at 8 tokens,
far above the 126 MB L2).  Each rank feeds `--tokens` (default 8) tokens per
step: one rank is the benchmark's single-GPU decode configuration at T = 8;
N ranks run the 40-layer expert-parallel decode stack with 8 N tokens per step
(64 at N = 8), experts split evenly over the ranks, dispatch and combine by
NCCL all-to-all, the shared expert on each token's home rank.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  metric = token-layers per second
(tokens x layers / time): the MoE-layer tokens/s of the benchmark definition.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, FF, E, K8, LAYERS = 2048, 512, 256, 8, 40
EXPERT_BYTES = 3 * 512 * 2048 * 17 // 32          # 1,671,168 B: gate + up + down of one expert
FLOP_PER_ASSIGNMENT = 2 * 3 * 512 * 2048          # 6,291,456
METRIC = "moe_layer_tokens_per_s"
UNIT = "token-layers/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=8, help="tokens per rank per step")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--prefill-tokens", type=int, default=4096)
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--path", default="auto", choices=["auto", "gemv", "tc"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    return ap.parse_args()


# ------------------------------------------------------------------ helpers
class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
            self.t.join(timeout=1)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops", 1647.9)), "measured"
    return 6650.0, 1590.0, "fallback"


def cpu_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# --------------------------------------------------------- CPU baseline arm
def cpu_layer_rate(tokens: int, limit_s: float):
    """The reference's CPU implementation of the path -- its C dequantiser over the three matrices of an
    expert + a plain fp32 matmul (oracle/_ref when present, else the oracle port) -- on all host cores.
    A sample of (token, expert) evaluations of one T-token layer; returns token-layers/s."""
    import numpy as np
    from oracle import oracle as O
    from q36_b200 import synth
    rng = np.random.default_rng(0)
    w = synth.layer(seed=0, n_expert=4)
    X = synth.activations(rng, tokens)
    xq, xs = O.quant_e4m3(X)
    xd = O.dequant_e4m3(xq, xs)
    cores = cpu_cores()
    t0 = time.perf_counter()
    n_eval, spent = 0, 0.0
    kind = "port"
    while spent < limit_s and n_eval < 40 * tokens * (K8 + 1):
        e = n_eval % 4
        sec, _, kind, nthr = O.cpu_expert_seconds(w["gate"][e], w["up"][e], w["down"][e], D, FF, xd[n_eval % tokens],
                                                  reps=3, threads=cores)
        n_eval += 3
        spent = time.perf_counter() - t0
    per_eval = spent / n_eval
    rate = 1.0 / (per_eval * (K8 + 1))          # one token through one layer = 9 expert evaluations
    return rate, {"value": rate, "unit": UNIT, "cores": cores, "kind": kind,
                  "sample": f"{n_eval} (token, expert) evaluations of one {tokens}-token layer in {spent:.1f} s: "
                            "C dequantiser over gate/up/down + fp32 matmul, OpenMP over rows"}, per_eval


def workload_config(NL, T, world, experts_per_rank, launch):
    """The `config` object of both arms' JSON lines."""
    return {"workload": f"decode stack: {NL} distinct MoE layers (256+1 MXFP4 experts, D=2048, FF=512, top-8), "
                        f"{T} tokens per rank per step ({world * T} global)",
            "tokens_per_rank": T, "layers": NL, "experts_per_rank": experts_per_rank,
            "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": f"inputs larger than L2: each step streams {NL} layers of distinct expert weights",
            "launch": launch}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens * args.gpus
    per_step_limit = max(0.5, min(5.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_layer_rate(T, per_step_limit / 4)
    vals, base = [], None
    t0 = time.perf_counter()
    for _ in range(args.steps):
        r, base, per_eval = cpu_layer_rate(T, per_step_limit)
        vals.append(r)
    wall = time.perf_counter() - t0
    v = sorted(vals)[len(vals) // 2]
    base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * T * args.layers / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the same workload as the GPU arm's line (a bounded sample of it per step: see cpu_baseline.sample;
        # ms_per_step extrapolates the sample to a whole step)
        "config": workload_config(args.layers, args.tokens, args.gpus, E // max(1, args.gpus), "host cores, OpenMP"),
        "cpu_baseline": base, "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": wall}))


# ------------------------------------------------------------------ GPU arm
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from q36_b200 import build as qb
    qb.build()
    from q36_b200 import moe, synth, ep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for N > 1"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T, NL = args.tokens, args.layers
    path = {"auto": moe.PATH_AUTO, "gemv": moe.PATH_GEMV, "tc": moe.PATH_TC}[args.path]
    hbm_peak, bf16_peak, peak_kind = measured_peaks()

    # ---- 40 distinct layers, this rank's expert shard, generated on the device
    se0, se1 = rank * E // world, (rank + 1) * E // world
    layers = [moe.MoELayer(se0=se0, se1=se1, device=dev).random_planes(seed=1000 + l) for l in range(NL)]
    rng = np.random.default_rng(1234 + rank)
    # one pinned host block and one device block per kind, a view per layer: a step's inputs and results cross
    # the bus in three copies
    hXa = torch.stack([torch.from_numpy(synth.activations(rng, T)).to(torch.bfloat16) for _ in range(NL)]).pin_memory()
    hLa = torch.stack([torch.from_numpy(synth.router_logits(rng, T)) for _ in range(NL)]).pin_memory()
    hOa = torch.empty((NL, T, D), dtype=torch.float32).pin_memory()
    dXa, dLa = hXa.to(dev), hLa.to(dev)
    dOa = torch.empty((NL, T, D), dtype=torch.float32, device=dev)
    dX, dL, dO = [dXa[l] for l in range(NL)], [dLa[l] for l in range(NL)], [dOa[l] for l in range(NL)]
    ws = layers[0].workspace(T)                   # one scratch, layers run back to back on one stream
    stack = ep.NativeEP(layers, world, rank, T) if world > 1 else None

    def step_device():
        if stack is not None:
            stack.step(dX, dL, dO)
        else:
            for l in range(NL):
                layers[l].forward(dX[l], dL[l], out=dO[l], path=path, ws=ws)

    def step_e2e():
        dXa.copy_(hXa, non_blocking=True)
        dLa.copy_(hLa, non_blocking=True)
        run()                                    # the same launches as the device-resident timing (graph replay at N = 1)
        hOa.copy_(dOa, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: one CUDA graph per step when single-GPU
    graph = None
    step_device()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if world == 1:     # (the expert-parallel step issues NCCL send/recv from native code and is not captured)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            step_device()
            s.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                step_device()
        torch.cuda.synchronize()
    run = (graph.replay if graph is not None else step_device)
    for _ in range(max(args.warmup, 3)):
        run()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        ev0.record()
        for _ in range(args.steps):
            run()
        ev1.record()
        barrier()
        # keep the sampler alive over at least a few samples of the same load
        t_end = time.time() + 1.0
        while time.time() < t_end:
            run()
        torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    tms = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    ms_per_step = ms / args.steps
    value = world * T * NL / (ms_per_step * 1e-3)

    # ---- end to end: pinned host inputs copied in and results copied out every step
    for _ in range(3):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(args.steps):
        step_e2e()
    ev1.record()
    barrier()
    e2e_ms = ev0.elapsed_time(ev1)
    tms = torch.tensor([e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    e2e_ms = float(tms.item()) / args.steps
    e2e = {"value": world * T * NL / (e2e_ms * 1e-3), "unit": UNIT,
           "h2d_bytes_per_step": NL * (T * D * 2 + T * (E + 1) * 4), "d2h_bytes_per_step": NL * T * D * 4,
           "ms_per_step": e2e_ms}

    # ---- roofline of the dominant kernel (gate/up: 2/3 of the expert bytes), timed launch by launch
    roof, extra = None, {}
    if world == 1:
        roof, extra = roofline_decode(moe, layers, dX, dL, T, path, hbm_peak, peak_kind, dev)

    # ---- prefill (benchmark configuration 2) on the tensor-core path
    prefill = None
    if world == 1 and not args.no_prefill:
        prefill = bench_prefill(moe, synth, layers, args.prefill_tokens, bf16_peak, peak_kind, dev)

    # kernels of this library per layer step at decode sizes: front (one cluster: router, dispatch, plan, row
    # quantiser), fused FFN, combine on the tensor-core path; front, quantise, gate/up, down, combine on the GEMV path
    launches_per_layer = (3 if path != moe.PATH_GEMV else 5) if (stack is None) else stack.launches_per_layer
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "mxfp4 x e4m3 -> f32", "data": "synthetic",
        "config": workload_config(NL, T, world, se1 - se0, "CUDA graph of one step" if graph is not None else "stream launches"),
        "e2e": e2e, "gpu_launches": launches_per_layer * NL * args.steps, "clocks": clk.summary(),
        "roofline": roof, "peaks": peak_kind,
    }
    out.update(extra)
    if prefill:
        out["prefill"] = prefill
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_layer_rate(T, args.cpu_seconds)[1]
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def roofline_decode(moe, layers, dX, dL, T, path, hbm_peak, peak_kind, dev):
    """Times the expert-FFN launch(es) of every layer with CUDA events on the launching stream (cold weights:
    every layer is distinct) and sets the algorithmic bytes of a launch against its duration.  On the
    tensor-core path at decode sizes gate/up and down are ONE persistent launch (k_ffn_fused_small); on the
    GEMV path they are two and the gate/up launch (2/3 of the bytes) is the dominant kernel."""
    import torch
    NL = len(layers)
    use = moe.PATH_GEMV if path == moe.PATH_GEMV else moe.PATH_TC
    fused = use == moe.PATH_TC and T <= 16
    n, R = T * K8, T * (K8 + 1)
    soffs = torch.tensor([n, n + T], dtype=torch.int32, device=dev)
    touched, staged = [], []
    wsb = torch.empty(int(moe.lib.q36_moe_ffn_ws_bytes(E, R, D, FF)), dtype=torch.uint8, device=dev)
    bufs = (torch.zeros((R, FF), dtype=torch.uint8, device=dev), torch.zeros((R, FF // 32), dtype=torch.uint8, device=dev),
            torch.zeros((R, D), dtype=torch.float32, device=dev))
    for l in range(NL):                                   # stage every layer's sorted rows once (untimed)
        idx, wt = moe.router_topk(dL[l], E, K8)
        ec, eo, el, pos = moe.dispatch(idx.reshape(-1), E)
        Xq, Xs = moe.quant_scatter(dX[l], pos, K8, n, R)
        staged.append((eo, Xq, Xs))
        touched.append(int((ec > 0).sum().item()))

    def run_stage(stages):
        for l in range(NL):
            ly = layers[l]
            eo, Xq, Xs = staged[l]
            moe.expert_ffn_sorted(ly.Wg, ly.Wu, ly.Wd, E, eo, Xq, Xs, D, FF, use, stages=stages, bufs=bufs, ws=wsb,
                                  shared=(ly.Sg, ly.Su, ly.Sd), soffs=soffs, sync_check=False, max_group_rows=T)

    def time_stage(stages):
        """One CUDA graph with the launch of every layer back to back (no host gaps), replayed under events."""
        run_stage(stages)
        torch.cuda.synchronize()
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                run_stage(stages)
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * NL)

    if fused:
        # the call is [status memset, plan kernel, fused kernel]: the first two are timed alone and taken out
        t_all, t_setup = time_stage(3), time_stage(4)
        t_a, t_b = [t_all - t_setup], [0.0]
    else:
        t_a, t_b = [time_stage(1)], [time_stage(2)]
    if use == moe.PATH_TC:
        moe.check(moe.lib.q36_moe_ws_status(wsb.data_ptr(), moe.stream_ptr()), "device status")
    U = sum(touched) / len(touched)                       # distinct routed experts touched per layer
    x_bytes, h_bytes, y_bytes = R * (D + D // 32), R * (FF + FF // 32), R * D * 4
    gu_bytes = (U + 1) * (EXPERT_BYTES * 2 // 3) + x_bytes + h_bytes
    dn_bytes = (U + 1) * (EXPERT_BYTES // 3) + h_bytes + y_bytes
    a_ms, b_ms = sum(t_a) / len(t_a), sum(t_b) / len(t_b)
    extra = {"distinct_experts_per_layer": U}
    if fused:
        nbytes = gu_bytes + dn_bytes
        ach = nbytes / (a_ms * 1e-3) / 1e9
        # dram__bytes_read + dram__bytes_write of one launch of this kernel on this layer shape at T = 8, from the
        # ncu capture summarised in profiles/k_ffn_fused_small_decode_T8.md (scaled by the rows when T differs)
        traffic = 103.4e6 * (nbytes / 98.46e6)
        extra["setup_us_per_launch"] = t_setup * 1e3
        roof = {"bound": "hbm", "kernel": "k_ffn_fused_small (gate/up + SwiGLU + down in one launch)",
                "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak, "traffic": traffic,
                "bytes_per_launch": nbytes, "us_per_launch": a_ms * 1e3, "peak_kind": peak_kind,
                "frac_of_8TBps_nominal": ach / 8000.0}
        return roof, extra
    ach = gu_bytes / (a_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": "k_gateup_gemv" if use == moe.PATH_GEMV else "k_grouped_mma<2>",
            "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak, "traffic": None,
            "bytes_per_launch": gu_bytes, "us_per_launch": a_ms * 1e3, "peak_kind": peak_kind,
            "frac_of_8TBps_nominal": ach / 8000.0}
    ach_d = dn_bytes / (b_ms * 1e-3) / 1e9
    extra["roofline_down"] = {"bound": "hbm", "kernel": "k_down_gemv" if use == moe.PATH_GEMV else "k_grouped_mma<1>",
                              "achieved": ach_d, "peak": hbm_peak, "unit": "GB/s", "frac": ach_d / hbm_peak,
                              "bytes_per_launch": dn_bytes, "us_per_launch": b_ms * 1e3}
    return roof, extra


def bench_prefill(moe, synth, layers, Tp, bf16_peak, peak_kind, dev):
    """Benchmark configuration 2: one layer, Tp tokens, Zipf-skewed routing, tensor-core path.  Rotates over
    distinct layers so weights come from HBM."""
    import numpy as np
    import torch
    rng = np.random.default_rng(7)
    NLp = min(len(layers), 8)
    X = torch.from_numpy(synth.activations(rng, Tp)).to(dev).to(torch.bfloat16)
    L = torch.from_numpy(synth.router_logits(rng, Tp, zipf=True)).to(dev)
    out = torch.empty((Tp, D), dtype=torch.float32, device=dev)
    ws = layers[0].workspace(Tp)
    for l in range(NLp):
        layers[l].forward(X, L, out=out, path=moe.PATH_TC, ws=ws)
    torch.cuda.synchronize()
    layers[0].check_device_status()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    ev0.record()
    for _ in range(reps):
        for l in range(NLp):
            layers[l].forward(X, L, out=out, path=moe.PATH_TC, ws=ws)
    ev1.record()
    torch.cuda.synchronize()
    layers[0].check_device_status()
    ms = ev0.elapsed_time(ev1) / (reps * NLp)
    flop = Tp * (K8 + 1) * FLOP_PER_ASSIGNMENT
    tf = flop / (ms * 1e-3) / 1e12
    return {"workload": f"prefill: 1 layer, {Tp} tokens, Zipf-skewed routing, tcgen05 path", "ms_per_layer": ms,
            "tokens_per_s": Tp / (ms * 1e-3), "tflops": tf, "peak_mxf8f6f4_nominal_tflops": 4500.0,
            "frac_of_nominal": tf / 4500.0, "frac_of_2x_bf16": tf / (2 * bf16_peak), "peak_kind": peak_kind}


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
