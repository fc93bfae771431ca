#!/usr/bin/env python
"""MoE-layer throughput benchmark (the role of the reference's bench.c harness: warm-up, repetitions, mean and
spread, deterministic synthetic inputs; bench.c:64-88,283,306-335).

Workload (`config.workload`): decode through a stack of 40 DISTINCT MoE layers (256 routed + 1 shared MXFP4
experts each, D = 2048, FF = 512, top-8), so that every step streams fresh expert weights from HBM (about
40 x 98 MB at 8 tokens, far above the 126 MB L2).  Each rank feeds `--tokens` (default 8) tokens per step: one
rank is the benchmark's single-GPU decode configuration at T = 8; N ranks run the 40-layer expert-parallel decode
stack with 8 N tokens per step (64 at N = 8), experts split evenly over the ranks, dispatch and combine by the
library's own kernels over NVLink peer memory, the shared expert on each token's home rank.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  metric = token-layers per second (tokens x layers / time): the MoE-layer
tokens/s of the benchmark definition.  The K-step timing is repeated until about `--min-seconds` of device time
have been measured; `ms_per_step` is the median over the repetitions and `ms_per_step_std` their spread.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, FF, E, K8, LAYERS = 2048, 512, 256, 8, 40
EXPERT_BYTES = 3 * 512 * 2048 * 17 // 32          # 1,671,168 B: gate + up + down of one expert
FLOP_PER_ASSIGNMENT = 2 * 3 * 512 * 2048          # 6,291,456
ROW_BYTES_SENT = D + D // 32 + 16                 # a dispatched row: E4M3 codes, scale bytes, expert id
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
    ap.add_argument("--min-seconds", type=float, default=1.0, help="device time to measure per timing (repetitions of --steps)")
    ap.add_argument("--prefill-tokens", type=int, default=4096)
    ap.add_argument("--zipf", action="store_true", help="Zipf-skewed router logits for the decode stack too")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--prefill-only", action="store_true", help="only the prefill configuration (for profiling): prints {prefill: ...}")
    ap.add_argument("--prefill-graph-layers", type=int, default=8)
    ap.add_argument("--prefill-stack", action="store_true",
                    help="benchmark configuration 4 instead: the 40-layer prefill stack, --stack-tokens tokens in all, expert-parallel over "
                         "the ranks with the dispatch of layer l + 1 overlapped with the expert work of layer l")
    ap.add_argument("--stack-tokens", type=int, default=32768)
    ap.add_argument("--no-overlap", action="store_true", help="--prefill-stack: every phase on one stream")
    ap.add_argument("--table", action="store_true",
                    help="one GPU: a pp / tg / batch-width table over the layer stack, mean and std over -r repetitions (wall clock)")
    ap.add_argument("-p", dest="pp", default="512,2048,4096", help="--table: prefill sizes")
    ap.add_argument("-n", dest="tg", type=int, default=128, help="--table: decode steps per repetition")
    ap.add_argument("-r", dest="reps", type=int, default=3, help="--table: repetitions")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-config3", action="store_true", help="skip the fixed-batch line (64 tokens in all, split over the ranks)")
    ap.add_argument("--no-roofline", action="store_true")
    ap.add_argument("--path", default="auto", choices=["auto", "gemv", "tc"])
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"], help="expert-parallel exchange at N > 1")
    ap.add_argument("--cpu-seconds", type=float, default=8.0)
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


def measured_traffic(kernel: str):
    """DRAM bytes per launch of `kernel` from the committed ncu capture record (q36_b200/ncu_traffic.json:
    dram__bytes_read.sum + dram__bytes_write.sum of one launch, with the algorithmic bytes of that same launch)."""
    p = os.path.join(ROOT, "q36_b200", "ncu_traffic.json")
    try:
        return json.load(open(p)).get(kernel)
    except Exception:
        return None


def cpu_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def workload_config(NL, T, world):
    """The `config` object: the same in both arms' JSON lines."""
    return {"workload": f"decode stack: {NL} distinct MoE layers (256+1 MXFP4 experts, D=2048, FF=512, top-8), "
                        f"{T} tokens per rank per step ({world * T} global)",
            "tokens_per_rank": T, "layers": NL, "experts_per_rank": E // world,
            "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": f"inputs larger than L2: each step streams {NL} layers of distinct expert weights"}


# --------------------------------------------------------- CPU baseline arm
def cpu_layer_rate(tokens: int, limit_s: float, threads: int):
    """The reference's CPU implementation of the path -- its C dequantiser over the three matrices of an expert +
    a plain fp32 matmul (oracle/_ref when present, else the oracle port) -- on `threads` host cores.  A sample of
    (token, expert) evaluations of one T-token layer; returns (token-layers/s, description, seconds spent)."""
    import numpy as np
    from oracle import oracle as O
    from q36_b200 import synth
    rng = np.random.default_rng(0)
    w = synth.layer(seed=0, n_expert=4)
    X = synth.activations(rng, tokens)
    xq, xs = O.quant_e4m3(X)
    xd = O.dequant_e4m3(xq, xs)
    t0 = time.perf_counter()
    n_eval, spent, kind = 0, 0.0, "port"
    while spent < limit_s:
        e = n_eval % 4
        _, _, kind, _ = O.cpu_expert_seconds(w["gate"][e], w["up"][e], w["down"][e], D, FF, xd[n_eval % tokens], reps=3,
                                             threads=threads)
        n_eval += 3
        spent = time.perf_counter() - t0
    per_eval = spent / n_eval
    rate = 1.0 / (per_eval * (K8 + 1))          # one token through one layer = 9 expert evaluations
    return rate, {"value": rate, "unit": UNIT, "cores": threads, "kind": "reference" if kind == "reference" else "port",
                  "sample": f"{n_eval} (token, expert) evaluations of one {tokens}-token layer in {spent:.1f} s: the reference's C "
                            f"dequantiser over gate/up/down + fp32 matmul, {'OpenMP over rows' if threads > 1 else 'one thread'}"}, spent


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens * args.gpus
    cores = cpu_cores()
    per_step_limit = max(0.5, min(5.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_layer_rate(T, per_step_limit / 4, cores)
    vals, base, step_s = [], None, []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        r, base, spent = cpu_layer_rate(T, per_step_limit, cores)
        vals.append(r)
        step_s.append(spent)
    wall = time.perf_counter() - t0
    v = statistics.median(vals)
    base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * statistics.median(step_s), "value_std": statistics.pstdev(vals),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the same workload as the GPU arm's line; every step is a bounded sample of it (cpu_baseline.sample), timed as it is
        "config": workload_config(args.layers, args.tokens, args.gpus), "launch": "host cores, OpenMP",
        "step_is": "a bounded sample of the workload; value = its measured rate",
        "cpu_baseline": base, "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": wall}))


# ------------------------------------------------------------------ GPU arm
class Stack:
    """NL distinct layers (this rank's expert shard of each), their inputs on the host (pinned) and on the device,
    a device-resident step (one CUDA graph when it can be captured) and the host-buffer step."""

    def __init__(self, torch, dist, moe, synth, ep, layers, world, rank, dev, T, path, transport, zipf, seed=1234):
        import numpy as np
        self.torch, self.dist, self.moe, self.world, self.rank, self.dev, self.T, self.path = torch, dist, moe, world, rank, dev, T, path
        self.layers, self.NL = layers, len(layers)
        NL = self.NL
        rng = np.random.default_rng(seed + rank)
        self.hX = torch.stack([torch.from_numpy(synth.activations(rng, T)).to(torch.bfloat16) for _ in range(NL)]).pin_memory()
        self.hL = torch.stack([torch.from_numpy(synth.router_logits(rng, T, zipf=zipf)) for _ in range(NL)]).pin_memory()
        self.hO = torch.empty((NL, T, D), dtype=torch.float32).pin_memory()
        self.dX, self.dL = self.hX.to(dev), self.hL.to(dev)
        self.dO = torch.empty((NL, T, D), dtype=torch.float32, device=dev)
        self.ep = ep.NativeEP(layers, world, rank, T, transport=transport) if world > 1 else None
        self.ws = layers[0].workspace(T) if world == 1 else None
        self.host = moe.HostStack(layers, T, ep=self.ep)
        self.graph = None
        self.launch = "stream launches"

    def step_device(self):
        if self.ep is not None:
            for l in range(self.NL):
                self.ep.layer(self.layers[l], self.dX[l], self.dL[l], self.dO[l])
        else:
            for l in range(self.NL):
                self.layers[l].forward(self.dX[l], self.dL[l], out=self.dO[l], path=self.path, ws=self.ws)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def check(self):
        if self.ep is not None:
            self.ep.check_device_status()
        else:
            self.layers[0].check_device_status()

    def capture(self, allow: bool):
        """One CUDA graph per step.  The expert-parallel step is kernels only (peer-memory transport), so it is
        captured like the single-GPU one; the NCCL comparison transport is issued as stream launches."""
        torch = self.torch
        self.step_device()
        self.barrier()
        self.check()
        if not allow:
            return
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            self.step_device()
            s.synchronize()
            self.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self.step_device()
        self.barrier()
        self.graph, self.launch = g, "CUDA graph of one step"

    def run(self):
        (self.graph.replay if self.graph is not None else self.step_device)()

    def time_steps(self, fn, steps, warmup, min_seconds, clocks=None):
        """Repetitions of `steps` calls of fn, each bracketed by barrier + synchronise and timed with CUDA events on
        the launching stream; the max over ranks of every repetition.  Returns (ms per step per repetition, reps)."""
        torch = self.torch
        for _ in range(max(warmup, 3)):
            fn()
        self.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        fn()
        ev1.record()
        self.barrier()
        est = max(ev0.elapsed_time(ev1), 1e-3)
        reps = int(min(400, max(3, math.ceil(min_seconds * 1e3 / (est * steps)))))
        if self.world > 1:     # every rank must run the same number of repetitions
            t = torch.tensor([reps], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            reps = int(t.item())
        per = []
        for _ in range(reps):
            self.barrier()
            ev0.record()
            for _ in range(steps):
                fn()
            ev1.record()
            self.barrier()
            per.append(ev0.elapsed_time(ev1))
        t = torch.tensor(per, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [x / steps for x in t.tolist()], reps

    def close(self):
        if self.ep is not None:
            self.ep.close()


def summarise(per_step_ms, steps):
    med = statistics.median(per_step_ms)
    return {"ms_per_step": med, "ms_per_step_mean": statistics.fmean(per_step_ms),
            "ms_per_step_std": statistics.pstdev(per_step_ms) if len(per_step_ms) > 1 else 0.0,
            "ms_per_step_min": min(per_step_ms), "reps": len(per_step_ms), "timed_region_s": sum(per_step_ms) * steps * 1e-3}


def make_layers(torch, moe, world, rank, dev, NL):
    """NL distinct layers.  Every layer is generated over all 256 experts from its seed and the rank keeps its
    contiguous shard (q36_engine.cu:4245), so that the stack computes the same function at every N."""
    se0, se1 = rank * E // world, (rank + 1) * E // world
    layers, full0 = [], None
    s = moe.expert_stride(FF, D)
    for l in range(NL):
        full = moe.MoELayer(device=dev).random_planes(seed=1000 + l)
        if world == 1:
            layers.append(full)
            continue
        sh = moe.MoELayer(se0=se0, se1=se1, device=dev)
        sh.set_device_planes(full.Wg[se0 * s:se1 * s].clone(), full.Wu[se0 * s:se1 * s].clone(), full.Wd[se0 * s:se1 * s].clone(),
                             full.Sg, full.Su, full.Sd)
        layers.append(sh)
        if l == 0:
            full0 = full          # kept for the output check of the expert-parallel step
    return layers, full0


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
    transport = ep.TRANSPORT_PEER if args.transport == "peer" else ep.TRANSPORT_NCCL
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    if args.prefill_only:
        layers, _ = make_layers(torch, moe, 1, 0, dev, min(NL, args.prefill_graph_layers))
        print(json.dumps({"prefill": bench_prefill(torch, moe, synth, layers, args.prefill_tokens, bf16_peak, peak_kind, dev, args.min_seconds)}))
        return
    layers, full0 = make_layers(torch, moe, world, rank, dev, NL)
    st = Stack(torch, dist, moe, synth, ep, layers, world, rank, dev, T, path, transport, args.zipf)
    st.capture(allow=(world == 1 or transport == ep.TRANSPORT_PEER))
    # kernels of this library per layer step: front (one cluster: router, dispatch, plan, row quantiser), fused FFN,
    # combine on the tensor-core path at decode sizes; front, quantise, gate/up, down, combine on the GEMV path
    launches_per_layer = (3 if path != moe.PATH_GEMV else 5) if world == 1 else st.ep.launches_per_layer

    # ---- correctness gate of the expert-parallel step: layer 0 of every rank against the single-GPU layer over all
    # 256 experts (same seeds), and the device status words; outside every timed region
    ep_check = None
    if world > 1:
        st.run()
        st.barrier()
        ref = full0.forward(st.dX[0], st.dL[0], path=moe.PATH_TC)
        torch.cuda.synchronize()
        err = float((st.dO[0] - ref).norm() / ref.norm())
        t = torch.tensor([err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ep_check = {"max_rel_l2": float(t.item()), "tolerance": 1e-5, "status": 0, "layers_checked": 1}
        del full0
        torch.cuda.empty_cache()

    # ---- device-resident timing
    with ClockSampler(local) as clk:
        per, reps = st.time_steps(st.run, args.steps, args.warmup, args.min_seconds)
    res = summarise(per, args.steps)
    status = 0
    try:
        st.check()
    except moe.MoEError as e:
        status = moe.lib.q36_moe_last_cuda_error()
        sys.stderr.write(f"rank {rank}: {e}\n")
    if world > 1:
        t = torch.tensor([status], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        status = int(t.item())
        ep_check["status"] = status
        if rank == 0 and (status != 0 or not ep_check["max_rel_l2"] < ep_check["tolerance"]):
            print(json.dumps({"metric": METRIC, "error": "expert-parallel output check failed", "ep_check": ep_check}))
        if status != 0 or not ep_check["max_rel_l2"] < ep_check["tolerance"]:
            dist.destroy_process_group()
            sys.exit(3)
    elif status != 0:
        print(json.dumps({"metric": METRIC, "error": f"a device-side wait gave up (code {status})"}))
        sys.exit(3)
    value = world * T * NL / (res["ms_per_step"] * 1e-3)

    # ---- end to end through the host-buffer entry point: pinned host inputs in, results out, every step
    e2e_per, _ = st.time_steps(lambda: st.host.step(st.hX, st.hL, st.hO, path), args.steps, args.warmup, min(args.min_seconds, 0.5))
    e2e_res = summarise(e2e_per, args.steps)
    e2e = {"value": world * T * NL / (e2e_res["ms_per_step"] * 1e-3), "unit": UNIT,
           "h2d_bytes_per_step": NL * (T * D * 2 + T * (E + 1) * 4), "d2h_bytes_per_step": NL * T * D * 4,
           "ms_per_step": e2e_res["ms_per_step"], "ms_per_step_std": e2e_res["ms_per_step_std"], "reps": e2e_res["reps"],
           "entry": "q36_moe_ep_stack_host" if world > 1 else "q36_moe_stack_host"}
    np.testing.assert_allclose(st.hO[0].numpy(), st.dO[0].cpu().numpy(), rtol=0, atol=0)   # the host path computes the same bits

    # ---- roofline
    roof, extra = None, {}
    if not args.no_roofline:
        if world == 1:
            roof, extra = roofline_decode(moe, layers, st.dX, st.dL, T, path, hbm_peak, peak_kind, dev)
        else:
            roof, extra = roofline_ep(torch, dist, moe, st, world, rank, T, res["ms_per_step"], hbm_peak, peak_kind, dev)

    # ---- benchmark configuration 3: a fixed batch of 64 tokens per step over the whole job
    config3 = None
    if not args.no_config3 and 64 % world == 0:
        T3 = 64 // world
        if T3 == T:
            config3 = {"tokens_global": 64, "tokens_per_rank": T3, "value": value, "unit": UNIT, "ms_per_step": res["ms_per_step"],
                       "ms_per_step_std": res["ms_per_step_std"], "note": "same as the headline workload at this N"}
        else:
            st.close()
            st3 = Stack(torch, dist, moe, synth, ep, layers, world, rank, dev, T3, path, transport, args.zipf, seed=4321)
            st3.capture(allow=(world == 1 or transport == ep.TRANSPORT_PEER))
            per3, _ = st3.time_steps(st3.run, args.steps, args.warmup, min(args.min_seconds, 0.5))
            r3 = summarise(per3, args.steps)
            st3.check()
            config3 = {"tokens_global": 64, "tokens_per_rank": T3, "value": 64 * NL / (r3["ms_per_step"] * 1e-3), "unit": UNIT,
                       "ms_per_step": r3["ms_per_step"], "ms_per_step_std": r3["ms_per_step_std"], "reps": r3["reps"],
                       "scaling": "strong", "launch": st3.launch}
            st3.close()
            st = None

    # ---- prefill (benchmark configuration 2) on the tensor-core path
    prefill = None
    if world == 1 and not args.no_prefill:
        prefill = bench_prefill(torch, moe, synth, layers, args.prefill_tokens, bf16_peak, peak_kind, dev, args.min_seconds)

    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": res["ms_per_step"], "ms_per_step_std": res["ms_per_step_std"], "ms_per_step_mean": res["ms_per_step_mean"],
        "ms_per_step_min": res["ms_per_step_min"], "reps": res["reps"], "timed_region_s": res["timed_region_s"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4 x e4m3 -> f32", "data": "synthetic",
        "config": workload_config(NL, T, world), "launch": "CUDA graph of one step" if (world == 1 or transport == ep.TRANSPORT_PEER) else "stream launches",
        "e2e": e2e, "gpu_launches": launches_per_layer * NL * args.steps * res["reps"], "clocks": clk.summary(),
        "roofline": roof, "peaks": peak_kind,
    }
    if world > 1:
        out["transport"] = args.transport
        out["ep_check"] = ep_check
    out.update(extra)
    if config3:
        out["config3"] = config3
    if prefill:
        out["prefill"] = prefill
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cores = cpu_cores()
        _, single, _ = cpu_layer_rate(T, args.cpu_seconds / 2, 1)
        _, allc, _ = cpu_layer_rate(T, args.cpu_seconds / 2, cores)
        allc["single_thread"] = {"value": single["value"], "unit": UNIT, "cores": 1, "sample": single["sample"]}
        out["cpu_baseline"] = allc
    if rank == 0:
        print(json.dumps(out))
    if st is not None:
        st.close()
    if world > 1:
        dist.destroy_process_group()


def roofline_ep(torch, dist, moe, st, world, rank, T, ms_per_step, hbm_peak, peak_kind, dev):
    """Per-rank roofline of the expert-parallel step: the bytes a rank must stream per layer (its touched resident
    experts + the shared expert + the rows it receives, computes and returns) against the whole layer step's time
    (the FFN launch is not timed alone here: waits on the peers sit inside the same step)."""
    NL = st.NL
    per = E // world
    touched, rows = 0.0, 0.0
    for l in range(NL):
        idx, _ = moe.router_topk(st.dL[l], E, K8)                       # this rank's tokens
        allidx = [torch.empty_like(idx) for _ in range(world)]
        dist.all_gather(allidx, idx)
        flat = torch.cat(allidx).reshape(-1)
        mine = flat[(flat >= rank * per) & (flat < (rank + 1) * per)]
        touched += float(torch.unique(mine).numel())
        rows += float(mine.numel())
    U, R = touched / NL, rows / NL
    nbytes = (U + 1) * EXPERT_BYTES + (R + T) * (D + D // 32 + 2 * (FF + FF // 32) + D * 4)
    t = torch.tensor([nbytes], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    nbytes = float(t.item())                                             # the busiest rank bounds the step
    us = ms_per_step * 1e3 / NL
    ach = nbytes / (us * 1e-6) / 1e9
    roof = {"bound": "hbm", "kernel": "whole expert-parallel layer step on the busiest rank (front, send, plan, unpack, k_ffn_fused_small, return, combine)",
            "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak, "traffic": None, "bytes_per_launch": nbytes,
            "us_per_launch": us, "peak_kind": peak_kind, "frac_of_8TBps_nominal": ach / 8000.0}
    real = R * ROW_BYTES_SENT + R * D * 4
    extra = {"distinct_experts_per_layer_per_rank": U, "rows_received_per_layer_per_rank": R,
             "all_to_all_bytes_per_layer_per_rank": {"dispatch_in": R * ROW_BYTES_SENT, "results_out": R * D * 4, "sent": real, "real": real,
                                                     "note": "only filled slots travel; capacity is address space, not traffic"}}
    return roof, extra


def roofline_decode(moe, layers, dX, dL, T, path, hbm_peak, peak_kind, dev):
    """Times the expert-FFN launch(es) of every layer with CUDA events on the launching stream (cold weights:
    every layer is distinct) and sets the algorithmic bytes of a launch against its duration.  On the
    tensor-core path at decode sizes gate/up and down are ONE persistent launch (k_ffn_fused_small); on the
    GEMV path they are two and the gate/up launch (2/3 of the bytes) is the dominant kernel."""
    import torch
    NL = len(layers)
    use = moe.PATH_GEMV if path == moe.PATH_GEMV else moe.PATH_TC
    fused = use == moe.PATH_TC and bool(moe.lib.q36_moe_one_launch_fits(T * (K8 + 1), E, D, FF)) and T * (K8 + 1) <= moe.lib.q36_moe_one_launch_rows()
    n, R = T * K8, T * (K8 + 1)
    soffs = torch.tensor([n, n + T], dtype=torch.int32, device=dev)
    touched, staged = [], []
    wsb = torch.zeros(int(moe.lib.q36_moe_ffn_ws_bytes(E, R, D, FF)), dtype=torch.uint8, device=dev)
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
        vals = []
        for _ in range(7):
            e0.record()
            for _ in range(5):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            vals.append(e0.elapsed_time(e1) / (5 * NL))
        return statistics.median(vals)

    if fused:
        # the call is [plan kernel, fused kernel]: the plan is timed alone and taken out
        t_all, t_setup = time_stage(3), time_stage(4)
        a_ms, b_ms = t_all - t_setup, 0.0
    else:
        a_ms, b_ms = time_stage(1), time_stage(2)
    if use == moe.PATH_TC:
        moe.check(moe.lib.q36_moe_ws_status(wsb.data_ptr(), moe.stream_ptr()), "device status")
    U = sum(touched) / len(touched)                       # distinct routed experts touched per layer
    x_bytes, h_bytes, y_bytes = R * (D + D // 32), R * (FF + FF // 32), R * D * 4
    gu_bytes = (U + 1) * (EXPERT_BYTES * 2 // 3) + x_bytes + h_bytes
    dn_bytes = (U + 1) * (EXPERT_BYTES // 3) + h_bytes + y_bytes
    extra = {"distinct_experts_per_layer": U}
    if fused:
        nbytes = gu_bytes + dn_bytes
        ach = nbytes / (a_ms * 1e-3) / 1e9
        rec = measured_traffic("k_ffn_fused_small")
        traffic = rec["dram_bytes_per_launch"] * (nbytes / rec["algorithmic_bytes_per_launch"]) if rec else None
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


def bench_prefill(torch, moe, synth, layers, Tp, bf16_peak, peak_kind, dev, min_seconds):
    """Benchmark configuration 2: one layer, Tp tokens, Zipf-skewed routing, tensor-core path.  A CUDA graph of
    eight distinct layers (weights from HBM), replayed until about min_seconds / 2 of device time."""
    import numpy as np
    rng = np.random.default_rng(7)
    NLp = min(len(layers), 8)
    X = torch.from_numpy(synth.activations(rng, Tp)).to(dev).to(torch.bfloat16)
    L = torch.from_numpy(synth.router_logits(rng, Tp, zipf=True)).to(dev)
    out = torch.empty((Tp, D), dtype=torch.float32, device=dev)
    ws = layers[0].workspace(Tp)

    def step():
        for l in range(NLp):
            layers[l].forward(X, L, out=out, path=moe.PATH_TC, ws=ws)

    step()
    torch.cuda.synchronize()
    layers[0].check_device_status()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        step()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            step()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(); g.replay(); ev1.record()
    torch.cuda.synchronize()
    reps = int(min(200, max(5, math.ceil(0.5 * min_seconds * 1e3 / max(ev0.elapsed_time(ev1), 1e-3)))))
    vals = []
    for _ in range(reps):
        ev0.record()
        g.replay()
        ev1.record()
        torch.cuda.synchronize()
        vals.append(ev0.elapsed_time(ev1) / NLp)
    layers[0].check_device_status()
    ms = statistics.median(vals)
    flop = Tp * (K8 + 1) * FLOP_PER_ASSIGNMENT
    tf = flop / (ms * 1e-3) / 1e12
    return {"workload": f"prefill: 1 layer, {Tp} tokens, Zipf-skewed routing, tcgen05 path", "ms_per_layer": ms,
            "ms_per_layer_std": statistics.pstdev(vals), "reps": reps, "launch": f"CUDA graph of {NLp} distinct layers",
            "tokens_per_s": Tp / (ms * 1e-3), "tflops": tf, "peak_mxf8f6f4_nominal_tflops": 4500.0,
            "frac_of_nominal": tf / 4500.0, "frac_of_2x_bf16": tf / (2 * bf16_peak), "peak_kind": peak_kind}


def run_prefill_stack(args):
    """Benchmark configuration 4: NL layers x stack-tokens tokens (uniform N(0,1) router logits, top-8), expert-parallel
    over the ranks; two streams: phase 0 (route, quantise, store rows into the peers' windows) of layer l + 1 runs beside
    phases 1 and 2 (expert FFN, results back, combine) of layer l.  One rank: the same layers on one GPU."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from q36_b200 import build as qb
    qb.build()
    from q36_b200 import moe, synth, ep
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    NL, T = args.layers, args.stack_tokens // world
    _, bf16_peak, peak_kind = measured_peaks()
    layers, full0 = make_layers(torch, moe, world, rank, dev, NL)
    NIN = 4                                                    # distinct input sets, cycled over the layers
    rng = np.random.default_rng(99 + rank)
    X = [torch.from_numpy(synth.activations(rng, T)).to(dev).to(torch.bfloat16) for _ in range(NIN)]
    L = [torch.from_numpy(synth.router_logits(rng, T)).to(dev) for _ in range(NIN)]
    out = [torch.empty((T, D), dtype=torch.float32, device=dev) for _ in range(2)]
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    ep_check = None
    if world == 1:
        ws = layers[0].workspace(T)

        def one_pass():
            for l in range(NL):
                layers[l].forward(X[l % NIN], L[l % NIN], out=out[l & 1], path=moe.PATH_TC, ws=ws)
        launch = "stream launches, one stream"
    else:
        cap = min(T * K8, int(1.5 * T * K8 / world) + 256)      # rows per pair of ranks: 1.5 x the mean of uniform routing
        nat = ep.NativeEP(layers, world, rank, T, cap_rows=cap)
        wss = [nat.ws, nat.second_workspace()]
        e0 = [torch.cuda.Event() for _ in range(NL)]
        e2 = [torch.cuda.Event() for _ in range(NL)]

        def one_pass():
            if args.no_overlap:
                for l in range(NL):
                    for p in range(3):
                        nat.phase(p, layers[l], X[l % NIN], L[l % NIN], out[l & 1], ws=wss[l & 1])
                return
            cur = torch.cuda.current_stream()
            s1.wait_stream(cur)
            s2.wait_stream(cur)
            with torch.cuda.stream(s2):
                nat.phase(0, layers[0], X[0], L[0], out[0], ws=wss[0])
                e0[0].record(s2)
            for l in range(NL):
                if l + 1 < NL:
                    with torch.cuda.stream(s2):
                        if l >= 1:
                            s2.wait_event(e2[l - 1])       # its windows' and workspace's previous user (layer l - 1) is done
                        nat.phase(0, layers[l + 1], X[(l + 1) % NIN], L[(l + 1) % NIN], out[(l + 1) & 1], ws=wss[(l + 1) & 1])
                        e0[l + 1].record(s2)
                with torch.cuda.stream(s1):
                    s1.wait_event(e0[l])
                    nat.phase(1, layers[l], X[l % NIN], L[l % NIN], out[l & 1], ws=wss[l & 1])
                    nat.phase(2, layers[l], X[l % NIN], L[l % NIN], out[l & 1], ws=wss[l & 1])
                    e2[l].record(s1)
            cur.wait_stream(s1)
            cur.wait_stream(s2)
        launch = "stream launches, one stream" if args.no_overlap else "stream launches, two streams (dispatch of layer l + 1 beside the expert work of layer l)"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    one_pass()
    barrier()
    if world > 1:
        # layer NL - 1's output of this rank (out[(NL - 1) & 1]) against the single-GPU layer over all experts
        lchk = NL - 1
        fullL = moe.MoELayer(device=dev).random_planes(seed=1000 + lchk)
        ref = fullL.forward(X[lchk % NIN], L[lchk % NIN], path=moe.PATH_TC)
        torch.cuda.synchronize()
        err = float((out[lchk & 1] - ref).norm() / ref.norm())
        t = torch.tensor([err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        st_rc = 0
        for w in wss:
            st_rc = st_rc or moe.lib.q36_moe_ws_status(w.data_ptr(), moe.stream_ptr())
        ts = torch.tensor([abs(st_rc)], device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        ep_check = {"max_rel_l2": float(t.item()), "tolerance": 1e-4, "status": int(ts.item()), "layer_checked": lchk}
        del fullL, ref
        torch.cuda.empty_cache()
    else:
        layers[0].check_device_status()
    for _ in range(max(1, args.warmup - 1)):
        one_pass()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per = []
    for _ in range(max(3, args.steps)):
        barrier()
        ev0.record()
        one_pass()
        ev1.record()
        barrier()
        per.append(ev0.elapsed_time(ev1))
    t = torch.tensor(per, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    per = t.tolist()
    ms = statistics.median(per)
    tokens = T * world
    flop = tokens * (K8 + 1) * FLOP_PER_ASSIGNMENT * NL
    line = {"metric": "moe_prefill_stack_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s (through all layers)",
            "token_layers_per_s": tokens * NL / (ms * 1e-3), "n_gpus": world, "steps": len(per), "ms_per_pass": ms,
            "ms_per_pass_std": statistics.pstdev(per), "ms_per_layer": ms / NL, "tflops_per_gpu": flop / (ms * 1e-3) / 1e12 / world,
            "frac_of_nominal_mxf8f6f4_per_gpu": flop / (ms * 1e-3) / 1e12 / world / 4500.0, "scaling": "strong", "data": "synthetic",
            "config": {"workload": f"prefill stack: {NL} distinct MoE layers, {tokens} tokens in all ({T} per rank), uniform routing, top-8",
                       "layers": NL, "tokens": tokens, "parallelism": f"ep{world}" if world > 1 else "single"},
            "launch": launch, "ep_check": ep_check, "peaks": peak_kind}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        ok = ep_check["status"] == 0 and ep_check["max_rel_l2"] < ep_check["tolerance"]
        nat.close()
        dist.destroy_process_group()
        if not ok:
            sys.exit(3)


def run_table(args):
    """The caller loop around the layer stack, reported the way the engine's own harness reports a model
    (bench.c:306-335: `pp<N>` = N prompt tokens through the stack once, `tg<N>` = N single-token steps, each mean
    and sample standard deviation of tokens/s over -r repetitions timed by the wall clock around a synchronised
    region; bench.c:283-305: a step at batch width B against B = 1).  Every size runs as one CUDA graph of the whole
    stack with the path q36_moe_layer picks for it."""
    import torch
    from q36_b200 import ep, moe, synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    NL = args.layers
    layers, _ = make_layers(torch, moe, 1, 0, dev, NL)
    path = {"auto": moe.PATH_AUTO, "gemv": moe.PATH_GEMV, "tc": moe.PATH_TC}[args.path]

    def stack_for(T):
        st = Stack(torch, None, moe, synth, ep, layers, 1, 0, dev, T, path, ep.TRANSPORT_PEER, False)
        st.capture(True)
        for _ in range(3):
            st.run()
        torch.cuda.synchronize()
        return st

    def rates(st, calls, tokens):
        out = []
        for _ in range(max(1, args.reps)):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(calls):
                st.run()
            torch.cuda.synchronize()
            out.append(tokens / (time.perf_counter() - t0))
        st.check()
        return statistics.fmean(out), (statistics.stdev(out) if len(out) > 1 else 0.0)

    name = f"moe-stack-{NL}x({E}+1)xMXFP4"
    print("| model | test | t/s |\n|---|---|---:|")
    for T in [int(x) for x in args.pp.split(",") if x]:
        st = stack_for(T)
        m, sd = rates(st, 1, T)
        print(f"| {name} | pp{T} | {m:.1f} \u00b1 {sd:.1f} |", flush=True)
        st.close()
        del st
    st = stack_for(1)
    m, sd = rates(st, args.tg, args.tg)
    print(f"| {name} | tg{args.tg} | {m:.1f} \u00b1 {sd:.1f} |", flush=True)
    print("\n| batch B | step ms | vs B=1 |\n|---|---:|---:|")
    t1 = None
    for B in (1, 2, 4, 8, 16, 32):
        if B > 1:
            st.close()
            st = stack_for(B)
        m, _ = rates(st, 20, 20)          # steps per second
        ms = 1e3 / m
        t1 = ms if t1 is None else t1
        print(f"| {B} | {ms:.3f} | {t1 * B / ms:.2f}x |", flush=True)
    st.close()


def main():
    args = parse()
    if args.table:
        run_table(args)
        return
    if args.prefill_stack:
        run_prefill_stack(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
