"""Time per layer of the GEMV path and the tensor-core path for a list of token counts, each as one CUDA
graph over 20 distinct layers (cold weights), CUDA events around the replays.

  python -m q36_b200.path_timing 1,2,4,8,16,64,256,4096
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np, torch
from q36_b200 import moe, synth
NL = 20
layers = [moe.MoELayer().random_planes(seed=l) for l in range(NL)]
rng = np.random.default_rng(0)
Ts = [int(a) for a in sys.argv[1].split(',')] if len(sys.argv) > 1 else [1, 2, 4, 8, 16, 64]
for T in Ts:
    X = torch.from_numpy(synth.activations(rng, T)).cuda().to(torch.bfloat16)
    L = torch.from_numpy(synth.router_logits(rng, T)).cuda()
    ws = layers[0].workspace(max(Ts))
    out = torch.empty((T, 2048), device='cuda')
    res = {}
    for name, path in (("gemv", moe.PATH_GEMV), ("tc", moe.PATH_TC)):
        if name == "gemv" and T > 64: continue
        def step():
            for ly in layers: ly.forward(X, L, out=out, path=path, ws=ws)
        step(); torch.cuda.synchronize()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            step(); s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s): step()
        torch.cuda.synchronize()
        for _ in range(3): g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5): g.replay()
        e1.record(); torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / 5 / NL * 1e3
    print(f"T={T}: us/layer " + " ".join(f"{k}={v:.1f}" for k, v in res.items()), flush=True)
layers[0].check_device_status()
