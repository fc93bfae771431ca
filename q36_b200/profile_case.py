"""One MoE layer forward over three distinct layers (so weights are cold in L2), twice: the small case the
ncu captures under profiles/ were taken on.

  python -m q36_b200.profile_case T [gemv|tc] [zipf]
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np, torch
from q36_b200 import moe, synth
T = int(sys.argv[1]) if len(sys.argv) > 1 else 8
path = {"gemv": moe.PATH_GEMV, "tc": moe.PATH_TC}[sys.argv[2] if len(sys.argv) > 2 else "gemv"]
zipf = len(sys.argv) > 3 and sys.argv[3] == "zipf"
layers = [moe.MoELayer().random_planes(seed=l) for l in range(3)]
rng = np.random.default_rng(0)
X = torch.from_numpy(synth.activations(rng, T)).cuda().to(torch.bfloat16)
L = torch.from_numpy(synth.router_logits(rng, T, zipf=zipf)).cuda()
for rep in range(2):
    for ly in layers:
        out = ly.forward(X, L, path=path)
torch.cuda.synchronize()
if path == moe.PATH_TC: layers[-1].check_device_status()
print("ok", float(out.abs().mean()))
