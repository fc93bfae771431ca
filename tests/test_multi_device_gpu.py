"""One host thread driving two devices in turn, the way the engine's multi-GPU driver does
(q36_multi_create / q36_multi_prefill loop over devices with cudaSetDevice, q36_engine.cu:4234-4306).
The library's per-device state (multiprocessor count, the kernels' shared-memory opt-in, the built-in scratch
address) must be right on the second device too.  Needs two CUDA devices; skipped otherwise."""
import numpy as np
import pytest

from q36_b200 import synth

pytestmark = pytest.mark.gpu


def test_layer_on_device_1_after_device_0(moe):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    E, K = synth.N_EXPERT, synth.N_USED
    rng = np.random.default_rng(31)
    outs = {}
    for T in (8, 300):                      # the one-launch decode kernel, then the two grouped-GEMM launches
        X = synth.activations(rng, T)
        L = synth.router_logits(rng, T)
        for dev in (0, 1):
            torch.cuda.set_device(dev)
            layer = moe.MoELayer(device=f"cuda:{dev}").random_planes(seed=77)
            xt = torch.from_numpy(X).to(f"cuda:{dev}").to(torch.bfloat16)
            lt = torch.from_numpy(L).to(f"cuda:{dev}")
            out = layer.forward(xt, lt, path=moe.PATH_TC)
            torch.cuda.synchronize(dev)
            layer.check_device_status()
            outs[(T, dev)] = out.cpu().numpy()
            # the built-in scratch of the no-allocation dispatch resolves its address per device as well
            eid = torch.from_numpy(rng.integers(0, E, size=4096).astype(np.int32)).to(f"cuda:{dev}")
            want = moe.dispatch(eid, E)
            ecount = torch.empty(E, dtype=torch.int32, device=eid.device)
            eoffs = torch.empty(E + 1, dtype=torch.int32, device=eid.device)
            elist = torch.empty(4096, dtype=torch.int32, device=eid.device)
            pos = torch.empty(4096, dtype=torch.int32, device=eid.device)
            moe.check(moe.lib.q36_moe_dispatch_noalloc(eid.data_ptr(), 4096, E, 0, E, ecount.data_ptr(), eoffs.data_ptr(),
                                                       elist.data_ptr(), pos.data_ptr(), moe.stream_ptr()), "noalloc")
            torch.cuda.synchronize(dev)
            assert torch.equal(elist, want[2]) and torch.equal(pos, want[3])
        np.testing.assert_array_equal(outs[(T, 0)], outs[(T, 1)])     # same seed, same inputs, same kernels
    torch.cuda.set_device(0)
