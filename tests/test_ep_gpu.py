"""Expert-parallel layer on 2 GPUs (NCCL all-to-all over NVLink) against the single-GPU layer.
Needs at least two CUDA devices; skipped otherwise."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

T = 8


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from q36_b200 import ep, moe, synth
    E, K = synth.N_EXPERT, synth.N_USED
    per = E // world
    shard = moe.MoELayer(se0=rank * per, se1=(rank + 1) * per, device=f"cuda:{rank}")
    full = moe.MoELayer(device=f"cuda:{rank}").random_planes(seed=11)
    s = moe.expert_stride(synth.EXPERT_FF, synth.D_MODEL)
    # the shard's planes are a slice of the full layer's (same bytes on every rank: same seed)
    shard.set_device_planes(full.Wg[rank * per * s:(rank + 1) * per * s], full.Wu[rank * per * s:(rank + 1) * per * s],
                            full.Wd[rank * per * s:(rank + 1) * per * s], full.Sg, full.Su, full.Sd)
    rng = np.random.default_rng(500 + rank)
    X = torch.from_numpy(synth.activations(rng, T)).cuda().to(torch.bfloat16)
    L = torch.from_numpy(synth.router_logits(rng, T)).cuda()
    worst = 0.0
    for path in (moe.PATH_GEMV, moe.PATH_TC):
        out = ep.ep_layer(ep.DeviceOps(moe), shard, X, L, world, rank, E, K, path)
        ref = full.forward(X, L, path=path)
        torch.cuda.synchronize()
        full.check_device_status()
        err = float((out - ref).norm() / ref.norm())
        worst = max(worst, err)
    # the native entry point (q36_moe_ep_layer): kernels and NCCL send/recv issued from C
    nat = ep.NativeEP([shard], world, rank, T)
    for _ in range(3):
        out = nat.layer(shard, X, L, torch.empty((T, synth.D_MODEL), dtype=torch.float32, device=X.device))
    torch.cuda.synchronize()
    nat.check_device_status()
    ref = full.forward(X, L, path=moe.PATH_TC)
    worst = max(worst, float((out - ref).norm() / ref.norm()))
    nat.close()
    q.put((rank, worst))
    dist.barrier()
    dist.destroy_process_group()


def test_ep_layer_two_gpus():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err in res:
        # same quantised rows, same kernels; only the summation grouping differs from the single-GPU layer
        assert err < 1e-5, f"rank {rank}: rel-L2 vs single-GPU layer {err}"
