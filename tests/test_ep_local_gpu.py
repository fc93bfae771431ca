"""The expert-parallel data path at 2, 4 and 8 ranks on ONE GPU: the ranks of one process take turns on the
device (q36_moe_ep_init_local), every phase of a call issued for all ranks before the next phase, so the kernels
that store into the peers' windows, the bounded waits, the slot arithmetic, the local plan and both FFN branches
all run exactly as they do across GPUs.  Each rank's output must match the single-GPU layer over all experts."""
import numpy as np
import pytest

from q36_b200 import synth

pytestmark = pytest.mark.gpu

E, K8, D, FF = synth.N_EXPERT, synth.N_USED, synth.D_MODEL, synth.EXPERT_FF


@pytest.fixture(scope="module")
def full(moe):
    return moe.MoELayer().random_planes(seed=11)


def _shards(moe, full, world):
    per = E // world
    s = moe.expert_stride(FF, D)
    out = []
    for r in range(world):
        sh = moe.MoELayer(se0=r * per, se1=(r + 1) * per)
        sh.set_device_planes(full.Wg[r * per * s:(r + 1) * per * s], full.Wu[r * per * s:(r + 1) * per * s],
                             full.Wd[r * per * s:(r + 1) * per * s], full.Sg, full.Su, full.Sd)
        out.append(sh)
    return out


def _inputs(world, T, seed, same_logits=False):
    import torch
    Xs, Ls = [], []
    row = None
    for r in range(world):
        rng = np.random.default_rng(seed + r)
        Xs.append(torch.from_numpy(synth.activations(rng, T)).cuda().to(torch.bfloat16))
        L = synth.router_logits(rng, T)
        if same_logits:                       # every token of every rank picks the SAME experts: groups of world * T rows
            row = L[0].copy() if row is None else row
            L = np.tile(row, (T, 1)).astype(np.float32)
            L[:, E] = rng.standard_normal(T)  # (the shared-gate logit stays per token)
        Ls.append(torch.from_numpy(L).cuda())
    return Xs, Ls


@pytest.mark.parametrize("world,T,same", [(2, 8, False), (4, 8, False), (8, 8, False),   # decode: the scaling bench's shapes
                                          (8, 8, True),      # 8 experts receive 64 rows each: 16-row token tiles of one group
                                          (2, 64, False),    # 1024 received slots: the one-block plan at its limit
                                          (2, 160, False),   # 2560 slots: the general dispatch kernels + one-launch FFN
                                          (2, 448, False)])  # 7168 slots: the two grouped-GEMM launches
def test_local_ranks_match_the_single_gpu_layer(moe, full, world, T, same):
    import torch
    from q36_b200 import ep
    shards = _shards(moe, full, world)
    loc = ep.LocalEP(world, [0] * world, T, E, K8, D, FF)
    try:
        for call in range(3):                 # three calls: both parities of the window, and the device call counter
            Xs, Ls = _inputs(world, T, 500 + 10 * call, same)
            outs = [torch.full((T, D), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
            loc.layer(shards, Xs, Ls, outs)
            torch.cuda.synchronize()
            for r in range(world):
                assert loc.status(r) == moe.OK, f"rank {r}: device status {moe.lib.q36_moe_last_cuda_error()}"
                ref = full.forward(Xs[r], Ls[r], path=moe.PATH_TC)
                torch.cuda.synchronize()
                full.check_device_status()
                err = float((outs[r] - ref).norm() / ref.norm())
                # same quantised rows, same kernels: only the grouping of the f32 sums differs.  At 448 tokens the
                # single-GPU layer still takes the one-launch kernel while a rank's 7168 rows take the two grouped-GEMM
                # launches: their f32 sums differ in order, so a code of the quantised intermediate may land on the
                # other side of a rounding boundary now and then
                lim = moe.lib.q36_moe_one_launch_rows()
                other = (world * T * K8 + T > lim) != (T * (K8 + 1) > lim)
                tol = 2e-3 if other else 1e-5
                assert err < tol, f"call {call} rank {r}: rel-L2 vs single-GPU layer {err}"
    finally:
        loc.close()


def test_prefill_sized_calls_return_one_partial_row_per_token_and_rank(moe, full):
    """Two-launch calls over the peer transport: the expert ranks sum a token's rows with the combine weights and
    return one row per (token, rank).  Window capacity 1.5 x the mean, as the prefill stack uses; the second call
    has fewer tokens than the window was opened for."""
    import torch
    from q36_b200 import ep
    world, T_max = 4, 1024
    shards = _shards(moe, full, world)
    loc = ep.LocalEP(world, [0] * world, T_max, E, K8, D, FF, cap_rows=T_max * K8 * 3 // (2 * world))
    try:
        for call, T in enumerate((T_max, 900, T_max)):
            Xs, Ls = _inputs(world, T, 700 + 10 * call)
            outs = [torch.full((T, D), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
            loc.layer(shards, Xs, Ls, outs)
            torch.cuda.synchronize()
            for r in range(world):
                assert loc.status(r) == moe.OK, f"rank {r}: device status {moe.lib.q36_moe_last_cuda_error()}"
                ref = full.forward(Xs[r], Ls[r], path=moe.PATH_TC)
                torch.cuda.synchronize()
                err = float((outs[r] - ref).norm() / ref.norm())
                assert err < 1e-5, f"call {call} rank {r}: rel-L2 vs single-GPU layer {err}"
    finally:
        loc.close()


def test_phase_0_of_the_next_call_may_run_ahead(moe, full):
    """Overlap: phase 0 (route + send) of call n + 1 is issued BEFORE phases 1 and 2 of call n, as a caller does to
    hide the dispatch behind the previous call's expert work.  Each phase keeps its own call counter on the device
    and the calls alternate between two private workspaces; the results must not change."""
    import torch
    from q36_b200 import ep
    world, T, calls = 4, 8, 5
    shards = _shards(moe, full, world)
    loc = ep.LocalEP(world, [0] * world, T, E, K8, D, FF)
    ws2 = [torch.zeros_like(w) for w in loc.ws]
    try:
        ins = [_inputs(world, T, 1200 + 10 * c) for c in range(calls)]
        outs = [[torch.full((T, D), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)] for _ in range(calls)]
        wsel = lambda c, r: None if c % 2 == 0 else ws2[r]

        def phase(p, c):
            for r in range(world):
                moe.check(loc.phase(p, r, shards[r], ins[c][0][r], ins[c][1][r], outs[c][r], ws=wsel(c, r)), f"call {c} rank {r} phase {p}")

        phase(0, 0)
        for c in range(calls):
            if c + 1 < calls:
                phase(0, c + 1)           # ahead of this call's expert work and combine
            phase(1, c)
            phase(2, c)
        torch.cuda.synchronize()
        for c in range(calls):
            for r in range(world):
                ref = full.forward(ins[c][0][r], ins[c][1][r], path=moe.PATH_TC)
                torch.cuda.synchronize()
                err = float((outs[c][r] - ref).norm() / ref.norm())
                assert err < 1e-5, f"call {c} rank {r}: rel-L2 {err}"
        for r in range(world):
            assert loc.status(r) == moe.OK
            assert moe.lib.q36_moe_ws_status(ws2[r].data_ptr(), moe.stream_ptr()) == moe.OK
    finally:
        loc.close()


def test_a_smaller_capacity_drops_rows_and_says_so(moe, full):
    """cap_rows below the worst case: rows beyond it are dropped (their term is missing from the sum), the status
    words say 0xD00, nothing hangs or overruns."""
    import torch
    from q36_b200 import ep
    world, T = 2, 8
    shards = _shards(moe, full, world)
    loc = ep.LocalEP(world, [0] * world, T, E, K8, D, FF, cap_rows=8)      # 64 rows per rank, ~32 per destination
    try:
        Xs, Ls = _inputs(world, T, 900)
        outs = [torch.zeros((T, D), dtype=torch.float32, device="cuda") for _ in range(world)]
        loc.layer(shards, Xs, Ls, outs)
        torch.cuda.synchronize()
        assert loc.status(0) == moe.EDEVICE
        assert moe.lib.q36_moe_last_cuda_error() == 200000 + 0xD00
        assert all(bool(torch.isfinite(o).all()) for o in outs)
    finally:
        loc.close()


def test_a_wait_that_nothing_satisfies_ends_with_a_status(moe, full):
    """Phase 1 without the peers' phase 0: the headers of this call never arrive, the bounded wait gives up, the
    kernels return and the host reads Q36_MOE_EDEVICE with the waiting source in the code.  The context stays usable."""
    import torch
    from q36_b200 import ep
    world, T = 2, 4
    shards = _shards(moe, full, world)
    loc = ep.LocalEP(world, [0] * world, T, E, K8, D, FF)
    try:
        Xs, Ls = _inputs(world, T, 950)
        outs = [torch.zeros((T, D), dtype=torch.float32, device="cuda") for _ in range(world)]
        assert loc.phase(0, 0, shards[0], Xs[0], Ls[0], outs[0]) == moe.OK    # rank 0 sends; rank 1 never does
        assert loc.phase(1, 0, shards[0], Xs[0], Ls[0], outs[0]) == moe.OK    # rank 0 waits for rank 1's header
        torch.cuda.synchronize()
        assert loc.status(0) == moe.EDEVICE
        assert moe.lib.q36_moe_last_cuda_error() == 200000 + 0xB00 + 1       # dispatch wait, source rank 1
        ref = full.forward(Xs[0], Ls[0], path=moe.PATH_TC)                    # the device still works
        torch.cuda.synchronize()
        assert bool(torch.isfinite(ref).all())
    finally:
        loc.close()
