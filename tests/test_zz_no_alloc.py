"""q36_moe_dispatch_noalloc: the dispatch for callers that cannot hand over scratch memory.

Some callers of this library have nowhere to get device memory from at the point of the call: a launcher
dropped into the engine's per-step path runs after every buffer was allocated once at engine creation, and a
host that drives the library through a fixed plugin signature passes only its inputs and outputs.  For them the
library carries a small scratch array of its own.  This test calls that entry point through the C ABI and
checks that it returns exactly what q36_moe_dispatch returns with a caller workspace -- twice in a row, because
the array keeps the previous call's contents and the second call must not be disturbed by them.

The file sorts last so that a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

E = 256


def _noalloc(moe, torch, eid, se0, se1):
    n = eid.numel()
    dev = eid.device
    ecount = torch.empty(E, dtype=torch.int32, device=dev)
    eoffs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    elist = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
    pos = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    rc = moe.lib.q36_moe_dispatch_noalloc(eid.data_ptr(), n, E, se0, se1, ecount.data_ptr(), eoffs.data_ptr(),
                                          elist.data_ptr(), pos.data_ptr(), moe.stream_ptr())
    moe.check(rc, "dispatch_noalloc")
    return ecount, eoffs, elist[:n], pos[:n]


def test_noalloc_dispatch_matches_workspace_dispatch_twice(moe):
    import torch
    assert torch.cuda.is_available()
    rng = np.random.default_rng(0)
    # two different problems back to back: the second runs over the first one's leftovers in the shared array
    for n, (se0, se1) in ((16384, (0, 256)), (5000, (32, 200))):
        eid = torch.from_numpy(rng.integers(0, E, size=n).astype(np.int32)).cuda()
        want = moe.dispatch(eid, E, se0, se1)
        got = _noalloc(moe, torch, eid, se0, se1)
        torch.cuda.synchronize()
        for g, w, name in zip(got, want, ("ecount", "eoffs", "elist", "pos")):
            assert torch.equal(g, w), f"{name} differs from q36_moe_dispatch (n={n})"


def test_noalloc_empty_input(moe):
    """No entries at all: every expert's count is zero and all offsets are zero, as with q36_moe_dispatch."""
    import torch
    eid = torch.zeros(0, dtype=torch.int32, device="cuda")
    want = moe.dispatch(eid, E, 0, E)
    got = _noalloc(moe, torch, eid, 0, E)
    torch.cuda.synchronize()
    assert torch.equal(got[0], want[0]) and int(got[0].sum()) == 0
    assert torch.equal(got[1], want[1]) and int(got[1].abs().sum()) == 0


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch(moe):
    import torch
    one = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = moe.lib.q36_moe_dispatch_noalloc(one.data_ptr(), 16385, E, 0, E, one.data_ptr(), one.data_ptr(),
                                          one.data_ptr(), one.data_ptr(), None)
    assert rc == moe.ENOSPACE
    rc = moe.lib.q36_moe_dispatch_noalloc(one.data_ptr(), 8, 513, 0, 513, one.data_ptr(), one.data_ptr(),
                                          one.data_ptr(), one.data_ptr(), None)
    assert rc == moe.ENOSPACE
