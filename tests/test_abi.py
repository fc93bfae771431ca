"""CPU tests of the boundary: the library builds for sm_100a, loads without a
GPU, exports every symbol the header declares, and rejects bad arguments
before touching the device."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    txt = open(os.path.join(ROOT, "include", "q36_moe.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(q36_moe_\w+)\s*\(", txt)))


def test_every_declared_symbol_is_exported(moe):
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(moe.lib, n), f"{n} declared in include/q36_moe.h but not exported"
    # and the binding covers each of them
    assert set(names) == set(moe._SIGS), set(names) ^ set(moe._SIGS)


def test_abi_version_and_errors(moe):
    assert moe.lib.q36_moe_abi_version() == 1
    assert moe.lib.q36_moe_strerror(0) == b"ok"
    assert b"invalid" in moe.lib.q36_moe_strerror(-1)


def test_stride_and_workspace_sizes(moe):
    assert moe.expert_stride(512, 2048) == 557056           # 512*2048*17/32 (one gate matrix)
    assert moe.expert_stride(2048, 512) == 557056
    assert 3 * moe.expert_stride(512, 2048) == 1671168       # bytes per expert
    w1 = moe.lib.q36_moe_workspace_bytes(1, 256, 8, 2048, 512)
    w8 = moe.lib.q36_moe_workspace_bytes(8, 256, 8, 2048, 512)
    assert 0 < w1 < w8
    assert moe.lib.q36_moe_workspace_bytes(0, 256, 8, 2048, 512) == 0


def test_host_repack_matches_oracle(moe, oracle):
    from q36_b200 import synth
    rng = np.random.default_rng(0)
    b = synth.mxfp4_blocks(rng, 4, 64, 256)
    want = oracle.split_planes(b, 256, 64, 1, 3)
    got = np.empty_like(want)
    rc = moe.lib.q36_moe_repack_mxfp4(b.ctypes.data, 256, 64, 1, 3, got.ctypes.data)
    assert rc == 0
    np.testing.assert_array_equal(got, want)


def test_bad_arguments_are_rejected_without_a_device(moe):
    L = moe.lib
    assert L.q36_moe_router_topk(None, 256, 8, None, None, 1.0, 1, 4, 256, None) == moe.EINVAL
    assert L.q36_moe_quant_e4m3(None, 0, None, None, 4, 2048, None) == moe.EINVAL
    assert L.q36_moe_repack_mxfp4(None, 2048, 512, 0, 1, None) == moe.EINVAL
    one = C.c_void_p(16)
    # k > 8, K not a multiple of 32, empty shard
    assert L.q36_moe_layer(one, one, one, None, None, None, 256, 0, 256, 9, 2048, 512, one, 0, one, 257, 256, 1.0, 1,
                           one, None, None, 4, 0, one, 1 << 30, None) == moe.EINVAL
    assert L.q36_moe_quant_e4m3(one, 0, one, one, 4, 100, None) == moe.EINVAL
    assert L.q36_moe_layer(one, one, one, None, None, None, 256, 8, 8, 8, 2048, 512, one, 0, one, 257, 256, 1.0, 1,
                           one, None, None, 4, 0, one, 1 << 30, None) == moe.EINVAL
    # workspace too small is reported, not overrun
    assert L.q36_moe_layer(one, one, one, None, None, None, 256, 0, 256, 8, 2048, 512, one, 0, one, 257, 256, 1.0, 1,
                           one, None, None, 4, 0, one, 1024, None) == moe.ENOSPACE
