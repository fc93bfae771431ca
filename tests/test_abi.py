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
    return sorted(set(re.findall(r"\b(q36_(?:moe|gguf)_\w+)\s*\(", txt)))


def test_every_declared_symbol_is_exported(moe):
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(moe.lib, n), f"{n} declared in include/q36_moe.h but not exported"
    # and the binding covers each of them
    assert set(names) == set(moe._SIGS), set(names) ^ set(moe._SIGS)


def test_abi_version_and_errors(moe):
    assert moe.lib.q36_moe_abi_version() == 2
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


def test_unsupported_expert_counts_and_shard_ranges_are_rejected(moe):
    """The router keeps n_expert / 32 logits per lane: any other count must be refused by the whole-layer entries
    too (it used to fall through to the 32-expert code and route over the first 32 logits only)."""
    L = moe.lib
    one = C.c_void_p(16)
    for E in (512, 96, 384, 48):
        assert L.q36_moe_layer(one, one, one, None, None, None, E, 0, E, 8, 2048, 512, one, 0, one, E + 1, E, 1.0, 1,
                               one, None, None, 4, 0, one, 1 << 30, None) == moe.EINVAL, E
        assert L.q36_moe_router_topk(one, E, 8, one, one, 1.0, 1, 4, E, None) == moe.EINVAL, E
    ws = C.c_void_p(4096)
    # shard ranges of the dispatch entries: negative, reversed, beyond n_expert
    for se0, se1 in ((-1, 8), (9, 8), (0, 257)):
        assert L.q36_moe_dispatch(one, 8, 256, se0, se1, one, one, one, one, ws, 1 << 20, None) == moe.EINVAL
        assert L.q36_moe_dispatch_noalloc(one, 8, 256, se0, se1, one, one, one, one, None) == moe.EINVAL


def test_one_launch_kernel_bounds_its_matrix_sizes(moe):
    """The decode kernel stages a tile's scale bytes in slots sized for K <= 2048: a larger layer has to take the
    two grouped-GEMM launches instead of overrunning shared memory."""
    L = moe.lib
    assert L.q36_moe_one_launch_fits(72, 256, 2048, 512) == 1
    assert L.q36_moe_one_launch_fits(72, 256, 4096, 512) == 0
    assert L.q36_moe_one_launch_fits(72, 256, 2048, 4096) == 0
    assert L.q36_moe_one_launch_fits(72, 256, 2048 + 128, 512) == 0       # not a multiple of 512
    assert L.q36_moe_one_launch_fits(1 << 20, 256, 2048, 512) == 0         # beyond the per-block tile table


_C_UNIT = r"""
#include <string.h>
#include "q36_moe.h"
#include "q36_moe_void.h"
int main(int argc, char **argv) {
    (void)argv;   /* host-only calls: work without a device */
    unsigned char blocks[2 * 4 * 1 * 17], planes[2 * 4 * 17];
    memset(blocks, 7, sizeof blocks);
    if (q36_moe_abi_version() != 2) return 2;
    if (q36_moe_expert_stride(4, 32) != 4 * 16 + 4) return 3;
    q36_cuda_moe_repack_mxfp4(blocks, 32, 4, 0, 2, planes);       /* succeeds: returns */
    if (planes[0] != 7) return 4;
    if (argc > 1) q36_cuda_moe_repack_mxfp4(0, 32, 4, 0, 2, planes);   /* fails: message + exit(1), like CK() */
    return 0;
}
"""


def test_plain_c99_unit_compiles_links_and_the_void_shim_exits_like_CK(moe, tmp_path):
    """A C99 translation unit that includes the two headers builds with -Wall -Werror -pedantic and links against
    the library; the void twins return on success and print + exit(1) on failure (q36_engine.cu:45)."""
    import subprocess
    src = tmp_path / "unit.c"
    src.write_text(_C_UNIT)
    exe = tmp_path / "unit"
    libdir = os.path.dirname(moe.LIB_PATH)
    cuda_lib = "/usr/local/cuda/lib64"
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), str(src),
           "-L", libdir, "-lq36moe", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath-link,{cuda_lib}", f"-Wl,-rpath,{cuda_lib}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    ok = subprocess.run([str(exe)], capture_output=True, text=True)
    assert ok.returncode == 0, (ok.returncode, ok.stderr)
    bad = subprocess.run([str(exe), "fail"], capture_output=True, text=True)
    assert bad.returncode == 1
    assert "repack_mxfp4" in bad.stderr and "invalid argument" in bad.stderr
