"""GGUF in: the library's reader against a file written here and against the reference's own reader.

CPU tests (no device): directory, metadata, alignment, error paths, and the repack of the expert tensors found
in the file.  The upload entries need a device and are covered in test_gpu_parity.py.
"""
import ctypes as C
import os

import numpy as np
import pytest

from q36_b200 import synth


@pytest.fixture(scope="module")
def small_file(tmp_path_factory):
    """Two MoE blocks with small matrices (E = 8, D = 128, FF = 64) plus metadata of every kind the reader must skip."""
    d = tmp_path_factory.mktemp("gguf")
    path = str(d / "two_blocks.gguf")
    rng = np.random.default_rng(5)
    ws, tensors = [], {}
    for L in (0, 3):
        w = synth.layer(seed=10 + L, n_expert=8, D=128, FF=64)
        ws.append(w)
        tensors.update(synth.layer_tensors(w, L, router=rng.standard_normal((8, 128), dtype=np.float32),
                                           shared_gate=rng.standard_normal(128, dtype=np.float32),
                                           post_norm=rng.standard_normal(128, dtype=np.float32)))
    tensors["output_norm.weight"] = (synth.GGML_F32, (128,), rng.standard_normal(128, dtype=np.float32).tobytes())
    meta = {"general.architecture": "qwen3moe", "qwen3moe.block_count": 4, "qwen3moe.expert_count": 8,
            "general.alignment": 64, "tokenizer.ggml.tokens": ["a", "bc", "def"], "tokenizer.ggml.token_type": [1, 2, 3],
            "qwen3moe.rope.freq_base": 1e6, "general.flag": True}
    synth.write_gguf(path, tensors, meta, alignment=64)
    return path, ws, tensors


def test_directory_matches_what_was_written_and_the_reference_reader(moe, oracle, small_file):
    path, ws, tensors = small_file
    with moe.GgufFile(path) as g:
        assert g.meta_u32("general.alignment") == 64
        assert g.meta_u32("qwen3moe.expert_count") == 8
        raw = open(path, "rb").read()
        for name, (typ, dims, data) in tensors.items():
            t, d, buf = g.tensor(name)
            assert (t, d) == (typ, tuple(dims)), name
            assert buf.tobytes() == bytes(data), name
            ref = oracle.ref_gguf_probe(path, name)
            if ref is not None:                       # the reference's gguf.c, compiled into oracle/_ref
                assert ref["type"] == t and ref["dims"] == d and ref["nbytes"] == buf.size
                assert ref["alignment"] == 64 and ref["n_tensors"] == len(tensors)
                assert raw[ref["file_offset"]:ref["file_offset"] + ref["nbytes"]] == buf.tobytes()
        assert g.layer_shape(0) == (8, 128, 64, (39, 39, 39))
        assert g.layer_shape(3) == (8, 128, 64, (39, 39, 39))


def test_expert_tensors_from_the_file_repack_like_upload(moe, oracle, small_file):
    """blk.N.ffn_*_exps.weight bytes found through the reader -> split planes == the oracle's restatement of upload()."""
    path, ws, _ = small_file
    with moe.GgufFile(path) as g:
        for L, w in zip((0, 3), ws):
            for key, name, K, M in (("gate", "ffn_gate_exps", 128, 64), ("down", "ffn_down_exps", 64, 128)):
                _, dims, buf = g.tensor(f"blk.{L}.{name}.weight")
                assert dims == (K, M, 8)
                want = oracle.split_planes(w[key], K, M, 2, 7)
                got = np.empty_like(want)
                assert moe.lib.q36_moe_repack_mxfp4(buf.ctypes.data, K, M, 2, 7, got.ctypes.data) == 0
                np.testing.assert_array_equal(got, want)


def test_reader_errors_are_reported_not_crashed(moe, small_file, tmp_path):
    path, _, tensors = small_file
    h = C.c_void_p()
    L = moe.lib
    assert L.q36_gguf_open(os.fsencode(str(tmp_path / "missing.gguf")), C.byref(h)) == moe.EIO
    assert b"open" in L.q36_gguf_last_error()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    assert L.q36_gguf_open(os.fsencode(str(bad)), C.byref(h)) == moe.EIO
    assert b"not a GGUF" in L.q36_gguf_last_error()
    raw = open(path, "rb").read()
    v2 = tmp_path / "v2.gguf"
    v2.write_bytes(raw[:4] + (2).to_bytes(4, "little") + raw[8:])
    assert L.q36_gguf_open(os.fsencode(str(v2)), C.byref(h)) == moe.EIO
    assert b"version 2" in L.q36_gguf_last_error()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(raw[:len(raw) - 100])                         # the last tensor now runs past the end
    assert L.q36_gguf_open(os.fsencode(str(cut)), C.byref(h)) == moe.EIO
    assert b"past the end" in L.q36_gguf_last_error()
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(raw[:200])                                  # inside the metadata
    assert L.q36_gguf_open(os.fsencode(str(trunc)), C.byref(h)) == moe.EIO
    with moe.GgufFile(path) as g:
        assert L.q36_gguf_tensor(g.h, b"blk.9.nope", None, None, None, None, None) == moe.EIO
        assert L.q36_moe_gguf_layer_shape(g.h, 1, None, None, None, None) == moe.EIO     # block 1 has no expert tensors
        one = C.c_void_p(16)
        assert L.q36_moe_gguf_upload_layer(g.h, 0, 0, 9, one, one, one) == moe.EINVAL     # e1 beyond the 8 experts
    # a Q8_0 shared expert, as in the published model, is refused with a message rather than misread
    t2 = dict(tensors)
    t2["blk.0.ffn_gate_shexp.weight"] = (synth.GGML_Q8_0, (128, 64), bytes(64 * 4 * 34))
    q8 = str(tmp_path / "q8.gguf")
    synth.write_gguf(q8, t2)
    with moe.GgufFile(q8) as g:
        one = C.c_void_p(16)
        assert L.q36_moe_gguf_upload_shared(g.h, 0, one, one, one) == moe.EUNSUPPORTED
        assert b"only MXFP4" in L.q36_gguf_last_error()
