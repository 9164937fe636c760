"""Weight container (.int4_t / .scale_t / .f32): byte-exact format and validation, on the CPU.

The expected bytes are built here with ``struct`` from the format statement (header fields and order as written by
better-inference/gguf_convert.cpp:62-88), independently of the library's writer.
"""
import os
import struct

import numpy as np
import pytest

from blackwell_b200 import synth, weight_files as wf
from blackwell_b200.shapes import ModelShape


def test_write_matches_format_bytes_and_reads_back(tmp_path):
    N, K = 48, 160
    packed, _, sc = synth.int4_weights(N, K, 3, full_range=True)
    prefix = str(tmp_path / "7_self_attn.q_proj")
    wf.write_w4(prefix, packed, sc)
    want_w = struct.pack("<5i", K, N, 16, K // 16, 1) + packed.tobytes()
    want_s = struct.pack("<5i", 0, 0, 0, K // 16, N) + sc.astype("<f4").tobytes()
    assert open(prefix + ".int4_t", "rb").read() == want_w
    assert open(prefix + ".scale_t", "rb").read() == want_s
    assert wf.dims_w4(prefix) == (K, N)
    p2, s2 = wf.read_w4(prefix)
    assert np.array_equal(p2, packed) and np.array_equal(s2.view(np.uint32), sc.view(np.uint32))


def test_reader_accepts_a_file_written_by_hand(tmp_path):
    """A file produced without the library (the layout of the reference's converters) loads."""
    N, K = 16, 64
    packed, _, sc = synth.int4_weights(N, K, 9)
    prefix = str(tmp_path / "lm_head")
    with open(prefix + ".int4_t", "wb") as f:
        f.write(np.array([K, N, 16, K // 16, 1], dtype="<i4").tobytes())
        f.write(packed.tobytes())
    with open(prefix + ".scale_t", "wb") as f:
        f.write(np.array([0, 0, 0, K // 16, N], dtype="<i4").tobytes())
        f.write(sc.tobytes())
    p2, s2 = wf.read_w4(prefix)
    assert np.array_equal(p2, packed) and np.array_equal(s2, sc)


def test_reader_rejects_damaged_files(tmp_path):
    N, K = 16, 64
    packed, _, sc = synth.int4_weights(N, K, 9)
    prefix = str(tmp_path / "w")
    with pytest.raises(wf.WeightFileError) as e:
        wf.read_w4(prefix)
    assert e.value.code == -1                                   # missing
    wf.write_w4(prefix, packed, sc)
    with open(prefix + ".int4_t", "r+b") as f:                  # truncated payload
        f.truncate(20 + N * K // 2 - 1)
    with pytest.raises(wf.WeightFileError) as e:
        wf.read_w4(prefix)
    assert e.value.code == -2
    wf.write_w4(prefix, packed, sc)
    with open(prefix + ".scale_t", "r+b") as f:                 # scale header names another matrix
        f.write(struct.pack("<5i", 0, 0, 0, K // 16, N + 1))
    with pytest.raises(wf.WeightFileError) as e:
        wf.read_w4(prefix)
    assert e.value.code == -3
    with pytest.raises(wf.WeightFileError):                     # K not a multiple of 16
        wf.write_w4(str(tmp_path / "bad"), np.zeros((4, 12), np.uint8), np.zeros((4, 1), np.float32))


def test_f32_files_and_synthetic_tree(tmp_path):
    shape = ModelShape("tiny", layers=2, hidden=128, inter=256, n_q_heads=2, n_kv_heads=1, head_dim=128, vocab=96)
    root = str(tmp_path / "weights_int4_tiny")
    nbytes = wf.write_synthetic_tree(root, shape, seed=5)
    names = sorted(os.listdir(root))
    assert len(names) == 2 * (7 * 2 + 2) + 1 + 2 * 2 + 1
    assert sum(os.path.getsize(os.path.join(root, n)) for n in names) == nbytes
    dims = wf.projection_dims(shape)
    for l in range(shape.layers):
        for name, (N, K) in dims.items():
            assert wf.dims_w4(os.path.join(root, f"{l}_{name}")) == (K, N)
        w = wf.read_f32(os.path.join(root, f"{l}_input_layernorm.f32"), shape.hidden)
        assert np.array_equal(w, synth.norm_weight(shape.hidden, 5 + 100 * l + 50))
    qk = wf.read_f32(os.path.join(root, "qk_norms.f32"), shape.layers * 2 * 128).reshape(shape.layers, 2, 128)
    assert np.array_equal(qk[1, 1], synth.norm_weight(128, 5 + 100 + 53))
    assert wf.dims_w4(os.path.join(root, "embed_tokens")) == (128, 96)
    with pytest.raises(wf.WeightFileError):                     # wrong length
        wf.read_f32(os.path.join(root, "final_norm.f32"), shape.hidden + 1)
    # weights written by the tree are inside the reference quantizer's range: no nibble 0 (q = -8)
    p, _ = wf.read_w4(os.path.join(root, "0_mlp.down_proj"))
    assert ((p & 15) != 0).all() and ((p >> 4) != 0).all()
