"""The on-disk archive follows kmll's export rules byte for byte: file naming (rowwise_scaled.rs:141-157), tensor index
map (model.rs:9082-9187), raw little-endian contents (src/main.rs:5948-5961), manifest key (model.rs:9047-9053) and the
validation by byte length (model.rs:8984-9069).  Host functions only: no GPU needed."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

from kmll_b200 import lib as klib
from kmll_b200 import runtime as rt


def paths(L, d, index, name, fmt):
    v, s = C.create_string_buffer(512), C.create_string_buffer(512)
    klib.check(L.kmll_archive_file_paths(d.encode(), index, name.encode(), fmt, v, s, 512))
    return v.value.decode(), s.value.decode()


def reference_stem(index, name):
    """format!("{index:04}_{stem}") with every non-ASCII-alphanumeric character of the name replaced by '_'."""
    return f"{index:04d}_" + re.sub(r"[^0-9A-Za-z]", "_", name)


def test_file_names_and_indices_follow_the_reference(tmp_path):
    L = klib.load()
    d = str(tmp_path)
    assert L.kmll_archive_tensor_index(-1, 0) == 0
    for layer, offset in ((0, 0), (0, 6), (3, 2), (31, 6)):
        assert L.kmll_archive_tensor_index(layer, offset) == 1 + layer * 7 + offset
    v, s = paths(L, d, 15, "layers.2.attention.wq.weight", rt.FORMAT_RS_I8)
    assert v == os.path.join(d, reference_stem(15, "layers.2.attention.wq.weight") + ".i8") == os.path.join(d, "0015_layers_2_attention_wq_weight.i8")
    assert s == os.path.join(d, "0015_layers_2_attention_wq_weight.scales.f32")
    v, s = paths(L, d, 0, "output.weight", rt.FORMAT_W4G128)
    assert v.endswith("0000_output_weight.w4") and s.endswith("0000_output_weight.gscales.f16")


def test_tensor_round_trip_is_raw_little_endian_bytes(tmp_path):
    L = klib.load()
    d = str(tmp_path / "export")
    rng = np.random.default_rng(0)
    q = rng.integers(-127, 128, (6, 10), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, 6).astype("<f4")
    klib.check(L.kmll_archive_write_tensor(d.encode(), 3, b"layers.0.attention.wv.weight", rt.FORMAT_RS_I8, 6, 10, q.ctypes.data, sc.ctypes.data))
    v, s = paths(L, d, 3, "layers.0.attention.wv.weight", rt.FORMAT_RS_I8)
    assert open(v, "rb").read() == q.tobytes()            # write_i8_file: one byte per value, row-major
    assert open(s, "rb").read() == sc.astype("<f4").tobytes()  # write_f32_file: little-endian f32
    q2, sc2 = np.zeros_like(q), np.zeros_like(sc)
    klib.check(L.kmll_archive_read_tensor(d.encode(), 3, b"layers.0.attention.wv.weight", rt.FORMAT_RS_I8, 6, 10, q2.ctypes.data, sc2.ctypes.data))
    assert np.array_equal(q, q2) and np.array_equal(sc.view(np.uint32), sc2.view(np.uint32))
    # from_i8_rows_symmetric_parts: lengths must match rows x cols
    assert L.kmll_archive_read_tensor(d.encode(), 3, b"layers.0.attention.wv.weight", rt.FORMAT_RS_I8, 6, 11, q2.ctypes.data, sc2.ctypes.data) != 0
    assert L.kmll_archive_read_tensor(d.encode(), 4, b"layers.0.attention.wv.weight", rt.FORMAT_RS_I8, 6, 10, q2.ctypes.data, sc2.ctypes.data) != 0


def small_config(fmt):
    return rt.DecoderConfig(n_layers=2, dim=128, n_heads=2, n_kv_heads=1, head_dim=64, hidden_dim=256, vocab_size=300, format=fmt)


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
def test_manifest_and_validation(tmp_path, fmt):
    L = klib.load()
    cfg = small_config(fmt)
    c = cfg._c()
    d = str(tmp_path / "archive")
    rng = np.random.default_rng(1)
    shapes = [(-1, 0, "output.weight", 300, 128)]
    for l in range(2):
        for o, (nm, r, k) in enumerate((("attention.wq.weight", 128, 128), ("attention.wk.weight", 64, 128), ("attention.wv.weight", 64, 128),
                                        ("attention.wo.weight", 128, 128), ("feed_forward.w1.weight", 256, 128), ("feed_forward.w3.weight", 256, 128),
                                        ("feed_forward.w2.weight", 128, 256))):
            shapes.append((l, o, f"layers.{l}.{nm}", r, k))
    for layer, off, name, rows, cols in shapes:
        if fmt == rt.FORMAT_RS_I8:
            vals, sc = rng.integers(-127, 128, (rows, cols), dtype=np.int8), rng.uniform(0, 1, rows).astype(np.float32)
        else:
            vals, sc = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8), rng.integers(0x1C00, 0x2400, (rows, cols // 128)).astype(np.uint16)
        klib.check(L.kmll_archive_write_tensor(d.encode(), L.kmll_archive_tensor_index(layer, off), name.encode(), fmt, rows, cols,
                                               vals.ctypes.data, sc.ctypes.data))
    assert L.kmll_archive_validate(d.encode(), C.byref(c), None) != 0  # no manifest yet
    klib.check(L.kmll_archive_write_manifest(d.encode(), C.byref(c), b"/models/demo/consolidated.safetensors"))
    manifest = json.load(open(os.path.join(d, "manifest.json")))
    assert manifest["quantization"] == ("row-symmetric-int8-with-f32-row-scales" if fmt == rt.FORMAT_RS_I8 else
                                        "group128-symmetric-int4-with-f16-group-scales")
    assert manifest["planned_tensor_count"] == manifest["exported_tensor_count"] == 1 + 2 * 7 and manifest["complete_export"] is True
    assert [t["index"] for t in manifest["tensors"]] == list(range(15)) and manifest["tensors"][0]["name"] == "output.weight"
    assert manifest["tensors"][9]["name"] == "layers.1.attention.wk.weight"  # 1 + 1 * 7 + 1
    klib.check(L.kmll_archive_validate(d.encode(), C.byref(c), None))
    klib.check(L.kmll_archive_validate(d.encode(), C.byref(c), b"/models/demo/consolidated.safetensors"))
    assert L.kmll_archive_validate(d.encode(), C.byref(c), b"/models/other.safetensors") != 0  # generated from another checkpoint
    other = small_config(rt.FORMAT_W4G128 if fmt == rt.FORMAT_RS_I8 else rt.FORMAT_RS_I8)._c()
    assert L.kmll_archive_validate(d.encode(), C.byref(other), None) != 0  # unsupported quantization for that decoder
    # a file with the wrong byte length fails the validation
    v, _ = paths(L, d, 4, "layers.0.attention.wo.weight", fmt)
    with open(v, "ab") as f:
        f.write(b"\0")
    assert L.kmll_archive_validate(d.encode(), C.byref(c), None) != 0
    assert b"bytes, expected" in L.kmll_last_error()
    assert L.kmll_archive_validate((d + "/manifest.json").encode(), C.byref(c), None) != 0  # not a directory
