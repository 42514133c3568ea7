"""CPU tests: the shared library loads without a GPU and exports every symbol the headers declare."""
import ctypes as C
import os

import pytest

from kmll_b200 import lib


def test_library_loads_and_exports_every_declared_symbol():
    handle = lib.load()
    declared = lib.declared_symbols()
    assert len(declared) >= 50
    raw = C.CDLL(lib.LIB_PATH)
    missing = [name for name in declared if not hasattr(raw, name)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    assert handle.kmll_version() >= 100
    assert handle.kmll_compiled_arch() == 100


def test_config_struct_mirror_matches_the_library():
    from kmll_b200 import runtime as rt
    handle = lib.load()
    assert handle.kmll_decoder_config_bytes() == C.sizeof(rt._Config)
    c = rt.DecoderConfig(n_layers=1, dim=128, n_heads=2, n_kv_heads=1, head_dim=64, hidden_dim=128, vocab_size=64, kv_bf16=True,
                         sliding_window=7)._c()
    assert (c.kv_bf16, c.sliding_window, c.tp_size, c.fused) == (1, 7, 1, 1)


def test_header_parser_sees_expected_signatures():
    protos = lib.parse_prototypes(lib.HEADERS[0])
    restype, argtypes = protos["kmll_linear_i8"]
    assert restype is C.c_int and len(argtypes) == 7
    assert protos["kmll_single_query_attention_workspace_floats"][0] is C.c_size_t
    assert protos["kmll_last_error"][0] is C.c_char_p


def test_partial_count_is_pure_host_function():
    handle = lib.load()
    assert handle.kmll_linear_top1_partial_count(0) == 0
    assert handle.kmll_linear_top1_partial_count(1) == 1
    assert handle.kmll_linear_top1_partial_count(32) == 1
    assert handle.kmll_linear_top1_partial_count(33) == 2
    assert handle.kmll_linear_top1_partial_count(32000) == 1000


def test_shape_errors_are_reported_not_aborted():
    handle = lib.load()
    # null pointers and bad shapes are rejected on the host before any CUDA call
    rc = handle.kmll_linear_w4g128(None, None, None, None, 16, 128, None)
    assert rc == -1 and b"null" in handle.kmll_last_error()
    rc = handle.kmll_linear_w4g128(None, 16, 16, 16, 16, 100, 16)
    assert rc == -2 and b"128" in handle.kmll_last_error()
    rc = handle.kmll_apply_rope(None, 16, 16, 5, 0, 8, 64, 16)
    assert rc == -2 and b"frequency" in handle.kmll_last_error()
    rc = handle.kmll_write_kv_cache(None, 16, 9, 8, 2, 4, 16)
    assert rc == -2 and b"position" in handle.kmll_last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", os.path.join(tmp_path, "nope.so"))
    with pytest.raises(lib.KmllError):
        lib.load()
