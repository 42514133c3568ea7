"""Decode attention through the entry point that owns its scratch (for hosts that cannot allocate device
memory): it must give the same result as the workspace-taking entry point, call after call, because both
run the same kernel and the built-in scratch is re-used between calls."""
import ctypes as C

import numpy as np
import pytest
import torch

from kmll_b200 import lib

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_noalloc_attention_matches_workspace_entry_point_on_consecutive_calls(cuda):
    L = lib.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    n_heads, n_kv, hd, max_seq = 32, 8, 128, 2304
    gen = torch.Generator(device="cuda").manual_seed(123)
    ws_floats = L.kmll_single_query_attention_workspace_floats(n_heads, hd, max_seq)
    workspace = torch.zeros(ws_floats, dtype=torch.float32, device="cuda")
    out_ref = torch.empty(n_heads * hd, device="cuda")
    out_new = torch.full((n_heads * hd,), float("nan"), device="cuda")
    # two calls in a row, different data and sequence lengths: the second call finds the first call's leftovers
    for seq_len in (2100, 65):
        q = torch.randn(n_heads * hd, generator=gen, device="cuda")
        kc = torch.randn(max_seq * n_kv * hd, generator=gen, device="cuda")
        vc = torch.randn(max_seq * n_kv * hd, generator=gen, device="cuda")
        rc = L.kmll_single_query_attention(stream, _ptr(q), _ptr(kc), _ptr(vc), seq_len, max_seq, n_heads, n_kv, hd, _ptr(workspace),
                                           _ptr(out_ref))
        assert rc == 0, L.kmll_last_error()
        rc = L.kmll_single_query_attention_noalloc(stream, _ptr(q), _ptr(kc), _ptr(vc), seq_len, max_seq, n_heads, n_kv, hd,
                                                   _ptr(out_new))
        assert rc == 0, L.kmll_last_error()
        torch.cuda.synchronize()
        diff = float(torch.max(torch.abs(out_new - out_ref)))
        assert np.isfinite(diff) and diff <= 5e-5, (seq_len, diff)  # the bound the other attention tests use


def test_noalloc_attention_rejects_geometry_beyond_its_scratch(cuda):
    L = lib.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    n_heads, n_kv, hd, max_seq = 128, 16, 128, 8192  # needs ~1.07 M floats of scratch: more than the built-in array
    assert L.kmll_single_query_attention_workspace_floats(n_heads, hd, max_seq) > 544768
    q = torch.zeros(n_heads * hd, device="cuda")
    cache = torch.zeros(16 * n_kv * hd, device="cuda")  # never touched: the call must fail before launching
    out = torch.zeros(n_heads * hd, device="cuda")
    rc = L.kmll_single_query_attention_noalloc(stream, _ptr(q), _ptr(cache), _ptr(cache), 4, max_seq, n_heads, n_kv, hd, _ptr(out))
    assert rc == -5 and b"scratch" in L.kmll_last_error()
