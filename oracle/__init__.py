"""CPU oracle for the quantized decode path: ctypes + numpy access to libkmll_oracle.so.

TEST INFRASTRUCTURE ONLY.  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import this module; the shipped package never does.  Each wrapper below calls the C
restatement in kmll_oracle.c, which cites the reference source lines it follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkmll_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in oracle/Makefile; returns the library path."""
    src = os.path.join(_HERE, "kmll_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libkmll_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load() -> C.CDLL:
    build()
    return C.CDLL(_LIB_PATH)


_lib = _load()

_f32p = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_u32p = C.POINTER(C.c_uint32)
_sz = C.c_size_t


def _p(a: np.ndarray, t):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(t)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


_lib.kmll_oracle_max_threads.restype = C.c_int
_lib.kmll_oracle_lcg_next.restype = C.c_float
_lib.kmll_oracle_lcg_next.argtypes = [C.POINTER(C.c_uint64)]
_lib.kmll_oracle_top1_packed.restype = C.c_uint64
_lib.kmll_oracle_top1_packed.argtypes = [_f32p, _sz]
_lib.kmll_oracle_bf16_from_f32.restype = C.c_uint16
_lib.kmll_oracle_bf16_from_f32.argtypes = [C.c_float]
_lib.kmll_oracle_bf16_to_f32.restype = C.c_float
_lib.kmll_oracle_bf16_to_f32.argtypes = [C.c_uint16]
_lib.kmll_oracle_f16_from_f32.restype = C.c_uint16
_lib.kmll_oracle_f16_from_f32.argtypes = [C.c_float]
_lib.kmll_oracle_f16_to_f32.restype = C.c_float
_lib.kmll_oracle_f16_to_f32.argtypes = [C.c_uint16]


def max_threads() -> int:
    return int(_lib.kmll_oracle_max_threads())


def set_threads(n: int) -> None:
    _lib.kmll_oracle_set_threads(C.c_int(n))


# ---- dtypes -------------------------------------------------------------------------------
def bf16_from_f32(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    _lib.kmll_oracle_bf16_from_f32_array(_p(x, _f32p), _sz(x.size), _p(out, _u16p))
    return out


def bf16_to_f32(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    _lib.kmll_oracle_bf16_to_f32_array(_p(bits, _u16p), _sz(bits.size), _p(out, _f32p))
    return out


def f16_from_f32_scalar(v: float) -> int:
    return int(_lib.kmll_oracle_f16_from_f32(C.c_float(v)))


def f16_to_f32_scalar(bits: int) -> float:
    return float(_lib.kmll_oracle_f16_to_f32(C.c_uint16(bits)))


# ---- seeded generator of the reference's stress harness ------------------------------------
class Lcg:
    """64-bit LCG of the reference's stress commands; the state advances across calls."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def next(self) -> float:
        return float(_lib.kmll_oracle_lcg_next(C.byref(self.state)))

    def fill_f32(self, n: int, scale: float = 1.0) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        _lib.kmll_oracle_lcg_fill_f32(_p(out, _f32p), _sz(n), C.byref(self.state), C.c_float(scale))
        return out

    def fill_bf16(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint16)
        _lib.kmll_oracle_lcg_fill_bf16(_p(out, _u16p), _sz(n), C.byref(self.state))
        return out


# ---- RS-I8 -----------------------------------------------------------------------------------
def rs_i8_quantize(weight_bf16_bits: np.ndarray):
    w = np.ascontiguousarray(weight_bf16_bits, dtype=np.uint16)
    rows, cols = w.shape
    values = np.empty((rows, cols), dtype=np.int8)
    scales = np.empty(rows, dtype=np.float32)
    _lib.kmll_oracle_rs_i8_quantize(_p(w, _u16p), _sz(rows), _sz(cols), _p(values, _i8p), _p(scales, _f32p))
    return values, scales


def rs_i8_dequant(values: np.ndarray, scales: np.ndarray) -> np.ndarray:
    rows, cols = values.shape
    out = np.empty((rows, cols), dtype=np.float32)
    _lib.kmll_oracle_rs_i8_dequant(_p(values, _i8p), _p(scales, _f32p), _sz(rows), _sz(cols), _p(out, _f32p))
    return out


def rs_i8_matvec(values: np.ndarray, scales: np.ndarray, x) -> np.ndarray:
    rows, cols = values.shape
    x = _f32(x)
    assert x.size == cols
    y = np.empty(rows, dtype=np.float32)
    _lib.kmll_oracle_rs_i8_matvec(_p(values, _i8p), _p(scales, _f32p), _sz(rows), _sz(cols), _p(x, _f32p), _p(y, _f32p))
    return y


def rs_i8_linear_batched(x, values: np.ndarray, scales: np.ndarray) -> np.ndarray:
    x = _f32(x)
    batch, in_dim = x.shape
    out_dim, cols = values.shape
    assert cols == in_dim
    y = np.empty((batch, out_dim), dtype=np.float32)
    _lib.kmll_oracle_rs_i8_linear_batched(_p(x, _f32p), _sz(batch), _p(values, _i8p), _p(scales, _f32p),
                                          _sz(out_dim), _sz(in_dim), _p(y, _f32p))
    return y


# ---- W4-G128 -------------------------------------------------------------------------------
def w4_quantize(weight_f32):
    w = _f32(weight_f32)
    rows, cols = w.shape
    assert cols % 128 == 0
    packed = np.empty((rows, cols // 2), dtype=np.uint8)
    gscales = np.empty((rows, cols // 128), dtype=np.uint16)
    _lib.kmll_oracle_w4_quantize(_p(w, _f32p), _sz(rows), _sz(cols), _p(packed, _u8p), _p(gscales, _u16p))
    return packed, gscales


def w4_dequant(packed: np.ndarray, gscales: np.ndarray) -> np.ndarray:
    rows, half = packed.shape
    cols = half * 2
    out = np.empty((rows, cols), dtype=np.float32)
    _lib.kmll_oracle_w4_dequant(_p(packed, _u8p), _p(gscales, _u16p), _sz(rows), _sz(cols), _p(out, _f32p))
    return out


def w4_matvec(packed: np.ndarray, gscales: np.ndarray, x) -> np.ndarray:
    rows, half = packed.shape
    cols = half * 2
    x = _f32(x)
    assert x.size == cols
    y = np.empty(rows, dtype=np.float32)
    _lib.kmll_oracle_w4_matvec(_p(packed, _u8p), _p(gscales, _u16p), _sz(rows), _sz(cols), _p(x, _f32p), _p(y, _f32p))
    return y


def w4_linear_batched(x, packed: np.ndarray, gscales: np.ndarray) -> np.ndarray:
    x = _f32(x)
    batch, in_dim = x.shape
    out_dim, half = packed.shape
    assert half * 2 == in_dim
    y = np.empty((batch, out_dim), dtype=np.float32)
    _lib.kmll_oracle_w4_linear_batched(_p(x, _f32p), _sz(batch), _p(packed, _u8p), _p(gscales, _u16p),
                                       _sz(out_dim), _sz(in_dim), _p(y, _f32p))
    return y


# ---- dense / elementwise -------------------------------------------------------------------
def matvec_bf16(x, weight_bits: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out_dim, in_dim = weight_bits.shape
    y = np.empty(out_dim, dtype=np.float32)
    _lib.kmll_oracle_matvec_bf16(_p(x, _f32p), _p(np.ascontiguousarray(weight_bits), _u16p), _sz(out_dim), _sz(in_dim), _p(y, _f32p))
    return y


def rmsnorm(x, weight_bits: np.ndarray, eps: float) -> np.ndarray:
    x = _f32(x)
    w = np.ascontiguousarray(weight_bits, dtype=np.uint16)
    if x.ndim == 1:
        y = np.empty_like(x)
        _lib.kmll_oracle_rmsnorm(_p(x, _f32p), _p(w, _u16p), _sz(x.size), C.c_float(eps), _p(y, _f32p))
        return y
    batch, dim = x.shape
    y = np.empty_like(x)
    _lib.kmll_oracle_rmsnorm_batched(_p(x, _f32p), _p(w, _u16p), _sz(batch), _sz(dim), C.c_float(eps), _p(y, _f32p))
    return y


def add(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    _lib.kmll_oracle_add(_p(a, _f32p), _p(b, _f32p), _sz(a.size), _p(out, _f32p))
    return out


def silu_mul(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    _lib.kmll_oracle_silu_mul(_p(gate, _f32p), _p(up, _f32p), _sz(gate.size), _p(out, _f32p))
    return out


def rope_frequencies(theta: float, rotary_dim: int) -> np.ndarray:
    out = np.empty(rotary_dim // 2, dtype=np.float32)
    _lib.kmll_oracle_rope_frequencies(C.c_float(theta), _sz(rotary_dim), _p(out, _f32p))
    return out


def rope_frequencies_yarn(theta, rotary_dim, factor, beta_fast, beta_slow, original_max_position) -> np.ndarray:
    out = np.empty(rotary_dim // 2, dtype=np.float32)
    _lib.kmll_oracle_rope_frequencies_yarn(C.c_float(theta), _sz(rotary_dim), C.c_float(factor), C.c_float(beta_fast),
                                           C.c_float(beta_slow), _sz(original_max_position), _p(out, _f32p))
    return out


def apply_rope(x, freqs, position: int, head_dim: int) -> np.ndarray:
    x, freqs = _f32(x), _f32(freqs)
    out = np.empty_like(x)
    flat = x.reshape(-1)
    _lib.kmll_oracle_apply_rope(_p(flat, _f32p), _sz(flat.size), _p(freqs, _f32p), _sz(freqs.size), _sz(position),
                                _sz(head_dim), _p(out.reshape(-1), _f32p))
    return out


def attention_scores(query, key_cache, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim) -> np.ndarray:
    query, key_cache = _f32(query), _f32(key_cache)
    scores = np.empty((n_heads, max_seq_len), dtype=np.float32)
    _lib.kmll_oracle_attention_scores(_p(query, _f32p), _p(key_cache, _f32p), _sz(seq_len), _sz(max_seq_len), _sz(n_heads),
                                      _sz(n_kv_heads), _sz(head_dim), _p(scores, _f32p))
    return scores


def softmax_value(scores, value_cache, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim) -> np.ndarray:
    scores, value_cache = _f32(scores), _f32(value_cache)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    _lib.kmll_oracle_softmax_value(_p(scores, _f32p), _p(value_cache, _f32p), _sz(seq_len), _sz(max_seq_len), _sz(n_heads),
                                   _sz(n_kv_heads), _sz(head_dim), _p(out, _f32p))
    return out


def single_query_attention(query, key_cache, value_cache, seq_len, n_heads, n_kv_heads, head_dim) -> np.ndarray:
    query, key_cache, value_cache = _f32(query), _f32(key_cache), _f32(value_cache)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    _lib.kmll_oracle_single_query_attention(_p(query, _f32p), _p(key_cache, _f32p), _p(value_cache, _f32p), _sz(seq_len),
                                            _sz(n_heads), _sz(n_kv_heads), _sz(head_dim), _p(out, _f32p))
    return out


def prefill_causal_attention(query_batch, key_cache, value_cache, prompt_len, n_heads, n_kv_heads, head_dim) -> np.ndarray:
    query_batch, key_cache, value_cache = _f32(query_batch), _f32(key_cache), _f32(value_cache)
    out = np.empty((prompt_len, n_heads * head_dim), dtype=np.float32)
    _lib.kmll_oracle_prefill_causal_attention(_p(query_batch, _f32p), _p(key_cache, _f32p), _p(value_cache, _f32p),
                                              _sz(prompt_len), _sz(n_heads), _sz(n_kv_heads), _sz(head_dim), _p(out, _f32p))
    return out


def softmax_rows(x) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    _lib.kmll_oracle_softmax_rows(_p(x, _f32p), _sz(rows), _sz(cols), _p(out, _f32p))
    return out


def top1_packed(logits) -> int:
    logits = _f32(logits)
    return int(_lib.kmll_oracle_top1_packed(_p(logits, _f32p), _sz(logits.size)))


def unpack_top1(packed: int):
    """(token, logit) from (f32 bits << 32) | token (crates/inference/src/model.rs:11808-11812)."""
    token = packed & 0xFFFFFFFF
    logit = np.array([(packed >> 32) & 0xFFFFFFFF], dtype=np.uint32).view(np.float32)[0]
    return int(token), float(logit)


def top_k(logits, k: int):
    logits = _f32(logits)
    k = min(k, logits.size)
    tokens = np.empty(k, dtype=np.uint32)
    values = np.empty(k, dtype=np.float32)
    _lib.kmll_oracle_top_k(_p(logits, _f32p), _sz(logits.size), _sz(k), _p(tokens, _u32p), _p(values, _f32p))
    return tokens, values


def embedding(table_bits: np.ndarray, token: int) -> np.ndarray:
    table = np.ascontiguousarray(table_bits, dtype=np.uint16)
    dim = table.shape[1]
    out = np.empty(dim, dtype=np.float32)
    _lib.kmll_oracle_embedding(_p(table, _u16p), _sz(dim), C.c_uint32(token), _p(out, _f32p))
    return out
