"""Python handle on the C++ decode runtime (include/kmll_b200_runtime.h).

Mirrors the surface of kmll's quantized runtime (MinistralAllLinearInt8Runtime,
crates/inference/src/model.rs:6327-6480): construct, `prefill`, `generate_greedy`.  All work runs in
libkmll_b200.so; this file only marshals arguments.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from .lib import KmllError, check, load

FORMAT_RS_I8 = 0
FORMAT_W4G128 = 1

T_ATTENTION_NORM, T_WQ, T_WK, T_WV, T_WO, T_FFN_NORM, T_W1, T_W3, T_W2, T_FINAL_NORM, T_EMBEDDING, T_OUTPUT, T_Q_NORM, T_K_NORM = range(14)


class _Config(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("dim", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("hidden_dim", C.c_int), ("vocab_size", C.c_int), ("rotary_dim", C.c_int), ("rope_theta", C.c_float),
                ("norm_eps", C.c_float), ("max_seq_len", C.c_int), ("format", C.c_int), ("fused", C.c_int), ("tp_rank", C.c_int),
                ("tp_size", C.c_int), ("kv_bf16", C.c_int), ("sliding_window", C.c_int)]


@dataclass
class DecoderConfig:
    """TextConfig of kmll (crates/inference/src/model.rs:271-366) reduced to the decoder path."""
    n_layers: int
    dim: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    hidden_dim: int
    vocab_size: int
    rope_theta: float = 1.0e6
    norm_eps: float = 1.0e-6
    max_seq_len: int = 4096
    rotary_dim: int | None = None
    format: int = FORMAT_W4G128
    fused: bool = True
    tp_rank: int = 0
    tp_size: int = 1
    kv_bf16: bool = False  # KV cache in bf16 (not kmll's f32 rows): half the cache bytes and attention traffic
    sliding_window: int = 0  # > 0: attend only the last `sliding_window` positions (kmll: full causal attention only)

    @staticmethod
    def mistral_7b(**kw) -> "DecoderConfig":
        return DecoderConfig(n_layers=32, dim=4096, n_heads=32, n_kv_heads=8, head_dim=128, hidden_dim=14336, vocab_size=32000,
                             rope_theta=1.0e6, norm_eps=1.0e-5, **kw)

    @staticmethod
    def qwen2_0_5b(**kw) -> "DecoderConfig":
        return DecoderConfig(n_layers=24, dim=896, n_heads=14, n_kv_heads=2, head_dim=64, hidden_dim=4864, vocab_size=151936,
                             rope_theta=1.0e6, norm_eps=1.0e-6, **kw)

    def linear_elements(self) -> int:
        """Weight elements streamed per decode token (all linear layers + lm_head)."""
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        per_layer = 2 * q * self.dim + 2 * kv * self.dim + 3 * self.hidden_dim * self.dim
        return self.n_layers * per_layer + self.vocab_size * self.dim

    def _c(self) -> _Config:
        return _Config(self.n_layers, self.dim, self.n_heads, self.n_kv_heads, self.head_dim, self.hidden_dim, self.vocab_size,
                       self.rotary_dim or self.head_dim, self.rope_theta, self.norm_eps, self.max_seq_len, self.format,
                       1 if self.fused else 0, self.tp_rank, self.tp_size, 1 if self.kv_bf16 else 0, int(self.sliding_window))


def _tensor_shape(cfg: DecoderConfig, tensor: int, sharded: bool):
    q, kv = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    tp = cfg.tp_size if sharded else 1
    return {T_WQ: (q // tp, cfg.dim), T_WK: (kv // tp, cfg.dim), T_WV: (kv // tp, cfg.dim), T_WO: (cfg.dim, q // tp),
            T_W1: (cfg.hidden_dim // tp, cfg.dim), T_W3: (cfg.hidden_dim // tp, cfg.dim), T_W2: (cfg.dim, cfg.hidden_dim // tp),
            T_OUTPUT: (cfg.vocab_size // tp, cfg.dim)}[tensor]


class Decoder:
    def __init__(self, cfg: DecoderConfig):
        self.cfg = cfg
        self._lib = load()
        self._h = C.c_void_p()
        c = cfg._c()
        check(self._lib.kmll_decoder_create(C.byref(c), C.byref(self._h)))

    def close(self) -> None:
        if self._h:
            self._lib.kmll_decoder_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def init_random(self, seed: int, std: float = 0.02, tie_embeddings: bool = False) -> None:
        check(self._lib.kmll_decoder_init_random(self._h, seed, std, 1 if tie_embeddings else 0))

    def tp_init(self, unique_id: bytes) -> None:
        buf = (C.c_ubyte * 128).from_buffer_copy(unique_id)
        check(self._lib.kmll_decoder_tp_init(self._h, buf))

    @staticmethod
    def tp_unique_id() -> bytes:
        buf = (C.c_ubyte * 128)()
        check(load().kmll_tp_unique_id(buf))
        return bytes(buf)

    def get_tensor(self, layer: int, tensor: int):
        """This rank's shard: bf16 bits (uint16) for norms/embedding, else (values, scales) numpy arrays."""
        cfg = self.cfg
        if tensor in (T_ATTENTION_NORM, T_FFN_NORM, T_FINAL_NORM, T_EMBEDDING, T_Q_NORM, T_K_NORM):
            n = cfg.vocab_size * cfg.dim if tensor == T_EMBEDDING else cfg.head_dim if tensor in (T_Q_NORM, T_K_NORM) else cfg.dim
            out = np.empty(n, dtype=np.uint16)
            check(self._lib.kmll_decoder_get_tensor(self._h, layer, tensor, out.ctypes.data, None))
            return out.reshape(-1, cfg.dim) if tensor == T_EMBEDDING else out
        rows, cols = _tensor_shape(cfg, tensor, True)
        if cfg.format == FORMAT_W4G128:
            values = np.empty((rows, cols // 2), dtype=np.uint8)
            scales = np.empty((rows, cols // 128), dtype=np.uint16)
        else:
            values = np.empty((rows, cols), dtype=np.int8)
            scales = np.empty(rows, dtype=np.float32)
        check(self._lib.kmll_decoder_get_tensor(self._h, layer, tensor, values.ctypes.data, scales.ctypes.data))
        return values, scales

    def set_tensor(self, layer: int, tensor: int, values: np.ndarray, scales: np.ndarray | None = None) -> None:
        values = np.ascontiguousarray(values)
        sp = None if scales is None else np.ascontiguousarray(scales).ctypes.data
        check(self._lib.kmll_decoder_set_tensor(self._h, layer, tensor, values.ctypes.data, sp))

    def export_archive(self, directory: str, weights_path: str = "") -> None:
        """Write kmll's export directory (manifest.json + one values / scales file pair per linear tensor)."""
        c = self.cfg._c()
        check(self._lib.kmll_decoder_export_archive(self._h, C.byref(c), directory.encode(), weights_path.encode()))

    def load_archive(self, directory: str, expected_weights_path: str | None = None) -> None:
        """Validate an export directory and upload its linear tensors (MinistralAllLinearInt8Runtime::new_from_export)."""
        c = self.cfg._c()
        check(self._lib.kmll_decoder_load_archive(self._h, C.byref(c), directory.encode(),
                                                  None if expected_weights_path is None else expected_weights_path.encode()))

    def set_rope_freqs(self, freqs) -> None:
        """Replace the RoPE frequency table (rotary_dim / 2 values), e.g. by YaRN-scaled frequencies."""
        f = np.ascontiguousarray(freqs, dtype=np.float32)
        check(self._lib.kmll_decoder_set_rope_freqs(self._h, f.ctypes.data, int(f.size)))

    def prefill(self, tokens, token_loop: bool = False) -> None:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        fn = self._lib.kmll_decoder_prefill_token_loop if token_loop else self._lib.kmll_decoder_prefill
        check(fn(self._h, self._stream(), t.ctypes.data, t.size))

    def generate_greedy(self, n_steps: int):
        """[(token, logit)] of n_steps greedy steps (GreedyGenerationStep, crates/inference/src/model.rs:6072-6077)."""
        tokens = np.zeros(n_steps, dtype=np.uint32)
        logits = np.zeros(n_steps, dtype=np.float32)
        check(self._lib.kmll_decoder_generate_greedy(self._h, self._stream(), n_steps, tokens.ctypes.data, logits.ctypes.data))
        return tokens, logits

    def enqueue_steps(self, n_steps: int) -> None:
        check(self._lib.kmll_decoder_enqueue_steps(self._h, self._stream(), n_steps))

    def history(self, first: int, count: int):
        """(tokens, logits) of the steps first .. first + count - 1 run since the last prefill / rewind."""
        packed = np.zeros(count, dtype=np.uint64)
        check(self._lib.kmll_decoder_history(self._h, self._stream(), first, count, packed.ctypes.data))
        return (packed & 0xFFFFFFFF).astype(np.uint32), (packed >> np.uint64(32)).astype(np.uint32).view(np.float32)

    def step_host(self, token: int) -> int:
        out = C.c_uint64()
        check(self._lib.kmll_decoder_step_host(self._h, self._stream(), token, C.byref(out)))
        return int(out.value)

    def rewind(self, position: int) -> None:
        check(self._lib.kmll_decoder_rewind(self._h, self._stream(), position))

    def set_pending(self, packed: int) -> None:
        check(self._lib.kmll_decoder_set_pending(self._h, self._stream(), C.c_uint64(packed)))

    def next_top(self) -> int:
        out = C.c_uint64()
        check(self._lib.kmll_decoder_next_top(self._h, self._stream(), C.byref(out)))
        return int(out.value)

    def last_hidden(self) -> np.ndarray:
        out = np.empty(self.cfg.dim, dtype=np.float32)
        check(self._lib.kmll_decoder_last_hidden(self._h, self._stream(), out.ctypes.data))
        return out

    @property
    def position(self) -> int:
        return int(self._lib.kmll_decoder_position(self._h))

    @property
    def launches_per_step(self) -> int:
        return int(self._lib.kmll_decoder_launches_per_step(self._h))

    @property
    def weight_bytes(self) -> int:
        return int(self._lib.kmll_decoder_weight_bytes(self._h))

    @property
    def kv_bytes(self) -> int:
        return int(self._lib.kmll_decoder_kv_bytes(self._h))

    @property
    def resident_bytes(self) -> int:
        """Bytes of every device allocation of the decoder (weights, KV cache, scratch)."""
        return int(self._lib.kmll_decoder_resident_bytes(self._h))


class BatchDecoder:
    """Lockstep batch of sequences decoded together (kmll_batch_*): shares a Decoder's weights, owns its KV caches.
    Prefill each sequence with the decoder, then `adopt(slot)` it; all sequences must be at the same position."""

    def __init__(self, decoder: Decoder, batch: int):
        self._lib = decoder._lib
        self.decoder = decoder
        self.batch = batch
        self._h = C.c_void_p()
        check(self._lib.kmll_batch_create(decoder._h, batch, C.byref(self._h)))

    def close(self) -> None:
        if self._h:
            self._lib.kmll_batch_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def adopt(self, slot: int) -> None:
        check(self._lib.kmll_batch_adopt(self._h, Decoder._stream(), slot))

    def generate_greedy(self, n_steps: int):
        """(tokens, logits), each [batch, n_steps]."""
        tokens = np.zeros((self.batch, n_steps), dtype=np.uint32)
        logits = np.zeros((self.batch, n_steps), dtype=np.float32)
        check(self._lib.kmll_batch_generate_greedy(self._h, Decoder._stream(), n_steps, tokens.ctypes.data, logits.ctypes.data))
        return tokens, logits

    def enqueue_steps(self, n_steps: int) -> None:
        check(self._lib.kmll_batch_enqueue_steps(self._h, Decoder._stream(), n_steps))

    @property
    def position(self) -> int:
        return int(self._lib.kmll_batch_position(self._h))

    @property
    def launches_per_step(self) -> int:
        return int(self._lib.kmll_batch_launches_per_step(self._h))


def unpack_top1(packed: int):
    """unpack_packed_top_logit (crates/inference/src/model.rs:11808-11812)."""
    token = packed & 0xFFFFFFFF
    logit = np.array([(packed >> 32) & 0xFFFFFFFF], dtype=np.uint32).view(np.float32)[0]
    return int(token), float(logit)


__all__ = ["Decoder", "BatchDecoder", "DecoderConfig", "KmllError", "FORMAT_RS_I8", "FORMAT_W4G128", "unpack_top1"]
