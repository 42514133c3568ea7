"""Session layer over the decoder: the surface kmll's callers use (trait TokenGenerationRuntime,
crates/inference/src/inference.rs:102-131) with its generation loops, host-side top-k sampling and memory report.

Host logic only: every token still comes from the CUDA decoder (kmll_b200.runtime.Decoder).  The arithmetic of the
sampler follows kmll's to the type: f32 for the scaled logits and their exponentials, f64 for the running total and the
threshold (inference.rs:7069-7125), the xorshift generator and its unit-interval mapping (inference.rs:7025-7052)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import ops
from .lib import KmllError, check
from .runtime import FORMAT_W4G128, Decoder, unpack_top1

DEFAULT_SEED = 0x9E3779B97F4A7C15  # SamplingOptions::default (inference.rs:353-360)
F32_EPSILON = float(np.finfo(np.float32).eps)
_M64 = (1 << 64) - 1


class XorShift64:
    """inference.rs:7025-7052: state ^= state << 13; ^= state >> 7; ^= state << 17 on 64 bits; seed 0 means the default."""

    def __init__(self, seed: int):
        self.state = (seed & _M64) or DEFAULT_SEED

    def next_u64(self) -> int:
        s = self.state
        s ^= (s << 13) & _M64
        s ^= s >> 7
        s ^= (s << 17) & _M64
        self.state = s
        return s

    def next_unit_f64(self) -> float:
        return float(self.next_u64() >> 11) * (1.0 / float(1 << 53))


@dataclass
class SamplingOptions:
    temperature: float = 1.0
    seed: int = DEFAULT_SEED


def validate_sampling_options(sampling: SamplingOptions) -> None:
    """inference.rs:7054-7067."""
    if not math.isfinite(sampling.temperature) or sampling.temperature < 0.0:
        raise ValueError(f"sampling temperature must be finite and nonnegative, got {sampling.temperature}")


def sample_from_top_logits(top_logits, sampling: SamplingOptions, rng: XorShift64):
    """inference.rs:7069-7125.  top_logits = [(token, logit)] best first; returns (token, logit, top_logits)."""
    if len(top_logits) == 0:
        raise ValueError("runtime produced no top logits")
    if any(not math.isfinite(float(l)) for _, l in top_logits):
        raise ValueError("top logits must be finite")
    validate_sampling_options(sampling)
    first = top_logits[0]
    if len(top_logits) == 1 or sampling.temperature <= F32_EPSILON:
        return int(first[0]), float(first[1]), top_logits
    f = np.float32
    t = f(sampling.temperature)
    scaled = [f(f(l) / t) for _, l in top_logits]
    max_scaled = f(-np.inf)
    for v in scaled:
        max_scaled = max(max_scaled, v)
    weights = []
    total = 0.0
    for v in scaled:
        w = float(np.exp(f(v - max_scaled), dtype=np.float32))
        total += w
        weights.append(w)
    if not math.isfinite(total) or total <= 0.0:
        raise ValueError(f"invalid sampling weight total {total}")
    threshold = rng.next_unit_f64() * total
    for (token, logit), w in zip(top_logits, weights):
        threshold -= w
        if threshold <= 0.0:
            return int(token), float(logit), top_logits
    last = top_logits[-1]
    return int(last[0]), float(last[1]), top_logits


@dataclass
class GenerationStep:
    """GreedyGenerationStep (crates/inference/src/model.rs:765-770)."""
    step: int
    token_id: int
    logit: float
    top_logits: list = field(default_factory=list)


@dataclass
class GenerationOptions:
    max_new_tokens: int = 16
    top_k: int = 1
    stop_token_id: int | None = None
    sampling: SamplingOptions | None = None  # None: greedy


def finish_reason(steps, stop_token_id):
    """generation_finish_reason (inference.rs:7005-7023): ("stop-token", id) or ("max-new-tokens", None)."""
    if stop_token_id is not None and steps and steps[-1].token_id == stop_token_id:
        return "stop-token", stop_token_id
    return "max-new-tokens", None


class Session:
    """One sequence on one decoder.  Method names and meaning follow TokenGenerationRuntime."""

    CHUNK = 16  # device-resident greedy steps between two looks at the stop token

    def __init__(self, decoder: Decoder):
        self.dec = decoder
        self._tokens: list[int] = []
        self._ready = False
        self._logits = torch.empty(decoder.cfg.vocab_size, dtype=torch.float32, device="cuda")

    # ---- TokenGenerationRuntime ----------------------------------------------------------------
    def backend(self) -> str:
        return "w4-g128" if self.dec.cfg.format == FORMAT_W4G128 else "rowwise-scaled-i8"

    def memory_stats(self) -> dict:
        """RuntimeMemoryStats (model.rs:803-808).  Scratch is everything resident that is neither a weight in its
        canonical layout nor KV cache: activations, workspaces, and the prepared-layout copy of W4-G128 weights."""
        w, kv, total = self.dec.weight_bytes, self.dec.kv_bytes, self.dec.resident_bytes
        return {"weights_bytes": w, "kv_cache_bytes": kv, "scratch_bytes": max(0, total - w - kv), "total_resident_bytes": total}

    @property
    def max_seq_len(self) -> int:
        return self.dec.cfg.max_seq_len

    def tokens(self) -> list[int]:
        return list(self._tokens)

    def reset_sequence(self) -> None:
        """Forget the sequence; the next prefill starts the KV cache from position 0."""
        self._tokens = []
        self._ready = False

    def synchronize(self) -> None:
        torch.cuda.current_stream().synchronize()

    def prefill(self, prompt_tokens) -> None:
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise KmllError(-2, "prompt tokens must not be empty")
        if len(prompt) > self.max_seq_len:
            raise KmllError(-2, f"prompt of {len(prompt)} tokens exceeds max_seq_len {self.max_seq_len}")
        self.reset_sequence()
        self.dec.prefill(np.asarray(prompt, dtype=np.int64))
        self._tokens = prompt
        self._ready = True

    def _require_ready(self):
        if not self._ready:
            raise KmllError(-5, "runtime must be prefilled before generating")

    def next_logits_to_host(self) -> np.ndarray:
        self._require_ready()
        check(self.dec._lib.kmll_decoder_next_logits(self.dec._h, self.dec._stream(), self._logits.data_ptr()))
        return self._logits.cpu().numpy()

    def next_top_logits(self, top_k: int):
        self._require_ready()
        k = max(1, int(top_k))
        check(self.dec._lib.kmll_decoder_next_logits(self.dec._h, self.dec._stream(), self._logits.data_ptr()))
        tok, val = ops.top_k_f32(self._logits, k)
        return [(int(t), float(v)) for t, v in zip(tok.cpu().tolist(), val.cpu().tolist())]

    def advance_with_token(self, token_id: int) -> None:
        self._require_ready()
        if len(self._tokens) >= self.max_seq_len:
            raise KmllError(-2, "sequence is at max_seq_len")
        self.dec.step_host(int(token_id))
        self._tokens.append(int(token_id))

    def generate_greedy_until(self, max_new_tokens: int, top_k: int = 1, stop_token_id: int | None = None):
        """Arg-max decoding; stops after the stop token has been taken into the sequence.  With top_k <= 1 the steps run
        on the device in chunks (the token is fed back without a host round trip) and a chunk that ran past the stop token
        is rolled back; with top_k > 1 every step also reports the k best logits, as kmll's loop does."""
        self._require_ready()
        steps = []
        if top_k > 1:
            for step in range(max_new_tokens):
                top = self.next_top_logits(top_k)
                token, logit = top[0]
                self.advance_with_token(token)
                steps.append(GenerationStep(step, token, logit, top))
                if stop_token_id is not None and token == stop_token_id:
                    break
            return steps
        while len(steps) < max_new_tokens:
            n = min(self.CHUNK if stop_token_id is not None else max_new_tokens, max_new_tokens - len(steps),
                    self.max_seq_len - len(self._tokens))
            if n <= 0:
                raise KmllError(-2, "sequence is at max_seq_len")
            start = self.dec.position
            toks, logits = self.dec.generate_greedy(n)
            taken = n
            if stop_token_id is not None:
                hit = [i for i in range(n) if int(toks[i]) == stop_token_id]
                if hit and hit[0] + 1 < n:  # the chunk ran past the stop token: go back; the token after it is the pending one
                    taken = hit[0] + 1
                    bits = int(np.asarray(logits[taken:taken + 1], dtype=np.float32).view(np.uint32)[0])
                    self.dec.rewind(start + taken)
                    self.dec.set_pending((bits << 32) | int(toks[taken]))
            for i in range(taken):
                steps.append(GenerationStep(len(steps), int(toks[i]), float(logits[i]), [(int(toks[i]), float(logits[i]))]))
                self._tokens.append(int(toks[i]))
            if stop_token_id is not None and steps and steps[-1].token_id == stop_token_id:
                break
        return steps

    def generate_sampled_top_k_until(self, max_new_tokens: int, top_k: int, stop_token_id: int | None, sampling: SamplingOptions):
        """generate_sampled_top_k_until (inference.rs:6595-6627)."""
        rng = XorShift64(sampling.seed)
        steps = []
        for step in range(max_new_tokens):
            top = self.next_top_logits(max(1, top_k))
            token, logit, top = sample_from_top_logits(top, sampling, rng)
            self.advance_with_token(token)
            steps.append(GenerationStep(step, token, logit, top))
            if stop_token_id is not None and token == stop_token_id:
                break
        return steps

    def run_generation_request(self, prompt_tokens, options: GenerationOptions) -> dict:
        """run_generation_with_runtime (inference.rs:6442-6480): prefill and decode timed separately, a synchronisation
        at both ends of each."""
        import time
        if len(prompt_tokens) + options.max_new_tokens > self.max_seq_len:
            raise KmllError(-2, f"prompt + max_new_tokens = {len(prompt_tokens) + options.max_new_tokens} exceeds max_seq_len {self.max_seq_len}")
        t0 = time.perf_counter()
        self.prefill(prompt_tokens)
        self.synchronize()
        prefill_s = time.perf_counter() - t0
        stats = self.memory_stats()
        t0 = time.perf_counter()
        if options.sampling is None:
            steps = self.generate_greedy_until(options.max_new_tokens, options.top_k, options.stop_token_id)
        else:
            steps = self.generate_sampled_top_k_until(options.max_new_tokens, options.top_k, options.stop_token_id, options.sampling)
        self.synchronize()
        decode_s = time.perf_counter() - t0
        all_tokens = self.tokens()
        return {"backend": self.backend(), "prompt_tokens": list(map(int, prompt_tokens)), "generated_tokens": all_tokens[len(prompt_tokens):],
                "all_tokens": all_tokens, "memory_stats": stats, "timings": {"prefill_seconds": prefill_s, "decode_seconds": decode_s},
                "finish_reason": finish_reason(steps, options.stop_token_id), "steps": steps}


__all__ = ["Session", "SamplingOptions", "GenerationOptions", "GenerationStep", "XorShift64", "sample_from_top_logits",
           "validate_sampling_options", "finish_reason", "unpack_top1"]
