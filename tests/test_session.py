"""Host logic of the session layer: the xorshift generator, the top-k sampler and the finish reason follow kmll's
definitions (crates/inference/src/inference.rs:7005-7125); checked against an independent restatement in exact integer /
float64 arithmetic and against the properties the algorithm guarantees."""
import math

import numpy as np
import pytest

from kmll_b200.session import (DEFAULT_SEED, GenerationStep, SamplingOptions, XorShift64, finish_reason, sample_from_top_logits,
                               validate_sampling_options)


def xorshift_ref(state):
    m = (1 << 64) - 1
    state ^= (state << 13) & m
    state ^= state >> 7
    state ^= (state << 17) & m
    return state


def test_xorshift_sequence_and_zero_seed():
    r = XorShift64(1)
    s = 1
    for _ in range(100):
        s = xorshift_ref(s)
        assert r.next_u64() == s
    # known first outputs of xorshift64 (13, 7, 17) from state 1
    assert XorShift64(1).next_u64() == 0x40822041
    assert XorShift64(0).state == DEFAULT_SEED  # seed 0 selects the default seed
    u = XorShift64(123).next_unit_f64()
    assert 0.0 <= u < 1.0
    assert u == float(xorshift_ref(123) >> 11) / float(1 << 53)


def test_sampler_short_cuts():
    top = [(7, 3.0), (9, 2.5), (1, -1.0)]
    rng = XorShift64(5)
    before = rng.state
    assert sample_from_top_logits(top, SamplingOptions(temperature=0.0), rng)[:2] == (7, 3.0)
    assert sample_from_top_logits(top[:1], SamplingOptions(temperature=1.0), rng)[:2] == (7, 3.0)
    assert rng.state == before  # neither short cut draws a number
    with pytest.raises(ValueError):
        sample_from_top_logits([], SamplingOptions(), rng)
    with pytest.raises(ValueError):
        sample_from_top_logits([(1, float("nan"))], SamplingOptions(), rng)
    with pytest.raises(ValueError):
        validate_sampling_options(SamplingOptions(temperature=-1.0))
    with pytest.raises(ValueError):
        validate_sampling_options(SamplingOptions(temperature=float("inf")))


def sampler_ref(top, temperature, u):
    """The same algorithm written out again: f32 scaled logits and exponentials, f64 total and threshold."""
    f = np.float32
    scaled = [f(f(l) / f(temperature)) for _, l in top]
    mx = max(scaled)
    w = [float(np.exp(f(v - mx))) for v in scaled]
    thr = u * sum(w)
    for (tok, logit), wi in zip(top, w):
        thr -= wi
        if thr <= 0.0:
            return tok
    return top[-1][0]


@pytest.mark.parametrize("temperature", [0.3, 1.0, 2.5])
def test_sampler_matches_restatement_and_distribution(temperature):
    rng_np = np.random.default_rng(int(temperature * 10))
    top = sorted(((int(t), float(l)) for t, l in zip(rng_np.permutation(50)[:8], rng_np.normal(0, 2, 8))), key=lambda p: -p[1])
    a, b = XorShift64(99), XorShift64(99)
    counts = {}
    for _ in range(4000):
        u = b.next_unit_f64()
        tok, logit, _ = sample_from_top_logits(top, SamplingOptions(temperature=temperature, seed=99), a)
        assert tok == sampler_ref(top, temperature, u)
        assert logit == dict(top)[tok]
        counts[tok] = counts.get(tok, 0) + 1
    p = np.exp(np.array([l for _, l in top]) / temperature)
    p /= p.sum()
    for (tok, _), pi in zip(top, p):
        assert abs(counts.get(tok, 0) / 4000 - pi) < 0.04


def test_finish_reason():
    steps = [GenerationStep(0, 5, 1.0), GenerationStep(1, 2, 0.5)]
    assert finish_reason(steps, 2) == ("stop-token", 2)
    assert finish_reason(steps, 5) == ("max-new-tokens", None)
    assert finish_reason(steps, None) == ("max-new-tokens", None)
    assert finish_reason([], 2) == ("max-new-tokens", None)
    assert math.isclose(SamplingOptions().temperature, 1.0) and SamplingOptions().seed == 0x9E3779B97F4A7C15
