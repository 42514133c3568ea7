"""Session layer on the GPU: the TokenGenerationRuntime surface (crates/inference/src/inference.rs:102-131) over a small
decoder, against the decoder's own device loop and the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from kmll_b200 import runtime as rt
from kmll_b200.session import GenerationOptions, SamplingOptions, Session

pytestmark = pytest.mark.gpu


def small_decoder(fmt):
    cfg = rt.DecoderConfig(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, hidden_dim=512, vocab_size=640, max_seq_len=96,
                           rope_theta=1e6, norm_eps=1e-5, format=fmt)
    dec = rt.Decoder(cfg)
    dec.init_random(5, 0.05, False)
    return dec


@pytest.mark.parametrize("fmt", [rt.FORMAT_W4G128, rt.FORMAT_RS_I8])
def test_session_greedy_stop_token_and_top_logits(cuda, fmt):
    dec = small_decoder(fmt)
    prompt = np.random.default_rng(1).integers(0, 640, 12)
    s = Session(dec)
    with pytest.raises(rt.KmllError):
        s.next_top_logits(4)  # not prefilled
    s.prefill(prompt)
    # the best of the top-k logits is the decoder's own arg-max, and the logits agree with it
    top = s.next_top_logits(5)
    tok, logit = rt.unpack_top1(dec.next_top())
    assert top[0][0] == tok and abs(top[0][1] - logit) <= 1e-4 * max(1.0, abs(logit))
    assert all(top[i][1] >= top[i + 1][1] for i in range(4))
    logits = s.next_logits_to_host()
    assert logits.shape == (640,) and int(np.argmax(logits)) == tok
    free = s.generate_greedy_until(40)
    assert [st.step for st in free] == list(range(40)) and s.tokens()[:12] == [int(t) for t in prompt]
    assert s.tokens()[12:] == [st.token_id for st in free]
    # a stop token that occurs in the free run ends the run right after it, whatever the chunking
    stop = free[21].token_id
    first = [st.token_id for st in free].index(stop)
    for chunk in (16, 5, 1):
        s.CHUNK = chunk
        s.prefill(prompt)
        steps = s.generate_greedy_until(40, 1, stop)
        assert [st.token_id for st in steps] == [st.token_id for st in free[:first + 1]]
        assert s.tokens() == [int(t) for t in prompt] + [st.token_id for st in steps]
        # the sequence can go on from there exactly as the free run did
        more = s.generate_greedy_until(3)
        assert [st.token_id for st in more] == [st.token_id for st in free[first + 1:first + 4]]
    # the k-best loop takes the same tokens
    s.prefill(prompt)
    steps = s.generate_greedy_until(10, 3, None)
    assert [st.token_id for st in steps] == [st.token_id for st in free[:10]] and all(len(st.top_logits) == 3 for st in steps)
    dec.close()


def test_session_sampling_and_report(cuda):
    dec = small_decoder(rt.FORMAT_W4G128)
    prompt = np.random.default_rng(2).integers(0, 640, 9)
    s = Session(dec)
    s.prefill(prompt)
    greedy = [st.token_id for st in s.generate_greedy_until(12)]
    # temperature 0 is arg-max decoding
    s.prefill(prompt)
    cold = s.generate_sampled_top_k_until(12, 8, None, SamplingOptions(temperature=0.0, seed=1))
    assert [st.token_id for st in cold] == greedy
    # the same seed gives the same run; every sampled token is one of the reported candidates
    runs = []
    for _ in range(2):
        res = s.run_generation_request(prompt, GenerationOptions(max_new_tokens=12, top_k=8, sampling=SamplingOptions(temperature=1.5, seed=7)))
        runs.append(res["generated_tokens"])
        assert all(st.token_id in [t for t, _ in st.top_logits] for st in res["steps"])
        assert res["finish_reason"] == ("max-new-tokens", None) and res["backend"] == "w4-g128"
        m = res["memory_stats"]
        assert m["total_resident_bytes"] == m["weights_bytes"] + m["kv_cache_bytes"] + m["scratch_bytes"] and m["kv_cache_bytes"] == 2 * 2 * 96 * 128 * 4
    assert runs[0] == runs[1] and runs[0] != greedy
    with pytest.raises(rt.KmllError):
        s.run_generation_request(prompt, GenerationOptions(max_new_tokens=200))
    dec.close()
