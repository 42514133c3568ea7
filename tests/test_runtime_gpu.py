"""GPU parity tests of the decode runtime against the CPU oracle model: same quantized bytes on both
sides, identical greedy tokens (checked against the oracle's top-2 margin), logits and hidden states
within kmll's tolerances."""
import numpy as np
import pytest
import torch

from kmll_b200 import runtime as rt
from kmll_b200.lib import KmllError
from oracle_model import OracleDecoder

pytestmark = pytest.mark.gpu
F = np.float32


def tiny(fmt, fused=True, **kw):
    base = dict(n_layers=2, dim=256, n_heads=4, n_kv_heads=2, head_dim=64, hidden_dim=512, vocab_size=640, rope_theta=1e6, norm_eps=1e-6,
                max_seq_len=48, format=fmt, fused=fused)
    base.update(kw)
    return rt.DecoderConfig(**base)


def make(cfg, seed=2, std=0.05, tie=False):
    dec = rt.Decoder(cfg)
    dec.init_random(seed, std, tie)
    return dec


def check_against_oracle(dec, cfg, prompt, n_steps, batched_prefill, hid_tol=2e-4, min_margin=1e-3, logit_tol=1e-3):
    ora = OracleDecoder(cfg, dec)
    logits = ora.prefill(prompt)
    dec.prefill(prompt, token_loop=not batched_prefill)
    hid = dec.last_hidden()
    scale = np.max(np.abs(ora.hidden))
    assert np.max(np.abs(hid - ora.hidden)) <= hid_tol * max(scale, 1.0), "hidden state after prefill"
    steps, _ = ora.generate_greedy(logits, n_steps)
    tokens, glogits = dec.generate_greedy(n_steps)
    for i, (tok, logit, margin) in enumerate(steps):
        if margin < min_margin:
            break  # a near-tie in the oracle: either token is a faithful arg-max, later steps diverge legitimately
        assert int(tokens[i]) == tok, f"greedy token differs at step {i} (oracle margin {margin})"
        assert abs(float(glogits[i]) - logit) <= logit_tol * max(abs(logit), 1.0)
    assert dec.position == len(prompt) + n_steps


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
@pytest.mark.parametrize("fused", [True, False])
def test_decode_matches_oracle(cuda, fmt, fused):
    cfg = tiny(fmt, fused)
    dec = make(cfg)
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab_size, 9)
    check_against_oracle(dec, cfg, prompt, 6, batched_prefill=False)
    dec.close()


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
@pytest.mark.parametrize("window", [1, 24, 70])
@pytest.mark.parametrize("batched_prefill", [False, True])
def test_sliding_window_matches_oracle(cuda, fmt, window, batched_prefill):
    """sliding_window: the oracle attends the last `window` rows of its cache.  max_seq_len 200 gives the decode kernel
    four 52-position slices; with 110-token prompts a window of 24 lies inside one slice or straddles two, one of 70
    covers slices partly, and the slices before the window leave without a partial.  f32 cache: the f32 tolerances."""
    cfg = tiny(fmt, True, n_heads=8, n_kv_heads=2, head_dim=128, dim=256, max_seq_len=200, sliding_window=window)
    dec = make(cfg)
    prompt = np.random.default_rng(window).integers(0, cfg.vocab_size, 110)
    check_against_oracle(dec, cfg, prompt, 8, batched_prefill=batched_prefill)
    dec.close()


def test_sliding_window_other_step_forms_and_bf16(cuda):
    for fused, rotary_dim, kv_bf16 in [(False, None, False), (True, 32, False), (True, None, True)]:
        cfg = tiny(rt.FORMAT_W4G128, fused, rotary_dim=rotary_dim, max_seq_len=96, sliding_window=20, kv_bf16=kv_bf16)
        dec = make(cfg)
        prompt = np.random.default_rng(6).integers(0, cfg.vocab_size, 66)
        check_against_oracle(dec, cfg, prompt, 5, batched_prefill=fused, **(BF16_KV_BOUND if kv_bf16 else {}))
        dec.close()


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_long_context_fused_step_matches_oracle(cuda, kv_bf16):
    """A cache of 1300 positions x 8 KV heads: the fused batch-1 step plans slices of 128 positions (8 stages of 16, one
    per warp) and attends through the tensor-core kernel for the f32 cache as well (operands split into two bf16 parts,
    about 2^-17 per product): the f32 tolerances of the other tests hold."""
    cfg = tiny(rt.FORMAT_W4G128, True, n_heads=8, n_kv_heads=8, head_dim=64, dim=512, max_seq_len=1300, kv_bf16=kv_bf16)
    dec = make(cfg)
    prompt = np.random.default_rng(21).integers(0, cfg.vocab_size, 1210)
    check_against_oracle(dec, cfg, prompt, 6, batched_prefill=True, **(BF16_KV_BOUND if kv_bf16 else {}))
    dec.close()


@pytest.mark.parametrize("kv_bf16", [False, True])
@pytest.mark.parametrize("batched_prefill", [False, True])
def test_single_token_prompt(cuda, kv_bf16, batched_prefill):
    """The shortest sequences: a one-token prompt (one query row, one key), then steps whose blocks hold only the row
    being written plus a handful of cached rows."""
    cfg = tiny(rt.FORMAT_RS_I8, True, n_heads=8, n_kv_heads=2, head_dim=128, dim=256, max_seq_len=40, kv_bf16=kv_bf16)
    dec = make(cfg)
    check_against_oracle(dec, cfg, np.asarray([7]), 6, batched_prefill=batched_prefill, **(BF16_KV_BOUND if kv_bf16 else {}))
    dec.close()


BF16_KV_BOUND = dict(hid_tol=2e-3, min_margin=1e-2, logit_tol=5e-3)


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
@pytest.mark.parametrize("head_dim,n_heads,n_kv", [(64, 4, 2), (128, 8, 1), (128, 8, 2)])
@pytest.mark.parametrize("batched_prefill", [False, True])
def test_bf16_kv_cache_matches_oracle(cuda, fmt, head_dim, n_heads, n_kv, batched_prefill):
    """kv_bf16: the oracle rounds the K / V rows it stores to bf16 (nearest-even) and is otherwise unchanged.  The bound
    is the option's own: a K / V value that the two sides compute a few f32 ulps apart can fall on either side of a bf16
    rounding tie, which moves that cache element by one bf16 ulp (2^-8 relative) - hidden state within 2e-3 of its scale,
    logits within 5e-3, tokens compared while the oracle's top-2 margin is at least 1e-2.  The sequence crosses a
    64-position tile so that staged rows, the row being written and both prefill paths are covered.  The cache bytes are
    half those of the f32 cache."""
    cfg = tiny(fmt, True, n_heads=n_heads, n_kv_heads=n_kv, head_dim=head_dim, dim=256, max_seq_len=160, kv_bf16=True)
    dec = make(cfg)
    ref = make(tiny(fmt, True, n_heads=n_heads, n_kv_heads=n_kv, head_dim=head_dim, dim=256, max_seq_len=160))
    assert dec.kv_bytes * 2 == ref.kv_bytes
    ref.close()
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab_size, 61)
    check_against_oracle(dec, cfg, prompt, 8, batched_prefill=batched_prefill, **BF16_KV_BOUND)
    dec.close()


@pytest.mark.parametrize("fused,rotary_dim", [(False, None), (True, 32), (False, 32)])
def test_bf16_kv_cache_on_the_other_step_forms(cuda, fused, rotary_dim):
    """The operator-by-operator step and the partial-rotary step (RoPE + cache write in a kernel of their own) over a
    bf16 cache."""
    cfg = tiny(rt.FORMAT_W4G128, fused, rotary_dim=rotary_dim, max_seq_len=96, kv_bf16=True)
    dec = make(cfg)
    prompt = np.random.default_rng(5).integers(0, cfg.vocab_size, 66)
    check_against_oracle(dec, cfg, prompt, 5, batched_prefill=fused, **BF16_KV_BOUND)
    dec.close()


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
def test_batched_prefill_matches_oracle_and_token_loop(cuda, fmt):
    cfg = tiny(fmt, True, n_heads=8, n_kv_heads=2, head_dim=128, dim=256, max_seq_len=64)
    dec = make(cfg)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, cfg.vocab_size, 21)
    check_against_oracle(dec, cfg, prompt, 5, batched_prefill=True)
    # batched prefill and the per-token path leave the same pending token and (nearly) the same hidden state
    dec.prefill(prompt)
    a_top, a_hid = dec.next_top(), dec.last_hidden()
    dec.prefill(prompt, token_loop=True)
    b_top, b_hid = dec.next_top(), dec.last_hidden()
    assert rt.unpack_top1(a_top)[0] == rt.unpack_top1(b_top)[0]
    assert np.max(np.abs(a_hid - b_hid)) <= 2e-4 * max(np.max(np.abs(b_hid)), 1.0)
    dec.close()


def test_fused_and_unfused_paths_agree(cuda):
    prompt = np.arange(1, 8)
    outs = []
    for fused in (True, False):
        cfg = tiny(rt.FORMAT_W4G128, fused)
        dec = make(cfg, seed=5)
        dec.prefill(prompt, token_loop=True)
        outs.append(dec.generate_greedy(10))
        dec.close()
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.max(np.abs(outs[0][1] - outs[1][1])) <= 1e-3


def test_step_host_equals_graph_loop_and_is_repeatable(cuda):
    cfg = tiny(rt.FORMAT_W4G128)
    dec = make(cfg, seed=7)
    prompt = np.array([5, 17, 300, 2])
    dec.prefill(prompt)
    tokens, logits = dec.generate_greedy(8)
    dec.prefill(prompt)
    packed = dec.next_top()
    via_host = []
    for _ in range(8):
        tok, logit = rt.unpack_top1(packed)
        via_host.append((tok, logit))
        packed = dec.step_host(tok)
    assert [t for t, _ in via_host] == tokens.tolist()
    assert np.array_equal(np.array([l for _, l in via_host], dtype=F), logits)
    # the decode loop is deterministic: a second run gives bit-identical logits
    dec.prefill(prompt)
    tokens2, logits2 = dec.generate_greedy(8)
    assert np.array_equal(tokens, tokens2) and np.array_equal(logits, logits2)
    dec.close()


def test_tied_embeddings_use_the_embedding_table_as_output(cuda):
    import oracle
    for fmt in (rt.FORMAT_RS_I8, rt.FORMAT_W4G128):
        cfg = tiny(fmt)
        dec = make(cfg, tie=True)
        emb = dec.get_tensor(-1, rt.T_EMBEDDING)
        values, scales = dec.get_tensor(-1, rt.T_OUTPUT)
        if fmt == rt.FORMAT_RS_I8:
            q, sc = oracle.rs_i8_quantize(emb)
            assert np.array_equal(values, q) and np.array_equal(scales, sc)
        else:
            p, gs = oracle.w4_quantize(oracle.bf16_to_f32(emb))
            assert np.array_equal(values, p) and np.array_equal(scales, gs)
        dec.close()


def test_runtime_errors(cuda):
    cfg = tiny(rt.FORMAT_W4G128, max_seq_len=8)
    dec = make(cfg)
    with pytest.raises(KmllError):
        dec.generate_greedy(1)  # runtime must be prefilled before generation
    with pytest.raises(KmllError):
        dec.prefill(np.arange(9))  # longer than max_seq_len
    with pytest.raises(KmllError):
        dec.prefill(np.array([cfg.vocab_size]))  # token out of range
    dec.prefill(np.arange(5))
    with pytest.raises(KmllError):
        dec.generate_greedy(4)  # position would exceed max sequence length
    dec.generate_greedy(3)
    dec.close()
    with pytest.raises(KmllError):
        rt.Decoder(tiny(rt.FORMAT_W4G128, n_heads=3))  # heads not divisible
    with pytest.raises(KmllError):
        rt.Decoder(tiny(rt.FORMAT_W4G128, dim=200))  # not a multiple of the group size


def test_qwen2_shape_slice(cuda):
    """Qwen2-0.5B geometry (hidden 896, 14/2 heads of 64, intermediate 4864, tied embeddings) with 2 layers and a
    small vocabulary: exercises K = 896 and 4864 (not multiples of the 2 KB stage) against the oracle."""
    cfg = rt.DecoderConfig(n_layers=2, dim=896, n_heads=14, n_kv_heads=2, head_dim=64, hidden_dim=4864, vocab_size=1024,
                           rope_theta=1e6, norm_eps=1e-6, max_seq_len=40, format=rt.FORMAT_W4G128)
    dec = make(cfg, seed=2, std=0.02, tie=True)
    rng = np.random.default_rng(2)
    check_against_oracle(dec, cfg, rng.integers(0, cfg.vocab_size, 12), 4, batched_prefill=True)
    dec.close()


def test_timeline_attach_and_detach_recapture_the_step_graph(cuda):
    """The per-token CUDA graph bakes the timeline slots of its launches: after the buffer is detached the decoder must
    capture the graph again, so replays leave the (possibly freed) buffer alone; attaching later must trace again."""
    import ctypes as C
    from kmll_b200 import lib as klib
    L = klib.load()
    cfg = tiny(rt.FORMAT_W4G128)
    dec = make(cfg, seed=7)
    prompt = np.array([5, 17, 300, 2])
    dec.prefill(prompt)
    ref_tokens, _ = dec.generate_greedy(6)  # graph captured with no buffer attached
    buf = torch.zeros(1 << 16, dtype=torch.int64, device="cuda")
    count = C.c_int(0)
    klib.check(L.kmll_trace_attach(C.c_void_p(buf.data_ptr()), buf.numel() * 8))
    dec.prefill(prompt)
    tokens, _ = dec.generate_greedy(6)
    torch.cuda.synchronize()
    klib.check(L.kmll_trace_launches(None, None, None, 0, C.byref(count)))
    assert count.value > 0 and int(torch.count_nonzero(buf)) > 0, "attaching after the first capture must trace the step"
    assert tokens.tolist() == ref_tokens.tolist()
    klib.check(L.kmll_trace_attach(None, 0))
    buf.zero_()
    dec.prefill(prompt)
    tokens, _ = dec.generate_greedy(6)
    torch.cuda.synchronize()
    assert int(torch.count_nonzero(buf)) == 0, "a detached buffer must not be written by later replays"
    assert tokens.tolist() == ref_tokens.tolist()
    dec.close()


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
def test_archive_round_trip_gives_the_same_model(cuda, fmt, tmp_path):
    """Export a decoder's linear tensors in kmll's archive layout, load them into a fresh decoder (norms and embeddings
    travel separately, as in kmll where they stay in the checkpoint): the tensors are bit-identical and the greedy
    tokens equal the in-memory model's."""
    cfg = tiny(fmt)
    dec = make(cfg, seed=11)
    prompt = np.array([7, 300, 12, 5, 99])
    dec.prefill(prompt)
    ref_tokens, ref_logits = dec.generate_greedy(8)
    d = str(tmp_path / "export")
    dec.export_archive(d, "/models/demo.safetensors")
    fresh = rt.Decoder(cfg)
    for layer in range(cfg.n_layers):
        fresh.set_tensor(layer, rt.T_ATTENTION_NORM, dec.get_tensor(layer, rt.T_ATTENTION_NORM))
        fresh.set_tensor(layer, rt.T_FFN_NORM, dec.get_tensor(layer, rt.T_FFN_NORM))
    fresh.set_tensor(-1, rt.T_FINAL_NORM, dec.get_tensor(-1, rt.T_FINAL_NORM))
    fresh.set_tensor(-1, rt.T_EMBEDDING, dec.get_tensor(-1, rt.T_EMBEDDING))
    fresh.load_archive(d, "/models/demo.safetensors")
    for layer, tensor in ((0, rt.T_WQ), (1, rt.T_W2), (-1, rt.T_OUTPUT)):
        a, b = dec.get_tensor(layer, tensor), fresh.get_tensor(layer, tensor)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint8), b[1].view(np.uint8))
    fresh.prefill(prompt)
    tokens, logits = fresh.generate_greedy(8)
    assert np.array_equal(tokens, ref_tokens) and np.array_equal(logits, ref_logits)
    with pytest.raises(KmllError):
        fresh.load_archive(d, "/models/another.safetensors")
    dec.close()
    fresh.close()
