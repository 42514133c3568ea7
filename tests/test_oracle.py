"""CPU tests: the C oracle against the committed known-answer vectors (tests/golden/kat.npz, made by
an independent numpy restatement) and against the literal KATs of the reference's own unit tests."""
import numpy as np

import oracle

F = np.float32


def test_lcg_matches_reference_generator(golden):
    g = oracle.Lcg(0x1234)
    got = np.array([g.next() for _ in range(8)], dtype=F)
    assert np.array_equal(got.view(np.uint32), golden["lcg_seed_0x1234_first8"].view(np.uint32))
    assert np.all(np.abs(got) <= 1.0)


def test_bf16_roundtrip_and_rounding():
    # Bf16::from_f32 rounds to nearest even on the dropped 16 bits (dtypes.rs:153-157)
    vals = np.array([1.0, 1.00390625, 1.01171875, -2.5, 0.0, 3.0e38, 1e-40], dtype=F)
    bits = oracle.bf16_from_f32(vals)
    import torch
    ref = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, ref)
    assert np.array_equal(oracle.bf16_to_f32(bits).view(np.uint32), bits.astype(np.uint32) << 16)


def test_f16_conversion_matches_ieee():
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-5, 2000), rng.normal(0, 3e4, 500),
                           [0.0, 65504.0, 65519.9, 65520.0, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5]]).astype(F)
    got = np.array([oracle.f16_from_f32_scalar(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, vals.astype(np.float16).view(np.uint16))
    back = np.array([oracle.f16_to_f32_scalar(int(b)) for b in got], dtype=F)
    assert np.array_equal(back, got.view(np.float16).astype(F))


def test_rope_known_answer(golden):
    # crates/inference/src/model.rs:12227-12249, tolerance 1e-6 as in the reference test
    out = oracle.apply_rope(golden["rope_kat_input"], golden["rope_kat_freqs"], 1, 6)
    assert np.max(np.abs(out - golden["rope_kat_expected"])) < 1e-6
    assert out[4] == 9.0 and out[5] == 10.0


def test_rope_frequencies_known_answer(golden):
    # crates/inference/src/model.rs:12216-12225
    freqs = oracle.rope_frequencies(10000.0, 64)
    assert freqs.size == 32
    assert abs(freqs[0] - 1.0) < 1e-6
    assert abs(freqs[1] - golden["rope_freq_kat"][1]) < 1e-6


def test_rs_i8_quantize_and_linear_match_golden(golden):
    for idx in range(8):
        m, n, k = golden[f"gemm_i8_{idx}_shape"]
        q, sc = oracle.rs_i8_quantize(golden[f"gemm_i8_{idx}_wbits"])
        assert np.array_equal(q, golden[f"gemm_i8_{idx}_q"]), idx
        assert np.array_equal(sc.view(np.uint32), golden[f"gemm_i8_{idx}_scales"].view(np.uint32)), idx
        y = oracle.rs_i8_linear_batched(golden[f"gemm_i8_{idx}_x"], q, sc)
        assert np.array_equal(y.view(np.uint32), golden[f"gemm_i8_{idx}_y"].view(np.uint32)), idx
        # matvec_cpu (rowwise_scaled.rs:108-126) gives the same bits row by row
        y0 = oracle.rs_i8_matvec(q, sc, golden[f"gemm_i8_{idx}_x"][0])
        assert np.array_equal(y0.view(np.uint32), golden[f"gemm_i8_{idx}_y"][0].view(np.uint32))
        # dequant = scaled_value
        assert np.array_equal(oracle.rs_i8_dequant(q, sc), q.astype(F) * sc[:, None])


def test_rs_i8_stress_inputs_replay_from_seed(golden):
    # the golden inputs themselves come from the reference's LCG and seeds (src/main.rs:482,613-621)
    for idx in range(8):
        m, n, k = golden[f"gemm_i8_{idx}_shape"]
        g = oracle.Lcg(((0 << 32) ^ idx ^ 0x9E3779B97F4A7C15) ^ 0x89)
        x = g.fill_f32(m * k).reshape(m, k)
        wb = g.fill_bf16(n * k).reshape(n, k)
        assert np.array_equal(x, golden[f"gemm_i8_{idx}_x"])
        assert np.array_equal(wb, golden[f"gemm_i8_{idx}_wbits"])


def test_top1_i8_matches_golden_and_forced_row(golden):
    for idx in range(6):
        rows, cols = golden[f"top1_i8_{idx}_shape"]
        q, sc = oracle.rs_i8_quantize(golden[f"top1_i8_{idx}_wbits"])
        logits = oracle.rs_i8_matvec(q, sc, golden[f"top1_i8_{idx}_x"])
        token, logit = oracle.unpack_top1(oracle.top1_packed(logits))
        exp_token, exp_bits = golden[f"top1_i8_{idx}_expected"]
        assert token == int(exp_token)
        assert np.array([logit], dtype=F).view(np.uint32)[0] == int(exp_bits)
        assert token == (0 if rows == 1 else rows // 3)  # the planted +-4.0 row wins (src/main.rs:4145-4150)


def test_argmax_tie_prefers_lower_index(golden):
    # src/main.rs:4024-4054: forced logit at len/3 and len-1, lower index must win
    for idx in range(8):
        logits = golden[f"argmax_{idx}_logits"]
        token, logit = oracle.unpack_top1(oracle.top1_packed(logits))
        assert token == int(golden[f"argmax_{idx}_expected"][0])
        assert logit == 12345.0


def test_top_k_is_stable_descending():
    logits = np.array([0.5, 2.0, -1.0, 2.0, 0.5, -0.0, 0.0], dtype=F)
    tokens, values = oracle.top_k(logits, 5)
    assert tokens.tolist() == [1, 3, 0, 4, 6]  # total_cmp: +0.0 > -0.0; ties keep the lower index first
    assert values.tolist() == [2.0, 2.0, 0.5, 0.5, 0.0]


def test_w4_matches_golden(golden):
    packed, gs = oracle.w4_quantize(golden["w4_w"])
    assert np.array_equal(packed, golden["w4_packed"])
    assert np.array_equal(gs, golden["w4_gscales"])
    deq = oracle.w4_dequant(packed, gs)
    assert np.array_equal(deq.view(np.uint32), golden["w4_dequant"].view(np.uint32))
    y = oracle.w4_matvec(packed, gs, golden["w4_x"])
    assert np.array_equal(y.view(np.uint32), golden["w4_y"].view(np.uint32))
    # nibble 0 is never produced; an all-zero group gets scale 1.0 and nibble 8
    assert (packed & 0xF).min() >= 1 and (packed >> 4).min() >= 1
    assert gs[3, 1] == np.array([1.0], dtype=np.float16).view(np.uint16)[0]
    assert np.all(packed[3, 64:128] == 0x88)


def test_rmsnorm_add_silu_follow_reference_formulas():
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, 257).astype(F)
    w = oracle.bf16_from_f32(rng.uniform(0.5, 1.5, 257).astype(F))
    y = oracle.rmsnorm(x, w, 1e-6)
    ss = F(0)
    for v in x:
        ss = F(ss + F(v * v))
    inv = F(1.0) / np.sqrt(F(ss / F(257) + F(1e-6)), dtype=F)
    ref = (x * inv).astype(F) * oracle.bf16_to_f32(w)
    assert np.array_equal(y.view(np.uint32), ref.astype(F).view(np.uint32))
    g = rng.normal(0, 2, 100).astype(F)
    u = rng.normal(0, 2, 100).astype(F)
    s = oracle.silu_mul(g, u)
    assert np.allclose(s, g / (1 + np.exp(-g.astype(np.float64))) * u, rtol=1e-6, atol=1e-7)
    assert np.array_equal(oracle.add(g, u), g + u)


def test_attention_composition_and_softmax_rows():
    rng = np.random.default_rng(2)
    n_heads, n_kv, hd, seq, max_seq = 4, 2, 8, 5, 7
    q = rng.normal(0, 1, n_heads * hd).astype(F)
    kc = rng.normal(0, 1, (max_seq, n_kv, hd)).astype(F)
    vc = rng.normal(0, 1, (max_seq, n_kv, hd)).astype(F)
    sc = oracle.attention_scores(q, kc, seq, max_seq, n_heads, n_kv, hd)
    out = oracle.softmax_value(sc, vc, seq, max_seq, n_heads, n_kv, hd)
    # float64 restatement
    ref = np.zeros(n_heads * hd)
    for h in range(n_heads):
        kvh = h // (n_heads // n_kv)
        s = (kc[:seq, kvh].astype(np.float64) @ q[h * hd:(h + 1) * hd].astype(np.float64)) / np.sqrt(hd)
        p = np.exp(s - s.max())
        ref[h * hd:(h + 1) * hd] = (p / p.sum()) @ vc[:seq, kvh].astype(np.float64)
    assert np.allclose(out, ref, atol=1e-6)
    assert np.allclose(oracle.single_query_attention(q, kc, vc, seq, n_heads, n_kv, hd), out, atol=1e-7)
    x = rng.normal(0, 3, (6, 33)).astype(F)
    sm = oracle.softmax_rows(x)
    assert np.allclose(sm.sum(axis=1), 1.0, atol=1e-6)
    e = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    assert np.allclose(sm, e / e.sum(axis=1, keepdims=True), atol=1e-7)


def test_oracle_is_thread_count_invariant():
    rng = np.random.default_rng(3)
    wb = oracle.bf16_from_f32(rng.normal(0, 0.02, (64, 256)).astype(F))
    x = rng.normal(0, 1, 256).astype(F)
    q, sc = oracle.rs_i8_quantize(wb)
    n = oracle.max_threads()
    y_mt = oracle.rs_i8_matvec(q, sc, x)
    oracle.set_threads(1)
    y_1 = oracle.rs_i8_matvec(q, sc, x)
    oracle.set_threads(n)
    assert np.array_equal(y_mt.view(np.uint32), y_1.view(np.uint32))
