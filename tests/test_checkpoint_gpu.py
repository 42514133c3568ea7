"""A checkpoint directory (config.json + sharded safetensors in the naming checkpoints use) loaded into the quantized
decoder: the device tensors are the oracle's quantization of the stored bf16 values, and decoding with YaRN-scaled
rotation frequencies agrees with the CPU oracle model."""
import json

import numpy as np
import pytest

import oracle
from kmll_b200 import runtime as rt
from kmll_b200.checkpoint import CheckpointError, load_decoder, rope_frequencies, write_safetensors
from oracle_model import OracleDecoder

pytestmark = pytest.mark.gpu
F = np.float32


def make_checkpoint(tmp_path, yarn=True, tied=False, with_qk_norm=False, sliding_window=None):
    cfg = {"model_type": "mistral3", "text_config": {
        **({"sliding_window": sliding_window} if sliding_window else {}),
        "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "max_position_embeddings": 4096, "vocab_size": 640, "rms_norm_eps": 1e-5, "eos_token_id": 2,
        "rope_parameters": ({"rope_type": "yarn", "rope_theta": 1e6, "factor": 16.0, "original_max_position_embeddings": 64, "beta_fast": 32.0,
                             "beta_slow": 1.0} if yarn else {"rope_type": "default", "rope_theta": 1e6})}}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    rng = np.random.default_rng(4)

    def bf16(*shape, std=0.05, mean=0.0):
        return oracle.bf16_from_f32((rng.normal(mean, std, shape)).astype(F)).reshape(shape)

    t = {"model.embed_tokens.weight": bf16(640, 256), "model.norm.weight": bf16(256, std=0.1, mean=1.0)}
    if not tied:
        t["lm_head.weight"] = bf16(640, 256)
    for l in range(2):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"] = bf16(256, std=0.1, mean=1.0)
        t[p + "post_attention_layernorm.weight"] = bf16(256, std=0.1, mean=1.0)
        t[p + "self_attn.q_proj.weight"] = bf16(256, 256)
        t[p + "self_attn.k_proj.weight"] = bf16(128, 256)
        t[p + "self_attn.v_proj.weight"] = bf16(128, 256)
        t[p + "self_attn.o_proj.weight"] = bf16(256, 256)
        t[p + "mlp.gate_proj.weight"] = bf16(512, 256)
        t[p + "mlp.up_proj.weight"] = bf16(512, 256)
        t[p + "mlp.down_proj.weight"] = bf16(256, 512)
        if with_qk_norm:
            t[p + "self_attn.q_norm.weight"] = bf16(64, std=0.1, mean=1.0)
            if with_qk_norm != "q only":
                t[p + "self_attn.k_norm.weight"] = bf16(64, std=0.1, mean=1.0)
    names = list(t)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for shard, keys in shards.items():
        write_safetensors(str(tmp_path / shard), {k: t[k] for k in keys})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {k: s for s, keys in shards.items() for k in keys}}))
    return t


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
def test_load_checkpoint_quantizes_like_the_oracle_and_decodes_with_yarn(cuda, tmp_path, fmt):
    t = make_checkpoint(tmp_path)
    dec, cfg = load_decoder(str(tmp_path), fmt, max_seq_len=96)
    assert cfg.rope_yarn is not None and cfg.eos_token_id == 2 and dec.cfg.max_seq_len == 96
    # the tensors on the device are the oracle's quantization of the checkpoint's values
    for layer, tid, name in ((1, rt.T_WQ, "model.layers.1.self_attn.q_proj.weight"), (0, rt.T_W2, "model.layers.0.mlp.down_proj.weight"),
                             (-1, rt.T_OUTPUT, "lm_head.weight"), (0, rt.T_W3, "model.layers.0.mlp.up_proj.weight")):
        values, scales = dec.get_tensor(layer, tid)
        if fmt == rt.FORMAT_RS_I8:
            q, sc = oracle.rs_i8_quantize(t[name])
        else:
            q, sc = oracle.w4_quantize(oracle.bf16_to_f32(t[name]).reshape(t[name].shape))
        assert np.array_equal(values, q) and np.array_equal(np.asarray(scales).view(sc.dtype), sc)
    assert np.array_equal(dec.get_tensor(-1, rt.T_EMBEDDING), t["model.embed_tokens.weight"])
    assert np.array_equal(dec.get_tensor(1, rt.T_FFN_NORM), t["model.layers.1.post_attention_layernorm.weight"])
    # decoding beyond the original context of the YaRN config: the oracle model with the same frequency table agrees
    freqs = rope_frequencies(cfg)
    assert not np.array_equal(freqs, oracle.rope_frequencies(1e6, 64))
    ora = OracleDecoder(dec.cfg, dec, freqs=freqs)
    prompt = np.random.default_rng(5).integers(0, 640, 70)
    logits = ora.prefill(prompt)
    dec.prefill(prompt)
    steps, _ = ora.generate_greedy(logits, 6)
    tokens, glogits = dec.generate_greedy(6)
    for i, (tok, logit, margin) in enumerate(steps):
        if margin < 1e-3:
            break
        assert int(tokens[i]) == tok and abs(float(glogits[i]) - logit) <= 1e-3 * max(abs(logit), 1.0)
    dec.close()


def test_tied_embeddings_and_refusals(cuda, tmp_path):
    a = tmp_path / "tied"
    a.mkdir()
    t = make_checkpoint(a, yarn=False, tied=True)
    dec, cfg = load_decoder(str(a), rt.FORMAT_RS_I8, max_seq_len=32)
    q, sc = oracle.rs_i8_quantize(t["model.embed_tokens.weight"])
    values, scales = dec.get_tensor(-1, rt.T_OUTPUT)
    assert np.array_equal(values, q) and np.array_equal(scales, sc) and cfg.rope_yarn is None
    with pytest.raises(rt.KmllError):
        dec.set_rope_freqs(np.ones(7, dtype=F))  # rotary_dim / 2 = 32 values are wanted
    dec.close()
    b = tmp_path / "qk"
    b.mkdir()
    make_checkpoint(b, with_qk_norm="q only")
    with pytest.raises(CheckpointError):
        load_decoder(str(b), rt.FORMAT_W4G128, max_seq_len=32)


@pytest.mark.parametrize("fmt,fused", [(rt.FORMAT_W4G128, True), (rt.FORMAT_RS_I8, True), (rt.FORMAT_W4G128, False)])
def test_checkpoint_with_qk_norm_decodes_like_the_oracle(cuda, tmp_path, fmt, fused):
    """Per-head RMSNorm of the query and key rows before RoPE (Qwen3-style checkpoints): batched prefill, the graph step
    (fused and kmll's operator order) and the lockstep batch all agree with the oracle model."""
    t = make_checkpoint(tmp_path, yarn=False, with_qk_norm=True)
    dec, cfg = load_decoder(str(tmp_path), fmt, max_seq_len=64, fused=fused)
    assert np.array_equal(dec.get_tensor(1, rt.T_K_NORM), t["model.layers.1.self_attn.k_norm.weight"])
    ora = OracleDecoder(dec.cfg, dec)
    assert ora.qk_norm[0] is not None
    prompt = np.random.default_rng(6).integers(0, 640, 11)
    logits = ora.prefill(prompt)
    dec.prefill(prompt)
    hid = dec.last_hidden()
    assert np.max(np.abs(hid - ora.hidden)) <= 2e-4 * max(float(np.max(np.abs(ora.hidden))), 1.0)
    steps, _ = ora.generate_greedy(logits, 6)
    tokens, glogits = dec.generate_greedy(6)
    for i, (tok, logit, margin) in enumerate(steps):
        if margin < 1e-3:
            break
        assert int(tokens[i]) == tok and abs(float(glogits[i]) - logit) <= 1e-3 * max(abs(logit), 1.0)
    if fused:  # the lockstep batch takes the same tokens
        dec.prefill(prompt)
        bd = rt.BatchDecoder(dec, 3)
        for slot in range(3):
            bd.adopt(slot)
        btok, _ = bd.generate_greedy(6)
        assert all(btok[slot].tolist() == [int(v) for v in tokens] for slot in range(3))
        bd.close()
    dec.close()


def test_sliding_window_and_bf16_cache_from_a_checkpoint(cuda, tmp_path):
    """The checkpoint's own `sliding_window` is applied only on request ("config"); with it and the bf16 KV cache the decoder
    still follows the oracle model given the same two options."""
    make_checkpoint(tmp_path, yarn=False, sliding_window=24)
    dec, cfg = load_decoder(str(tmp_path), rt.FORMAT_W4G128, max_seq_len=96)
    assert cfg.sliding_window == 24 and dec.cfg.sliding_window == 0 and not dec.cfg.kv_bf16
    dec.close()
    dec, cfg = load_decoder(str(tmp_path), rt.FORMAT_W4G128, max_seq_len=96, sliding_window="config", kv_bf16=True)
    assert dec.cfg.sliding_window == 24 and dec.cfg.kv_bf16
    ora = OracleDecoder(dec.cfg, dec)
    prompt = np.random.default_rng(8).integers(0, 640, 70)
    logits = ora.prefill(prompt)
    dec.prefill(prompt)
    hid = dec.last_hidden()
    assert np.max(np.abs(hid - ora.hidden)) <= 2e-3 * max(float(np.max(np.abs(ora.hidden))), 1.0)
    steps, _ = ora.generate_greedy(logits, 6)
    tokens, glogits = dec.generate_greedy(6)
    for i, (tok, logit, margin) in enumerate(steps):
        if margin < 1e-2:
            break
        assert int(tokens[i]) == tok and abs(float(glogits[i]) - logit) <= 5e-3 * max(abs(logit), 1.0)
    dec.close()
