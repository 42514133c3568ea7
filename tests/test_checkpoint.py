"""Checkpoint reading as kmll does it (crates/inference/src/safetensors.rs, TextConfig::from_config_json and the rope
frequencies of crates/inference/src/model.rs): file layout, shards, tensor-name aliases, config parsing, YaRN."""
import json
import os

import numpy as np
import pytest

import oracle
from kmll_b200.checkpoint import (CheckpointError, ModelWeights, SafetensorsFile, TextConfig, model_tensor_aliases, rope_frequencies,
                                  rotary_dim_from_partial_factor, write_safetensors)


def test_safetensors_round_trip_and_ranges(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"a.weight": rng.integers(0, 65536, (5, 7)).astype(np.uint16), "b": rng.normal(0, 1, (3,)).astype(np.float32),
               "c": rng.integers(-128, 128, (2, 3, 4)).astype(np.int8)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors, {"format": "pt"})
    f = SafetensorsFile(path)
    assert f.data_start == 8 + f.header_len and f.header_len % 8 == 0
    assert sorted(t.name for t in f.tensors) == ["a.weight", "b", "c"]
    for name, arr in tensors.items():
        info = f.tensor_opt(name)
        assert info.shape == arr.shape and info.dtype == {"a.weight": "BF16", "b": "F32", "c": "I8"}[name]
        assert np.array_equal(f.read_tensor(info), arr)
    assert np.array_equal(f.read_tensor_range(f.tensor_opt("a.weight"), 9, 11), tensors["a.weight"].reshape(-1)[9:20])
    with pytest.raises(CheckpointError):
        f.read_tensor_range(f.tensor_opt("b"), 2, 2)
    # a header whose offsets do not match the shape is refused
    raw = bytearray(open(path, "rb").read())
    bad = raw.replace(b'"shape":[3]', b'"shape":[4]')
    bad_path = str(tmp_path / "bad.safetensors")
    open(bad_path, "wb").write(bad)
    with pytest.raises(CheckpointError):
        SafetensorsFile(bad_path)


def test_aliases_follow_kmll():
    assert model_tensor_aliases("tok_embeddings.weight") == ["language_model.model.embed_tokens.weight", "model.embed_tokens.weight",
                                                             "model.language_model.embed_tokens.weight"]
    assert model_tensor_aliases("output.weight") == ["language_model.lm_head.weight", "lm_head.weight"]
    assert model_tensor_aliases("layers.17.feed_forward.w3.weight") == ["language_model.model.layers.17.mlp.up_proj.weight",
                                                                         "model.layers.17.mlp.up_proj.weight",
                                                                         "model.language_model.layers.17.mlp.up_proj.weight"]
    assert model_tensor_aliases("layers.3.attention.k_norm.weight")[1] == "model.layers.3.self_attn.k_norm.weight"
    assert model_tensor_aliases("layers.3.unknown.weight") == [] and model_tensor_aliases("something") == []


def test_sharded_directory_and_alias_lookup(tmp_path):
    a = {"model.embed_tokens.weight": np.arange(12, dtype=np.uint16).reshape(3, 4)}
    b = {"model.layers.0.self_attn.q_proj.weight": np.arange(8, dtype=np.uint16).reshape(2, 4), "model.norm.weight": np.ones(4, dtype=np.uint16)}
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), a)
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    index = {"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in a}, **{k: "model-00002-of-00002.safetensors" for k in b}}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    w = ModelWeights(str(tmp_path))
    assert w.source_path.endswith("index.json") and len(w.files) == 2
    assert np.array_equal(w.read("tok_embeddings.weight", "BF16", (3, 4)), a["model.embed_tokens.weight"])
    assert np.array_equal(w.read("layers.0.attention.wq.weight"), b["model.layers.0.self_attn.q_proj.weight"])
    assert w.tensor_opt("output.weight") is None
    with pytest.raises(CheckpointError):
        w.read("layers.0.attention.wk.weight")
    with pytest.raises(CheckpointError):
        w.read("norm.weight", "F32")
    # a single file is found as consolidated.safetensors first, then model.safetensors
    single = tmp_path / "single"
    single.mkdir()
    write_safetensors(str(single / "model.safetensors"), a)
    assert ModelWeights(str(single)).source_path.endswith("model.safetensors")
    write_safetensors(str(single / "consolidated.safetensors"), b)
    assert ModelWeights(str(single)).source_path.endswith("consolidated.safetensors")


BASE = {"hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "max_position_embeddings": 4096, "vocab_size": 640, "rms_norm_eps": 1e-5}


def test_config_json():
    c = TextConfig.from_config_json(json.dumps({**BASE, "rope_theta": 1e6, "eos_token_id": 2}))
    assert (c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.head_dim, c.rotary_dim) == (256, 512, 2, 4, 2, 64, 64)
    assert c.rope_theta == 1e6 and c.rope_yarn is None and c.eos_token_id == 2 and c.norm_eps == 1e-5
    # defaults and the nested text_config / rope_parameters forms
    assert TextConfig.from_config_json(json.dumps(BASE)).rope_theta == 10000.0
    nested = {"model_type": "mistral3", "eos_token_id": 7,
              "text_config": {**BASE, "rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6, "factor": 16.0, "original_max_position_embeddings": 16384,
                                                          "beta_fast": 32.0, "beta_slow": 1.0, "partial_rotary_factor": 0.5}}}
    c = TextConfig.from_config_json(json.dumps(nested))
    assert c.rotary_dim == 32 and c.rope_theta == 1e6 and c.eos_token_id == 7
    assert c.rope_yarn.factor == 16.0 and c.rope_yarn.original_max_position_embeddings == 16384 and c.rope_yarn.attention_factor == 1.0
    for broken in ({k: v for k, v in BASE.items() if k != "head_dim"}, {**BASE, "num_key_value_heads": 3}, {**BASE, "partial_rotary_factor": 0.3},
                   {**BASE, "model_type": "qwen3_5_text"},
                   {**BASE, "rope_parameters": {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 4096, "beta_fast": 32.0,
                                                "beta_slow": 1.0, "mscale": 1.3}}):
        with pytest.raises(CheckpointError):
            TextConfig.from_config_json(json.dumps(broken))
    assert rotary_dim_from_partial_factor(128, 1.0) == 128 and rotary_dim_from_partial_factor(128, 0.25) == 32
    # `sliding_window` is read but not applied unless the caller asks for it (kmll runs full causal attention)
    assert TextConfig.from_config_json(json.dumps(BASE)).sliding_window is None
    assert TextConfig.from_config_json(json.dumps({**BASE, "sliding_window": 4096})).sliding_window == 4096
    assert TextConfig.from_config_json(json.dumps({**BASE, "sliding_window": None})).sliding_window is None
    assert TextConfig.from_config_json(json.dumps({"text_config": {**BASE, "sliding_window": 128}})).sliding_window == 128


def test_rope_frequencies_match_the_oracle():
    plain = TextConfig.from_config_json(json.dumps({**BASE, "rope_theta": 1e6, "head_dim": 128, "hidden_size": 512}))
    assert np.array_equal(rope_frequencies(plain), oracle.rope_frequencies(1e6, 128))
    yarn = TextConfig.from_config_json(json.dumps({**BASE, "head_dim": 128, "hidden_size": 512,
                                                   "rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6, "factor": 16.0,
                                                                       "original_max_position_embeddings": 16384, "beta_fast": 32.0, "beta_slow": 1.0}}))
    got = rope_frequencies(yarn)
    ref = oracle.rope_frequencies_yarn(1e6, 128, 16.0, 32.0, 1.0, 16384)
    assert got.shape == ref.shape == (64,)
    assert np.allclose(got, ref, rtol=2e-6, atol=0.0)  # powf / logf may differ by an ulp between libm and numpy
    assert got[0] == 1.0 and got[-1] < ref[0] / 16.0  # high frequencies are kept, low ones are interpolated
