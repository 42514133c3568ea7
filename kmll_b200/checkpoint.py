"""Checkpoints as kmll reads them: safetensors files (one file or a sharded directory with an index), kmll's tensor-name
aliases, `config.json`, RoPE frequencies incl. YaRN - and the load of such a directory into a quantized Decoder.

Follows crates/inference/src/safetensors.rs (file layout :56-163, model directory :184-284, shards :286-379, aliases
:436-488) and crates/inference/src/model.rs (TextConfig::from_config_json :271-366, rope frequencies :9239-9306).
Host-side I/O only; the weights are quantized on the device by the library's own quantizers."""
from __future__ import annotations

import json
import math
import os
import struct
from dataclasses import dataclass

import numpy as np

_DTYPES = {"BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4), "I8": (np.int8, 1), "U8": (np.uint8, 1),
           "I32": (np.int32, 4), "I64": (np.int64, 8), "F64": (np.float64, 8)}


class CheckpointError(ValueError):
    pass


@dataclass
class TensorInfo:
    """safetensors.rs:14-48."""
    name: str
    dtype: str
    shape: tuple
    data_offsets: tuple

    def element_count(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

    def byte_len(self) -> int:
        return self.data_offsets[1] - self.data_offsets[0]


class SafetensorsFile:
    """8-byte little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then the tensor bytes
    (safetensors.rs:56-163).  Tensors are read on demand; BF16 comes back as its uint16 bit patterns."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            raw = f.read(8)
            if len(raw) != 8:
                raise CheckpointError(f"{path}: too short for a safetensors header")
            self.header_len = struct.unpack("<Q", raw)[0]
            size = os.path.getsize(path)
            if self.header_len > size - 8:
                raise CheckpointError(f"{path}: header length {self.header_len} exceeds the file")
            header = json.loads(f.read(self.header_len).decode("utf-8"))
        self.data_start = 8 + self.header_len
        self.tensors: list[TensorInfo] = []
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            begin, end = (int(v) for v in entry["data_offsets"])
            info = TensorInfo(name, entry["dtype"], tuple(int(d) for d in entry["shape"]), (begin, end))
            if info.dtype not in _DTYPES:
                raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {info.dtype}")
            if end < begin or self.data_start + end > size or info.byte_len() != info.element_count() * _DTYPES[info.dtype][1]:
                raise CheckpointError(f"{path}: tensor {name} has inconsistent offsets {begin}..{end} for shape {info.shape}")
            self.tensors.append(info)
        self._by_name = {t.name: t for t in self.tensors}

    def tensor_opt(self, name: str):
        """The tensor of that name, or of one of its aliases (resolve_file_tensor, safetensors.rs:381-391)."""
        if name in self._by_name:
            return self._by_name[name]
        for alias in model_tensor_aliases(name):
            if alias in self._by_name:
                return self._by_name[alias]
        return None

    def read_tensor(self, info: TensorInfo) -> np.ndarray:
        return self.read_tensor_range(info, 0, info.element_count()).reshape(info.shape)

    def read_tensor_range(self, info: TensorInfo, element_start: int, element_count: int) -> np.ndarray:
        """read_tensor_range (safetensors.rs:121-149): a contiguous run of elements."""
        dt, size = _DTYPES[info.dtype]
        if element_start < 0 or element_count < 0 or element_start + element_count > info.element_count():
            raise CheckpointError(f"{info.name}: range {element_start}+{element_count} outside {info.element_count()} elements")
        with open(self.path, "rb") as f:
            f.seek(self.data_start + info.data_offsets[0] + element_start * size)
            data = f.read(element_count * size)
        if len(data) != element_count * size:
            raise CheckpointError(f"{info.name}: file ends inside the tensor")
        return np.frombuffer(data, dtype=dt).copy()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Writer of the same layout (tests, exporting random-init models).  uint16 arrays are stored as BF16."""
    names = {np.dtype(np.uint16): "BF16", np.dtype(np.float16): "F16", np.dtype(np.float32): "F32", np.dtype(np.int8): "I8",
             np.dtype(np.uint8): "U8", np.dtype(np.int32): "I32", np.dtype(np.int64): "I64", np.dtype(np.float64): "F64"}
    header, blobs, offset = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        if arr.dtype not in names:
            raise CheckpointError(f"{name}: dtype {arr.dtype} cannot be stored")
        blob = arr.tobytes()
        header[name] = {"dtype": names[arr.dtype], "shape": list(arr.shape), "data_offsets": [offset, offset + len(blob)]}
        blobs.append(blob)
        offset += len(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for blob in blobs:
            f.write(blob)


def model_tensor_aliases(name: str) -> list[str]:
    """kmll's internal names -> the names checkpoints use (safetensors.rs:440-488), in kmll's order of preference."""
    top = {"tok_embeddings.weight": ["language_model.model.embed_tokens.weight", "model.embed_tokens.weight", "model.language_model.embed_tokens.weight"],
           "norm.weight": ["language_model.model.norm.weight", "model.norm.weight", "model.language_model.norm.weight"],
           "output.weight": ["language_model.lm_head.weight", "lm_head.weight"]}
    if name in top:
        return list(top[name])
    if not name.startswith("layers."):
        return []
    rest = name[len("layers."):]
    if "." not in rest:
        return []
    layer, suffix = rest.split(".", 1)
    hf = {"attention_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
          "attention.wq.weight": "self_attn.q_proj.weight", "attention.wk.weight": "self_attn.k_proj.weight",
          "attention.wv.weight": "self_attn.v_proj.weight", "attention.wo.weight": "self_attn.o_proj.weight",
          "attention.q_norm.weight": "self_attn.q_norm.weight", "attention.k_norm.weight": "self_attn.k_norm.weight",
          "feed_forward.w1.weight": "mlp.gate_proj.weight", "feed_forward.w2.weight": "mlp.down_proj.weight",
          "feed_forward.w3.weight": "mlp.up_proj.weight"}.get(suffix)
    if hf is None:
        return []
    return [f"language_model.model.layers.{layer}.{hf}", f"model.layers.{layer}.{hf}", f"model.language_model.layers.{layer}.{hf}"]


class ModelWeights:
    """A model directory: `model.safetensors.index.json` + shards, else `consolidated.safetensors`, else
    `model.safetensors` (ModelWeights::open_model_dir, safetensors.rs:190-218)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        self.files: list[SafetensorsFile] = []
        self._file_of: dict[str, int] = {}
        if os.path.exists(index_path):
            with open(index_path) as f:
                weight_map = json.load(f).get("weight_map")
            if not isinstance(weight_map, dict) or not weight_map:
                raise CheckpointError(f"{index_path}: no weight_map")
            shard_names: list[str] = []
            for tensor, shard in weight_map.items():
                if shard not in shard_names:
                    shard_names.append(shard)
            self.files = [SafetensorsFile(os.path.join(model_dir, s)) for s in shard_names]
            for tensor, shard in weight_map.items():
                fi = shard_names.index(shard)
                if tensor not in self.files[fi]._by_name:
                    raise CheckpointError(f"{index_path}: tensor {tensor} is not in {shard}")
                self._file_of[tensor] = fi
            self.source_path = index_path
        else:
            path = os.path.join(model_dir, "consolidated.safetensors")
            if not os.path.exists(path):
                path = os.path.join(model_dir, "model.safetensors")
            self.files = [SafetensorsFile(path)]
            self._file_of = {t.name: 0 for t in self.files[0].tensors}
            self.source_path = path

    def tensor_opt(self, name: str):
        for candidate in [name] + model_tensor_aliases(name):
            fi = self._file_of.get(candidate)
            if fi is not None:
                return self.files[fi], self.files[fi]._by_name[candidate]
        return None

    def tensor(self, name: str):
        found = self.tensor_opt(name)
        if found is None:
            raise CheckpointError(f"missing tensor {name}")
        return found

    def read(self, name: str, dtype: str | None = None, shape: tuple | None = None) -> np.ndarray:
        f, info = self.tensor(name)
        if dtype is not None and info.dtype != dtype:
            raise CheckpointError(f"tensor {info.name} has dtype {info.dtype}, expected {dtype}")
        if shape is not None and tuple(info.shape) != tuple(shape):
            raise CheckpointError(f"tensor {info.name} has shape {info.shape}, expected {tuple(shape)}")
        return f.read_tensor(info)


@dataclass
class YarnRopeConfig:
    factor: float
    original_max_position_embeddings: int
    beta_fast: float
    beta_slow: float
    attention_factor: float = 1.0


@dataclass
class TextConfig:
    """The fields of kmll's TextConfig that the full-attention decoder uses (model.rs:236-266)."""
    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    rotary_dim: int
    rope_theta: float
    rope_yarn: YarnRopeConfig | None
    max_position_embeddings: int
    vocab_size: int
    norm_eps: float
    eos_token_id: int | None
    sliding_window: int | None = None  # config.json's `sliding_window`; kmll does not read it (full causal attention)

    @staticmethod
    def from_config_json(text: str) -> "TextConfig":
        """TextConfig::from_config_json (model.rs:271-366): a `text_config` object wins over the top level; rope settings
        come from `rope_parameters` when present."""
        top = json.loads(text)
        cfg = top.get("text_config") if isinstance(top.get("text_config"), dict) else top
        model_type = cfg.get("model_type", top.get("model_type"))
        if model_type in ("qwen3_5_text", "qwen3_5") or "layer_types" in cfg and any(t != "full_attention" for t in cfg["layer_types"]):
            raise CheckpointError(f"model type {model_type} with linear-attention layers is outside the full-attention decoder path")

        def need(obj, key, kind):
            if key not in obj:
                raise CheckpointError(f"config.json: missing field {key}")
            return kind(obj[key])

        rope = cfg.get("rope_parameters") if isinstance(cfg.get("rope_parameters"), dict) else None
        partial = float((rope or {}).get("partial_rotary_factor", cfg.get("partial_rotary_factor", 1.0)))
        head_dim = need(cfg, "head_dim", int)
        rotary_dim = rotary_dim_from_partial_factor(head_dim, partial)
        yarn = None
        if rope is not None and rope.get("rope_type", rope.get("type")) == "yarn":
            yarn = YarnRopeConfig(need(rope, "factor", float), need(rope, "original_max_position_embeddings", int), need(rope, "beta_fast", float),
                                  need(rope, "beta_slow", float), float(rope.get("mscale", 1.0)))
        eos = cfg.get("eos_token_id", top.get("eos_token_id"))
        window = cfg.get("sliding_window", top.get("sliding_window"))
        out = TextConfig(dim=need(cfg, "hidden_size", int), hidden_dim=need(cfg, "intermediate_size", int), n_layers=need(cfg, "num_hidden_layers", int),
                         n_heads=need(cfg, "num_attention_heads", int), n_kv_heads=need(cfg, "num_key_value_heads", int), head_dim=head_dim,
                         rotary_dim=rotary_dim, rope_theta=float((rope or {}).get("rope_theta", cfg.get("rope_theta", 10000.0))), rope_yarn=yarn,
                         max_position_embeddings=need(cfg, "max_position_embeddings", int), vocab_size=need(cfg, "vocab_size", int),
                         norm_eps=need(cfg, "rms_norm_eps", float), eos_token_id=int(eos) if isinstance(eos, int) else None,
                         sliding_window=int(window) if isinstance(window, int) and not isinstance(window, bool) and window > 0 else None)
        out.validate_for_inference()
        return out

    def validate_for_inference(self) -> None:
        """validate_for_inference (model.rs:368-525), the checks that apply to this decoder."""
        for field in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, field) <= 0:
                raise CheckpointError(f"text config {field} must be nonzero")
        if self.n_heads % self.n_kv_heads:
            raise CheckpointError(f"num_attention_heads {self.n_heads} is not a multiple of num_key_value_heads {self.n_kv_heads}")
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise CheckpointError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        if not math.isfinite(self.rope_theta) or self.rope_theta <= 0 or not math.isfinite(self.norm_eps) or self.norm_eps <= 0:
            raise CheckpointError("rope_theta and rms_norm_eps must be finite and positive")
        y = self.rope_yarn
        if y is not None:
            if not (math.isfinite(y.factor) and y.factor > 0 and y.original_max_position_embeddings > 0 and y.beta_fast > 0 and y.beta_slow > 0):
                raise CheckpointError("YaRN parameters must be finite and positive")
            if abs(y.attention_factor - 1.0) > float(np.finfo(np.float32).eps):
                raise CheckpointError(f"non-neutral YaRN attention_factor {y.attention_factor} is not supported yet")


def rotary_dim_from_partial_factor(head_dim: int, factor: float) -> int:
    if not math.isfinite(factor) or factor <= 0.0 or factor > 1.0:
        raise CheckpointError(f"partial_rotary_factor {factor} must be in (0, 1]")
    rotary = int(np.float32(head_dim) * np.float32(factor))  # truncation, as `as usize` does (model.rs:474)
    if rotary <= 0 or rotary % 2 or rotary > head_dim:
        raise CheckpointError(f"partial_rotary_factor {factor} gives invalid rotary_dim {rotary} for head_dim {head_dim}")
    return rotary


def rope_frequencies(cfg: TextConfig) -> np.ndarray:
    """rope_frequencies / yarn_rope_frequencies (model.rs:9239-9306), evaluated in f32 like the reference."""
    f = np.float32
    half = cfg.rotary_dim // 2
    theta = f(cfg.rope_theta)
    # powf through float64 and one rounding: what a correctly rounded powf returns (numpy's float32 power is an ulp off at times)
    base = np.array([f(1.0) / f(float(theta) ** float(f(2 * i) / f(cfg.rotary_dim))) for i in range(half)], dtype=np.float32)
    y = cfg.rope_yarn
    if y is None:
        return base

    def correction_dim(rotations):
        ratio = f(y.original_max_position_embeddings) / f(f(rotations) * f(2.0) * f(math.pi))
        num = f(f(cfg.rotary_dim) * f(math.log(float(ratio))))
        return f(num / f(f(2.0) * f(math.log(float(theta)))))

    low = f(max(np.floor(correction_dim(y.beta_fast)), f(0.0)))
    high = f(min(np.ceil(correction_dim(y.beta_slow)), f(cfg.rotary_dim - 1)))
    if abs(low - high) < np.finfo(np.float32).eps:
        high = f(high + f(0.001))
    out = np.empty(half, dtype=np.float32)
    for i in range(half):
        ramp = f(min(max((f(i) - low) / (high - low), f(0.0)), f(1.0)))
        weight = f(f(1.0) - ramp)
        interpolation = f(base[i] / f(y.factor))
        out[i] = f(interpolation * f(f(1.0) - weight) + base[i] * weight)
    return out


def load_decoder(model_dir: str, fmt: int, max_seq_len: int | None = None, fused: bool = True, kv_bf16: bool = False,
                 sliding_window: int | str = 0):
    """config.json + safetensors -> a Decoder with its linear weights quantized to `fmt` on the device (RS-I8 from the
    bf16 values as kmll's exporter does, rowwise_scaled.rs:21-51; W4-G128 from their f32 values).  Returns (decoder, config).
    sliding_window: 0 = full causal attention as kmll runs every model; a positive number = that window; "config" = the
    checkpoint's own `sliding_window` when it has one."""
    import torch

    from . import ops
    from . import runtime as rt
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = TextConfig.from_config_json(f.read())
    weights = ModelWeights(model_dir)
    qk_norm = weights.tensor_opt("layers.0.attention.q_norm.weight") is not None
    if qk_norm != (weights.tensor_opt("layers.0.attention.k_norm.weight") is not None):
        raise CheckpointError("a checkpoint must carry both q_norm and k_norm or neither")
    if sliding_window == "config":
        sliding_window = cfg.sliding_window or 0
    dcfg = rt.DecoderConfig(n_layers=cfg.n_layers, dim=cfg.dim, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim,
                            hidden_dim=cfg.hidden_dim, vocab_size=cfg.vocab_size, rope_theta=cfg.rope_theta, norm_eps=cfg.norm_eps,
                            max_seq_len=max_seq_len or cfg.max_position_embeddings, rotary_dim=cfg.rotary_dim, format=fmt, fused=fused, kv_bf16=kv_bf16,
                            sliding_window=sliding_window)
    dec = rt.Decoder(dcfg)
    q, kv = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim

    def bf16(name, shape):
        f_, info = weights.tensor(name)
        if info.dtype != "BF16" or tuple(info.shape) != tuple(shape):
            raise CheckpointError(f"tensor {info.name}: {info.dtype} {info.shape}, expected BF16 {tuple(shape)}")
        return f_.read_tensor(info)

    def linear(layer, tensor, name, shape):
        bits = torch.from_numpy(bf16(name, shape).view(np.int16)).cuda().view(torch.bfloat16)
        if fmt == rt.FORMAT_RS_I8:
            m = ops.DeviceRowwiseScaledI8Matrix.from_bf16_rows_symmetric(bits)
            dec.set_tensor(layer, tensor, m.values.cpu().numpy(), m.scales.cpu().numpy())
        else:
            m = ops.DeviceW4G128Matrix.from_f32_rows(bits.float())
            dec.set_tensor(layer, tensor, m.packed.cpu().numpy(), m.gscales.view(torch.int16).cpu().numpy().view(np.uint16))

    dec.set_tensor(-1, rt.T_EMBEDDING, bf16("tok_embeddings.weight", (cfg.vocab_size, cfg.dim)))
    dec.set_tensor(-1, rt.T_FINAL_NORM, bf16("norm.weight", (cfg.dim,)))
    out_name = "output.weight" if weights.tensor_opt("output.weight") is not None else "tok_embeddings.weight"  # tied embeddings
    linear(-1, rt.T_OUTPUT, out_name, (cfg.vocab_size, cfg.dim))
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        dec.set_tensor(l, rt.T_ATTENTION_NORM, bf16(p + "attention_norm.weight", (cfg.dim,)))
        dec.set_tensor(l, rt.T_FFN_NORM, bf16(p + "ffn_norm.weight", (cfg.dim,)))
        if qk_norm:  # per-head RMSNorm of query and key rows before RoPE (model.rs:10165-10194)
            dec.set_tensor(l, rt.T_Q_NORM, bf16(p + "attention.q_norm.weight", (cfg.head_dim,)))
            dec.set_tensor(l, rt.T_K_NORM, bf16(p + "attention.k_norm.weight", (cfg.head_dim,)))
        linear(l, rt.T_WQ, p + "attention.wq.weight", (q, cfg.dim))
        linear(l, rt.T_WK, p + "attention.wk.weight", (kv, cfg.dim))
        linear(l, rt.T_WV, p + "attention.wv.weight", (kv, cfg.dim))
        linear(l, rt.T_WO, p + "attention.wo.weight", (cfg.dim, q))
        linear(l, rt.T_W1, p + "feed_forward.w1.weight", (cfg.hidden_dim, cfg.dim))
        linear(l, rt.T_W3, p + "feed_forward.w3.weight", (cfg.hidden_dim, cfg.dim))
        linear(l, rt.T_W2, p + "feed_forward.w2.weight", (cfg.dim, cfg.hidden_dim))
    if cfg.rope_yarn is not None:
        dec.set_rope_freqs(rope_frequencies(cfg))
    return dec, cfg


__all__ = ["SafetensorsFile", "ModelWeights", "TensorInfo", "TextConfig", "YarnRopeConfig", "CheckpointError", "model_tensor_aliases",
           "rope_frequencies", "rotary_dim_from_partial_factor", "write_safetensors", "load_decoder"]
