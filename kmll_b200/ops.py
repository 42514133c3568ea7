"""Host-side mirror of kmll's operator API (crates/inference/src/ops/mod.rs:8-35) over the C ABI.

Function names, argument meaning and error behaviour follow the reference operators; where kmll
panics on a shape mismatch these raise KmllError (code KMLL_ERR_SHAPE).  Tensors are torch CUDA
tensors used purely as device buffers: every call passes raw device pointers and the current
CUDA stream to libkmll_b200.so.  Nothing here computes on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .lib import KmllError, check, load

SINGLE_QUERY_ATTENTION_MAX_SEQ = 131072  # kmll caps its fused kernel at 4096 (kernels/inference.rs:11)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise KmllError(-2, "operand must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KmllError(-2, "operand must be contiguous")
    return t.data_ptr()


def _f32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.float32:
        raise KmllError(-2, f"{name} must be float32, got {t.dtype}")
    return t


# ---- weight containers ------------------------------------------------------------------------
@dataclass
class DeviceRowwiseScaledI8Matrix:
    """kmll's DeviceRowwiseScaledI8Matrix (crates/inference/src/rowwise_scaled.rs:184-189)."""
    values: torch.Tensor  # int8 [rows, cols]
    scales: torch.Tensor  # float32 [rows]
    rows: int
    cols: int
    fmt = "i8"

    @staticmethod
    def from_bf16_rows_symmetric(weight_bf16: torch.Tensor) -> "DeviceRowwiseScaledI8Matrix":
        """from_bf16_rows_symmetric (rowwise_scaled.rs:21-51) run on the device."""
        assert weight_bf16.dtype == torch.bfloat16 and weight_bf16.dim() == 2
        rows, cols = weight_bf16.shape
        values = torch.empty((rows, cols), dtype=torch.int8, device=weight_bf16.device)
        scales = torch.empty(rows, dtype=torch.float32, device=weight_bf16.device)
        check(load().kmll_quantize_rs_i8(_stream(), _p(weight_bf16.contiguous()), rows, cols, _p(values), _p(scales)))
        return DeviceRowwiseScaledI8Matrix(values, scales, rows, cols)

    @staticmethod
    def from_parts(values: torch.Tensor, scales: torch.Tensor) -> "DeviceRowwiseScaledI8Matrix":
        """from_i8_rows_symmetric_parts (rowwise_scaled.rs:65-92)."""
        if values.dim() != 2 or scales.numel() != values.shape[0]:
            raise KmllError(-2, f"rowwise scaled i8 matrix scales length {scales.numel()} does not match row count {values.shape[0]}")
        return DeviceRowwiseScaledI8Matrix(values.contiguous(), scales.contiguous(), values.shape[0], values.shape[1])

    def dequantize(self) -> torch.Tensor:
        out = torch.empty((self.rows, self.cols), dtype=torch.float32, device=self.values.device)
        check(load().kmll_dequant_rs_i8(_stream(), _p(self.values), _p(self.scales), self.rows, self.cols, _p(out)))
        return out

    def shard_rows(self, lo: int, hi: int) -> "DeviceRowwiseScaledI8Matrix":
        return DeviceRowwiseScaledI8Matrix(self.values[lo:hi].contiguous(), self.scales[lo:hi].contiguous(), hi - lo, self.cols)

    def shard_cols(self, lo: int, hi: int) -> "DeviceRowwiseScaledI8Matrix":
        return DeviceRowwiseScaledI8Matrix(self.values[:, lo:hi].contiguous(), self.scales, self.rows, hi - lo)


@dataclass
class DeviceW4G128Matrix:
    """4-bit group-128 symmetric weights: packed nibbles [rows, cols/2] + f16 group scales [rows, cols/128]."""
    packed: torch.Tensor   # uint8 [rows, cols/2]
    gscales: torch.Tensor  # float16 [rows, cols/128]
    rows: int
    cols: int
    fmt = "w4g128"

    @staticmethod
    def from_f32_rows(weight: torch.Tensor) -> "DeviceW4G128Matrix":
        assert weight.dtype == torch.float32 and weight.dim() == 2
        rows, cols = weight.shape
        if cols % 128:
            raise KmllError(-2, f"W4-G128 needs cols % 128 == 0, got {cols}")
        packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device=weight.device)
        gscales = torch.empty((rows, cols // 128), dtype=torch.float16, device=weight.device)
        check(load().kmll_quantize_w4g128(_stream(), _p(weight.contiguous()), rows, cols, _p(packed), _p(gscales)))
        return DeviceW4G128Matrix(packed, gscales, rows, cols)

    def dequantize(self) -> torch.Tensor:
        out = torch.empty((self.rows, self.cols), dtype=torch.float32, device=self.packed.device)
        check(load().kmll_dequant_w4g128(_stream(), _p(self.packed), _p(self.gscales), self.rows, self.cols, _p(out)))
        return out

    def shard_rows(self, lo: int, hi: int) -> "DeviceW4G128Matrix":
        return DeviceW4G128Matrix(self.packed[lo:hi].contiguous(), self.gscales[lo:hi].contiguous(), hi - lo, self.cols)

    def shard_cols(self, lo: int, hi: int) -> "DeviceW4G128Matrix":
        if lo % 128 or hi % 128:
            raise KmllError(-2, "W4-G128 column shards must start and end on multiples of 128")
        return DeviceW4G128Matrix(self.packed[:, lo // 2:hi // 2].contiguous(), self.gscales[:, lo // 128:hi // 128].contiguous(),
                                  self.rows, hi - lo)


@dataclass
class DeviceW4PMatrix:
    """W4-G128 weights in the prepared layout the batch-1 kernels stream (kmll_w4g128_prepare): records of 32 rows x one
    128-column group in tensor-core fragment order.  `pair` = gate and up matrices of a gated MLP interleaved."""
    prepared: torch.Tensor  # uint8
    rows: int
    cols: int
    pair: bool = False
    fmt = "w4p"

    @staticmethod
    def from_canonical(m: DeviceW4G128Matrix) -> "DeviceW4PMatrix":
        n = int(load().kmll_w4g128_prepared_bytes(m.rows, m.cols))
        out = torch.empty(n, dtype=torch.uint8, device=m.packed.device)
        check(load().kmll_w4g128_prepare(_stream(), _p(m.packed), _p(m.gscales), m.rows, m.cols, _p(out)))
        return DeviceW4PMatrix(out, m.rows, m.cols, False)

    @staticmethod
    def from_gate_up(gate: DeviceW4G128Matrix, up: DeviceW4G128Matrix) -> "DeviceW4PMatrix":
        if gate.rows != up.rows or gate.cols != up.cols:
            raise KmllError(-2, "gate and up matrices must have the same shape")
        n = int(load().kmll_w4g128_prepared_pair_bytes(gate.rows, gate.cols))
        out = torch.empty(n, dtype=torch.uint8, device=gate.packed.device)
        check(load().kmll_w4g128_prepare_pair(_stream(), _p(gate.packed), _p(gate.gscales), _p(up.packed), _p(up.gscales), gate.rows,
                                              gate.cols, _p(out)))
        return DeviceW4PMatrix(out, gate.rows, gate.cols, True)


Weight = DeviceRowwiseScaledI8Matrix | DeviceW4G128Matrix | DeviceW4PMatrix


def _w(weight: Weight):
    if isinstance(weight, DeviceRowwiseScaledI8Matrix):
        return "i8", _p(weight.values), _p(weight.scales)
    return "w4g128", _p(weight.packed), _p(weight.gscales)


def _fn(base: str, fmt: str):
    return getattr(load(), f"kmll_{base}_{fmt}")


def _same_fmt(*ws: Weight) -> str:
    fmts = {w.fmt for w in ws}
    if len(fmts) != 1:
        raise KmllError(-2, "all weights of a fused op must share one format")
    return fmts.pop()


def f32_to_bf16(x: torch.Tensor) -> torch.Tensor:
    """Bf16::from_f32 (crates/inference/src/dtypes.rs:153-157) on the device."""
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    check(load().kmll_f32_to_bf16(_stream(), _p(_f32(x, "x").contiguous()), x.numel(), _p(out)))
    return out


def fill_normal(n_or_shape, seed: int, std: float, device="cuda") -> torch.Tensor:
    out = torch.empty(n_or_shape, dtype=torch.float32, device=device)
    check(load().kmll_fill_normal_f32(_stream(), _p(out), out.numel(), seed, std))
    return out


# ---- linear family ------------------------------------------------------------------------------
def linear(x: torch.Tensor, weight: Weight, out: torch.Tensor | None = None) -> torch.Tensor:
    """ops::linear (ops/inference.rs:702-710): out = dequant(W) . x."""
    _f32(x, "input")
    if x.numel() != weight.cols:
        raise KmllError(-2, f"linear operand shape mismatch: input {x.numel()} vs cols {weight.cols}")
    out = torch.empty(weight.rows, dtype=torch.float32, device=x.device) if out is None else out
    if out.numel() != weight.rows:
        raise KmllError(-2, "linear output shape mismatch")
    if isinstance(weight, DeviceW4PMatrix):
        check(load().kmll_linear_w4p(_stream(), _p(x), None, 0.0, _p(weight.prepared), None, weight.rows, weight.cols, _p(out)))
        return out
    fmt, w, s = _w(weight)
    check(_fn("linear", fmt)(_stream(), _p(x), w, s, weight.rows, weight.cols, _p(out)))
    return out


def linear_residual(x, weight: Weight, residual, out=None):
    """linear_residual_bf16 (ops/inference.rs:872-921) for quantized weights: residual + W.x."""
    if x.numel() != weight.cols or residual.numel() != weight.rows:
        raise KmllError(-2, "linear residual shape mismatch")
    out = torch.empty(weight.rows, dtype=torch.float32, device=x.device) if out is None else out
    if isinstance(weight, DeviceW4PMatrix):
        check(load().kmll_linear_w4p(_stream(), _p(_f32(x, "input")), None, 0.0, _p(weight.prepared), _p(_f32(residual, "residual")),
                                     weight.rows, weight.cols, _p(out)))
        return out
    fmt, w, s = _w(weight)
    check(_fn("linear_residual", fmt)(_stream(), _p(_f32(x, "input")), w, s, _p(_f32(residual, "residual")), weight.rows, weight.cols, _p(out)))
    return out


def linear_triple(x, wq: Weight, wk: Weight, wv: Weight, norm_weight=None, eps: float = 0.0):
    """linear_triple_bf16 (ops/inference.rs:924-990) for quantized weights; optional fused RMSNorm."""
    fmt = _same_fmt(wq, wk, wv)
    if not (wq.cols == wk.cols == wv.cols == x.numel()) or wk.rows != wv.rows:
        raise KmllError(-2, "linear triple shape mismatch")
    q = torch.empty(wq.rows, dtype=torch.float32, device=x.device)
    k = torch.empty(wk.rows, dtype=torch.float32, device=x.device)
    v = torch.empty(wv.rows, dtype=torch.float32, device=x.device)
    if fmt == "w4p":
        check(load().kmll_linear_triple_w4p(_stream(), _p(_f32(x, "input")), _p(norm_weight), eps, _p(wq.prepared), _p(wk.prepared),
                                            _p(wv.prepared), wq.rows, wk.rows, wq.cols, _p(q), _p(k), _p(v)))
        return q, k, v
    (_, pq, sq), (_, pk, sk), (_, pv, sv) = _w(wq), _w(wk), _w(wv)
    if norm_weight is None:
        check(_fn("linear_triple", fmt)(_stream(), _p(_f32(x, "input")), pq, sq, pk, sk, pv, sv, wq.rows, wk.rows, wq.cols, _p(q), _p(k), _p(v)))
    else:
        check(_fn("rmsnorm_linear_triple", fmt)(_stream(), _p(_f32(x, "input")), _p(norm_weight), eps, pq, sq, pk, sk, pv, sv,
                                                wq.rows, wk.rows, wq.cols, _p(q), _p(k), _p(v)))
    return q, k, v


def linear_pair(x, wa: Weight, wb: Weight):
    """linear_pair_bf16 (ops/inference.rs:712-775) for quantized weights: two matrices of the same shape, one launch."""
    fmt = _same_fmt(wa, wb)
    if fmt == "w4p":
        raise KmllError(-3, "linear pair takes canonical weights")
    if (wa.rows, wa.cols) != (wb.rows, wb.cols) or wa.cols != x.numel():
        raise KmllError(-2, "paired linear operand shape mismatch")
    a = torch.empty(wa.rows, dtype=torch.float32, device=x.device)
    b = torch.empty(wb.rows, dtype=torch.float32, device=x.device)
    (_, pa, sa), (_, pb, sb) = _w(wa), _w(wb)
    check(_fn("linear_pair", fmt)(_stream(), _p(_f32(x, "input")), pa, sa, pb, sb, wa.rows, wa.cols, _p(a), _p(b)))
    return a, b


def silu_gate_up(x, w_gate: Weight, w_up: Weight | None, norm_weight=None, eps: float = 0.0, out=None):
    """silu_gate_up_bf16 (ops/inference.rs:777-869) for quantized weights: silu(Wg.x) * (Wu.x).  A prepared gate/up pair
    (DeviceW4PMatrix.from_gate_up) is passed as w_gate with w_up = None."""
    if isinstance(w_gate, DeviceW4PMatrix):
        if not w_gate.pair or w_up is not None or x.numel() != w_gate.cols:
            raise KmllError(-2, "silu gate/up over prepared weights takes one gate/up pair")
        out = torch.empty(w_gate.rows, dtype=torch.float32, device=x.device) if out is None else out
        check(load().kmll_silu_gate_up_w4p(_stream(), _p(_f32(x, "input")), _p(norm_weight), eps, _p(w_gate.prepared), w_gate.rows,
                                           w_gate.cols, _p(out)))
        return out
    fmt = _same_fmt(w_gate, w_up)
    if w_gate.rows != w_up.rows or w_gate.cols != w_up.cols or x.numel() != w_gate.cols:
        raise KmllError(-2, "silu gate/up shape mismatch")
    out = torch.empty(w_gate.rows, dtype=torch.float32, device=x.device) if out is None else out
    (_, pg, sg), (_, pu, su) = _w(w_gate), _w(w_up)
    if norm_weight is None:
        check(_fn("silu_gate_up", fmt)(_stream(), _p(_f32(x, "input")), pg, sg, pu, su, w_gate.rows, w_gate.cols, _p(out)))
    else:
        check(_fn("rmsnorm_silu_gate_up", fmt)(_stream(), _p(_f32(x, "input")), _p(norm_weight), eps, pg, sg, pu, su, w_gate.rows,
                                               w_gate.cols, _p(out)))
    return out


def linear_top1_partial_count(rows: int) -> int:
    """linear_top1_i8_scaled_partial_count (ops/inference.rs:258-260)."""
    return int(load().kmll_linear_top1_partial_count(rows))


def linear_top1(x, weight: Weight, partial_tokens=None, partial_logits=None, packed_out=None, norm_weight=None, eps: float = 0.0):
    """linear_top1_i8_scaled (ops/inference.rs:454-560): returns the packed u64 tensor (device)."""
    if x.numel() == 0:
        raise KmllError(-2, "linear top1 input must be nonempty")
    if x.numel() != weight.cols:
        raise KmllError(-2, "linear top1 input dim mismatch")
    n = linear_top1_partial_count(weight.rows)
    dev = x.device
    partial_tokens = torch.zeros(n, dtype=torch.int32, device=dev) if partial_tokens is None else partial_tokens
    partial_logits = torch.zeros(n, dtype=torch.float32, device=dev) if partial_logits is None else partial_logits
    packed_out = torch.zeros(1, dtype=torch.int64, device=dev) if packed_out is None else packed_out
    if partial_tokens.numel() < n or partial_logits.numel() < n:
        raise KmllError(-2, "linear top1 partial buffers too short")
    if isinstance(weight, DeviceW4PMatrix):
        check(load().kmll_linear_top1_w4p(_stream(), _p(_f32(x, "input")), _p(norm_weight), eps, _p(weight.prepared), weight.rows, weight.cols,
                                          _p(partial_tokens), _p(partial_logits), _p(packed_out)))
        return packed_out
    fmt, w, s = _w(weight)
    if norm_weight is None:
        check(_fn("linear_top1", fmt)(_stream(), _p(_f32(x, "input")), w, s, weight.rows, weight.cols, _p(partial_tokens), _p(partial_logits), _p(packed_out)))
    else:
        check(_fn("rmsnorm_linear_top1", fmt)(_stream(), _p(_f32(x, "input")), _p(norm_weight), eps, w, s, weight.rows, weight.cols,
                                              _p(partial_tokens), _p(partial_logits), _p(packed_out)))
    return packed_out


def unpack_top1(packed: int) -> tuple[int, float]:
    """unpack_packed_top_logit (crates/inference/src/model.rs:11808-11812)."""
    packed &= 0xFFFFFFFFFFFFFFFF
    token = packed & 0xFFFFFFFF
    logit = torch.tensor([(packed >> 32) & 0xFFFFFFFF], dtype=torch.int64).to(torch.int32).view(torch.float32).item()
    return token, logit


def linear_batched_workspace(batch: int, input_dim: int, device="cuda"):
    """Caller-owned scratch of the batched linears (None when the shape needs none)."""
    n = int(load().kmll_linear_batched_workspace_bytes(batch, input_dim))
    return torch.empty(n, dtype=torch.uint8, device=device) if n > 0 else None


def linear_batched(x, weight: Weight, batch: int, input_dim: int, output_dim: int, out=None, workspace=None):
    """linear_batched_i8_scaled (ops/matmul.rs:423-463): x is a row-major prefix [batch, input_dim]."""
    if weight.rows != output_dim or weight.cols != input_dim:
        raise KmllError(-2, "batched linear weight shape mismatch")
    if x.numel() < batch * input_dim:
        raise KmllError(-2, f"batched linear input too short: {x.numel()} < {batch * input_dim}")
    out = torch.empty((batch, output_dim), dtype=torch.float32, device=x.device) if out is None else out
    if out.numel() < batch * output_dim:
        raise KmllError(-2, "batched linear output too short")
    if batch == 0:
        return out
    fmt, w, s = _w(weight)
    ws = linear_batched_workspace(batch, input_dim, x.device) if workspace is None else workspace
    check(_fn("linear_batched", fmt)(_stream(), _p(_f32(x, "input")), w, s, batch, input_dim, output_dim, _p(ws), _p(out)))
    return out


def linear_qkv_batched(x, wq: Weight, wk: Weight, wv: Weight, batch: int, input_dim: int, workspace=None):
    """linear_qkv_batched_i8_scaled (ops/matmul.rs:465-510)."""
    fmt = _same_fmt(wq, wk, wv)
    if not (wq.cols == wk.cols == wv.cols == input_dim) or wk.rows != wv.rows:
        raise KmllError(-2, "batched qkv shape mismatch")
    if x.numel() < batch * input_dim:
        raise KmllError(-2, "batched qkv input too short")
    q = torch.empty((batch, wq.rows), dtype=torch.float32, device=x.device)
    k = torch.empty((batch, wk.rows), dtype=torch.float32, device=x.device)
    v = torch.empty((batch, wv.rows), dtype=torch.float32, device=x.device)
    (_, pq, sq), (_, pk, sk), (_, pv, sv) = _w(wq), _w(wk), _w(wv)
    ws = linear_batched_workspace(batch, input_dim, x.device) if workspace is None else workspace
    check(_fn("linear_qkv_batched", fmt)(_stream(), _p(_f32(x, "input")), pq, sq, pk, sk, pv, sv, batch, input_dim, wq.rows, wk.rows,
                                         _p(ws), _p(q), _p(k), _p(v)))
    return q, k, v


# ---- row reductions / elementwise -------------------------------------------------------------
def rmsnorm(x, weight_bf16, eps: float, out=None):
    """ops::rmsnorm (ops/inference.rs:631-653)."""
    if weight_bf16.numel() != x.numel():
        raise KmllError(-2, "RMSNorm operand shape mismatch")
    out = torch.empty_like(x) if out is None else out
    check(load().kmll_rmsnorm(_stream(), _p(_f32(x, "input")), _p(weight_bf16), x.numel(), eps, _p(out)))
    return out


def rmsnorm_batched_bf16(x, weight_bf16, batch: int, dim: int, eps: float, out=None):
    """ops::rmsnorm_batched_bf16 (ops/inference.rs:655-700); bf16 names the WEIGHT dtype as in kmll."""
    if x.numel() < batch * dim:
        raise KmllError(-2, f"batched RMSNorm input too short: {x.numel()} < {batch * dim}")
    if weight_bf16.numel() != dim:
        raise KmllError(-2, "batched RMSNorm weight length mismatch")
    out = torch.empty_like(x) if out is None else out
    if x.dtype == torch.bfloat16:
        check(load().kmll_rmsnorm_batched_bf16io(_stream(), _p(x), _p(weight_bf16), batch, dim, eps, _p(out)))
    else:
        check(load().kmll_rmsnorm_batched(_stream(), _p(_f32(x, "input")), _p(weight_bf16), batch, dim, eps, _p(out)))
    return out


def add(a, b, out=None):
    """ops::add (ops/inference.rs:1129-1150)."""
    if a.numel() != b.numel():
        raise KmllError(-2, "add operand shape mismatch")
    out = torch.empty_like(a) if out is None else out
    check(load().kmll_add(_stream(), _p(_f32(a, "lhs")), _p(_f32(b, "rhs")), a.numel(), _p(out)))
    return out


def add_prefix(a, b, count: int, out):
    """ops::add_prefix (ops/inference.rs:1152-1172)."""
    if min(a.numel(), b.numel(), out.numel()) < count:
        raise KmllError(-2, "add prefix operand too short")
    check(load().kmll_add_prefix(_stream(), _p(_f32(a, "lhs")), _p(_f32(b, "rhs")), count, _p(out)))
    return out


def silu_mul(gate, up, out=None):
    """ops::silu_mul (ops/inference.rs:1061-1082): (g / (1 + exp(-g))) * u."""
    if gate.numel() != up.numel():
        raise KmllError(-2, "silu_mul operand shape mismatch")
    out = torch.empty_like(gate) if out is None else out
    if gate.dtype == torch.bfloat16:
        check(load().kmll_silu_mul_bf16io(_stream(), _p(gate), _p(up), gate.numel(), _p(out)))
    else:
        check(load().kmll_silu_mul(_stream(), _p(_f32(gate, "gate")), _p(_f32(up, "up")), gate.numel(), _p(out)))
    return out


def silu_mul_prefix(gate, up, count: int, out):
    """ops::silu_mul_prefix (ops/inference.rs:1107-1127)."""
    if min(gate.numel(), up.numel(), out.numel()) < count:
        raise KmllError(-2, "silu_mul prefix operand too short")
    check(load().kmll_silu_mul_prefix(_stream(), _p(_f32(gate, "gate")), _p(_f32(up, "up")), count, _p(out)))
    return out


def softmax_rows(x, out=None):
    """Row softmax (three-pass math of kernels/inference.rs:1343-1398) over a [rows, cols] tensor."""
    rows, cols = x.shape
    out = torch.empty_like(x) if out is None else out
    if x.dtype == torch.bfloat16:
        check(load().kmll_softmax_rows_bf16io(_stream(), _p(x), rows, cols, _p(out)))
    else:
        check(load().kmll_softmax_rows(_stream(), _p(_f32(x, "input")), rows, cols, _p(out)))
    return out


def apply_rope(x, freqs, position: int, head_dim: int, out=None):
    """ops::apply_rope (ops/inference.rs:1400-1421)."""
    out = torch.empty_like(x) if out is None else out
    if out.numel() != x.numel():
        raise KmllError(-2, "RoPE output length mismatch")
    check(load().kmll_apply_rope(_stream(), _p(_f32(x, "input")), _p(_f32(freqs, "freqs")), freqs.numel(), position, head_dim,
                                 x.numel(), _p(out)))
    return out


def apply_rope_batched_bf16(x, freqs, positions, out=None):
    """RoPE over [batch, n_heads, head_dim] bf16 with one position per batch row (micro-suite form)."""
    batch, n_heads, head_dim = x.shape
    out = torch.empty_like(x) if out is None else out
    check(load().kmll_apply_rope_batched_bf16io(_stream(), _p(x), _p(_f32(freqs, "freqs")), freqs.numel(), _p(positions), batch,
                                                n_heads, head_dim, _p(out)))
    return out


def write_kv_cache(x, position: int, max_seq_len: int, n_kv_heads: int, head_dim: int, cache):
    """ops::write_kv_cache (ops/inference.rs:1462-1489)."""
    if x.numel() != n_kv_heads * head_dim:
        raise KmllError(-2, "KV cache write token shape mismatch")
    if cache.numel() != max_seq_len * n_kv_heads * head_dim:
        raise KmllError(-2, "KV cache buffer shape mismatch")
    check(load().kmll_write_kv_cache(_stream(), _p(_f32(x, "input")), position, max_seq_len, n_kv_heads, head_dim, _p(cache)))


def apply_rope_write_kv_cache(x, freqs, position: int, max_seq_len: int, n_kv_heads: int, head_dim: int, cache):
    """ops::apply_rope_write_kv_cache (ops/inference.rs:1423-1460)."""
    if x.numel() != n_kv_heads * head_dim:
        raise KmllError(-2, "RoPE KV cache write token shape mismatch")
    if cache.numel() != max_seq_len * n_kv_heads * head_dim:
        raise KmllError(-2, "RoPE KV cache buffer shape mismatch")
    check(load().kmll_apply_rope_write_kv_cache(_stream(), _p(_f32(x, "input")), _p(freqs), freqs.numel(), position, max_seq_len,
                                                n_kv_heads, head_dim, _p(cache)))


def prepare_incremental_attention(query, key, value, freqs, position, max_seq_len, n_heads, n_kv_heads, head_dim, query_rot,
                                  key_cache, value_cache):
    """ops::prepare_incremental_attention (ops/inference.rs:1291-1362)."""
    if query.numel() != n_heads * head_dim or query_rot.numel() != n_heads * head_dim:
        raise KmllError(-2, "query shape mismatch")
    if key.numel() != n_kv_heads * head_dim or value.numel() != n_kv_heads * head_dim:
        raise KmllError(-2, "key/value shape mismatch")
    if key_cache.numel() != max_seq_len * n_kv_heads * head_dim or value_cache.numel() != key_cache.numel():
        raise KmllError(-2, "KV cache shape mismatch")
    check(load().kmll_prepare_incremental_attention(_stream(), _p(query), _p(key), _p(value), _p(freqs), freqs.numel(), position,
                                                    max_seq_len, n_heads, n_kv_heads, head_dim, _p(query_rot), _p(key_cache),
                                                    _p(value_cache)))


def prepare_prefill_attention_batch(query_batch, key_batch, value_batch, freqs, prompt_len, q_len, kv_len, head_dim,
                                    query_rot_batch, key_cache, value_cache):
    """ops::prepare_prefill_attention_batch (ops/inference.rs:1220-1288)."""
    if query_batch.numel() < prompt_len * q_len or query_rot_batch.numel() < prompt_len * q_len:
        raise KmllError(-2, "prefill query batch too short")
    if key_batch.numel() < prompt_len * kv_len or value_batch.numel() < prompt_len * kv_len:
        raise KmllError(-2, "prefill key/value batch too short")
    if key_cache.numel() < prompt_len * kv_len or value_cache.numel() < prompt_len * kv_len:
        raise KmllError(-2, "KV cache too short for prefill prompt")
    check(load().kmll_prepare_prefill_attention_batch(_stream(), _p(query_batch), _p(key_batch), _p(value_batch), _p(freqs),
                                                      freqs.numel(), prompt_len, q_len, kv_len, head_dim, _p(query_rot_batch),
                                                      _p(key_cache), _p(value_cache)))


# ---- attention ----------------------------------------------------------------------------------
def attention_scores(query, key_cache, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim, scores=None):
    """ops::attention_scores (ops/inference.rs:1492-1544); scores is [n_heads, max_seq_len]."""
    scores = torch.zeros((n_heads, max_seq_len), dtype=torch.float32, device=query.device) if scores is None else scores
    check(load().kmll_attention_scores(_stream(), _p(query), _p(key_cache), seq_len, max_seq_len, n_heads, n_kv_heads, head_dim,
                                       _p(scores)))
    return scores


def softmax_value(scores, value_cache, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim, out=None):
    """ops::softmax_value (ops/inference.rs:1606-1654)."""
    out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=scores.device) if out is None else out
    check(load().kmll_softmax_value(_stream(), _p(scores), _p(value_cache), seq_len, max_seq_len, n_heads, n_kv_heads, head_dim,
                                    _p(out)))
    return out


def single_query_attention_workspace(n_heads, head_dim, max_seq_len, device="cuda") -> torch.Tensor:
    n = int(load().kmll_single_query_attention_workspace_floats(n_heads, head_dim, max_seq_len))
    return torch.zeros(n, dtype=torch.float32, device=device)


def single_query_attention(query, key_cache, value_cache, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim, out=None,
                           workspace=None):
    """ops::single_query_attention (ops/inference.rs:1657-1710)."""
    out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=query.device) if out is None else out
    workspace = single_query_attention_workspace(n_heads, head_dim, max_seq_len, query.device) if workspace is None else workspace
    check(load().kmll_single_query_attention(_stream(), _p(query), _p(key_cache), _p(value_cache), seq_len, max_seq_len, n_heads,
                                             n_kv_heads, head_dim, _p(workspace), _p(out)))
    return out


def single_query_attention_noalloc(query, key_cache, value_cache, seq_len, max_seq_len, n_heads, n_kv_heads, head_dim, out=None):
    """single_query_attention with the library's built-in scratch array (no workspace argument, nothing allocated by the C call)."""
    out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=query.device) if out is None else out
    check(load().kmll_single_query_attention_noalloc(_stream(), _p(query), _p(key_cache), _p(value_cache), seq_len, max_seq_len, n_heads,
                                                     n_kv_heads, head_dim, _p(out)))
    return out


def prefill_causal_attention(query_batch, key_cache, value_cache, prompt_len, max_seq_len, n_heads, n_kv_heads, head_dim, out=None):
    """ops::prefill_causal_attention (ops/inference.rs:1713-1771)."""
    out = torch.empty((prompt_len, n_heads * head_dim), dtype=torch.float32, device=query_batch.device) if out is None else out
    check(load().kmll_prefill_causal_attention(_stream(), _p(query_batch), _p(key_cache), _p(value_cache), prompt_len, max_seq_len,
                                               n_heads, n_kv_heads, head_dim, _p(out)))
    return out


# ---- embedding / logit selection ----------------------------------------------------------------
def embedding(table_bf16, token_id: int, dim: int, out=None):
    """ops::embedding (ops/inference.rs:562-588)."""
    if dim <= 0 or table_bf16.numel() % dim:
        raise KmllError(-2, "embedding table shape mismatch")
    vocab = table_bf16.numel() // dim
    out = torch.empty(dim, dtype=torch.float32, device=table_bf16.device) if out is None else out
    check(load().kmll_embedding(_stream(), _p(table_bf16), vocab, dim, token_id, _p(out)))
    return out


def embedding_tokens_bf16(table_bf16, tokens, token_count: int, dim: int, out=None):
    """ops::embedding_tokens_bf16 (ops/inference.rs:590-628); tokens is int32/uint32 on the device."""
    if tokens.numel() < token_count:
        raise KmllError(-2, f"batched embedding token buffer too short: {tokens.numel()} < {token_count}")
    if dim <= 0 or table_bf16.numel() % dim:
        raise KmllError(-2, "batched embedding weight shape mismatch")
    vocab = table_bf16.numel() // dim
    out = torch.empty((token_count, dim), dtype=torch.float32, device=table_bf16.device) if out is None else out
    check(load().kmll_embedding_tokens(_stream(), _p(table_bf16), vocab, dim, _p(tokens), token_count, _p(out)))
    return out


def argmax_f32_packed(logits, packed_out=None):
    """ops::argmax_f32_packed (ops/inference.rs:1858-1882)."""
    packed_out = torch.zeros(1, dtype=torch.int64, device=logits.device) if packed_out is None else packed_out
    check(load().kmll_argmax_f32_packed(_stream(), _p(_f32(logits, "logits")), logits.numel(), _p(packed_out)))
    return packed_out


def top_k_f32(logits, k: int):
    """ops::top_k_f32 (ops/inference.rs:1884-1916)."""
    tokens = torch.zeros(k, dtype=torch.int32, device=logits.device)
    values = torch.zeros(k, dtype=torch.float32, device=logits.device)
    check(load().kmll_top_k_f32(_stream(), _p(_f32(logits, "logits")), logits.numel(), k, _p(tokens), _p(values)))
    return tokens, values
