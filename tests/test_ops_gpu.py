"""GPU parity tests: every operator of the C ABI against the CPU oracle on the same seeded inputs.

Bit-exact where the work is integer/byte (quantized bytes, scales, dequantized weights, arg-max
tokens); kmll's own tolerance max_abs <= 1e-4*sqrt(K) (src/main.rs:4306) and a 1e-4 relative bound
(100x tighter than the 1e-2 the task allows) for f32 reductions whose order differs.
"""
import numpy as np
import pytest
import torch

import oracle
from kmll_b200 import ops
from kmll_b200.lib import KmllError

pytestmark = pytest.mark.gpu
F = np.float32


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype)
    return t.cuda()


def bf16_dev(bits):
    return dev(bits.view(np.int16), torch.bfloat16) if bits.dtype == np.uint16 else dev(bits)


def host(t):
    return t.detach().cpu().numpy()


def i8_weight(rng, rows, cols, scale=0.02):
    wb = oracle.bf16_from_f32(rng.normal(0, scale, (rows, cols)).astype(F))
    q, sc = oracle.rs_i8_quantize(wb)
    return wb, q, sc, ops.DeviceRowwiseScaledI8Matrix.from_parts(dev(q), dev(sc))


def w4_weight(rng, rows, cols, scale=0.02):
    w = rng.normal(0, scale, (rows, cols)).astype(F)
    packed, gs = oracle.w4_quantize(w)
    return w, packed, gs, ops.DeviceW4G128Matrix(dev(packed), dev(gs.view(np.int16), torch.float16), rows, cols)


def assert_close(got, ref, k, what=""):
    got, ref = np.asarray(got, dtype=F), np.asarray(ref, dtype=F)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    diff = float(np.max(np.abs(got - ref))) if got.size else 0.0
    scale = max(float(np.max(np.abs(ref))) if ref.size else 0.0, 1e-30)
    assert np.all(np.isfinite(got)), what
    assert diff <= 1e-4 * np.sqrt(max(k, 1)), (what, diff)
    assert diff / scale <= 1e-4, (what, diff, scale)


# ---- quantizers: bit-exact ---------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(4096, 4096), (17, 23), (1, 1), (64, 896)])
def test_quantize_rs_i8_bit_exact(cuda, rows, cols):
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (rows, cols)).astype(F)
    if rows > 2:
        w[1] = 0.0  # zero row -> scale 1.0
    wb = oracle.bf16_from_f32(w)
    wdev = ops.f32_to_bf16(dev(w))
    assert np.array_equal(host(wdev.view(torch.int16)).view(np.uint16), wb)
    m = ops.DeviceRowwiseScaledI8Matrix.from_bf16_rows_symmetric(wdev)
    q, sc = oracle.rs_i8_quantize(wb)
    assert np.array_equal(host(m.values), q)
    assert np.array_equal(host(m.scales).view(np.uint32), sc.view(np.uint32))
    assert np.array_equal(host(m.dequantize()).view(np.uint32), oracle.rs_i8_dequant(q, sc).view(np.uint32))


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (24, 384), (3, 128)])
def test_quantize_w4_bit_exact(cuda, rows, cols, golden):
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (rows, cols)).astype(F) if (rows, cols) != (24, 384) else golden["w4_w"]
    m = ops.DeviceW4G128Matrix.from_f32_rows(dev(w))
    packed, gs = oracle.w4_quantize(w)
    assert np.array_equal(host(m.packed), packed)
    assert np.array_equal(host(m.gscales.view(torch.int16)).view(np.uint16), gs)
    assert np.array_equal(host(m.dequantize()).view(np.uint32), oracle.w4_dequant(packed, gs).view(np.uint32))
    if (rows, cols) == (24, 384):
        assert np.array_equal(host(m.packed), golden["w4_packed"])


def test_w4_requires_group_multiple(cuda):
    with pytest.raises(KmllError):
        ops.DeviceW4G128Matrix.from_f32_rows(torch.zeros((4, 100), device="cuda"))


# ---- linear ----------------------------------------------------------------------------------------
def test_linear_i8_reference_stress_cases(cuda, golden):
    """kmll's gemm-stress linear-i8-scaled cases (src/main.rs:463-472, :3548-3609)."""
    for idx in range(8):
        m, n, k = (int(v) for v in golden[f"gemm_i8_{idx}_shape"])
        w = ops.DeviceRowwiseScaledI8Matrix.from_parts(dev(golden[f"gemm_i8_{idx}_q"]), dev(golden[f"gemm_i8_{idx}_scales"]))
        x = dev(golden[f"gemm_i8_{idx}_x"])
        y = ops.linear_batched(x, w, m, k, n)
        diff = np.max(np.abs(host(y) - golden[f"gemm_i8_{idx}_y"]))
        assert diff <= 1e-4 * np.sqrt(k), (idx, diff)
        y0 = ops.linear(x[0].contiguous(), w)
        assert np.max(np.abs(host(y0) - golden[f"gemm_i8_{idx}_y"][0])) <= 1e-4 * np.sqrt(k)


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1024, 4096), (4096, 14336), (1000, 256), (17, 64), (896, 896), (33, 19008)])
def test_linear_i8_vs_oracle(cuda, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    _, q, sc, w = i8_weight(rng, rows, cols)
    x = rng.normal(0, 1, cols).astype(F)
    assert_close(host(ops.linear(dev(x), w)), oracle.rs_i8_matvec(q, sc, x), cols, f"i8 {rows}x{cols}")


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1024, 4096), (4096, 14336), (1000, 256), (17, 128), (896, 896), (33, 18944)])
def test_linear_w4_vs_oracle(cuda, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    _, packed, gs, w = w4_weight(rng, rows, cols)
    x = rng.normal(0, 1, cols).astype(F)
    assert_close(host(ops.linear(dev(x), w)), oracle.w4_matvec(packed, gs, x), cols, f"w4 {rows}x{cols}")


def test_linear_large_and_tiny_activations(cuda):
    """The power-of-two activation scaling keeps f32 accuracy for huge, tiny and mixed magnitudes."""
    rng = np.random.default_rng(5)
    _, packed, gs, w = w4_weight(rng, 64, 1024)
    _, q, sc, wi = i8_weight(rng, 64, 1024)
    for mag in (1e-20, 1e-6, 1.0, 3e4, 1e9, 1e20):
        x = (rng.normal(0, 1, 1024) * mag).astype(F)
        x[::7] *= F(1e-4)
        assert_close(host(ops.linear(dev(x), w)) / mag, oracle.w4_matvec(packed, gs, x) / mag, 1024, f"w4 mag {mag}")
        assert_close(host(ops.linear(dev(x), wi)) / mag, oracle.rs_i8_matvec(q, sc, x) / mag, 1024, f"i8 mag {mag}")
    zero = torch.zeros(1024, device="cuda")
    assert torch.count_nonzero(ops.linear(zero, w)) == 0


def test_linear_is_deterministic(cuda):
    rng = np.random.default_rng(6)
    _, _, _, w = w4_weight(rng, 4096, 4096)
    x = dev(rng.normal(0, 1, 4096).astype(F))
    a = ops.linear(x, w).clone()
    for _ in range(3):
        assert torch.equal(ops.linear(x, w), a)


def test_linear_shape_errors(cuda):
    rng = np.random.default_rng(7)
    _, _, _, w = w4_weight(rng, 32, 256)
    with pytest.raises(KmllError):
        ops.linear(torch.zeros(255, device="cuda"), w)
    with pytest.raises(KmllError):
        ops.linear(torch.zeros(256, device="cuda"), w, out=torch.zeros(31, device="cuda"))
    with pytest.raises(KmllError):
        ops.linear(torch.zeros(256), w)  # host tensor: there is no CPU path


@pytest.mark.parametrize("fmt", ["i8", "w4"])
def test_config1_op_chain(cuda, fmt):
    """W 4096x4096 ~ N(0,0.02) seed 0, x and r f16-representable N(0,1); y = dequant(W).x; h = RMSNorm(y + r)."""
    rng = np.random.default_rng(0)
    w32 = rng.normal(0, 0.02, (4096, 4096)).astype(F)
    x = rng.normal(0, 1, 4096).astype(np.float16).astype(F)
    r = rng.normal(0, 1, 4096).astype(np.float16).astype(F)
    gamma = oracle.bf16_from_f32(rng.uniform(0.5, 1.5, 4096).astype(F))
    if fmt == "i8":
        wb = oracle.bf16_from_f32(w32)
        q, sc = oracle.rs_i8_quantize(wb)
        w = ops.DeviceRowwiseScaledI8Matrix.from_bf16_rows_symmetric(ops.f32_to_bf16(dev(w32)))
        assert np.array_equal(host(w.dequantize()).view(np.uint32), oracle.rs_i8_dequant(q, sc).view(np.uint32))
        y_ref = oracle.rs_i8_matvec(q, sc, x)
    else:
        packed, gs = oracle.w4_quantize(w32)
        w = ops.DeviceW4G128Matrix.from_f32_rows(dev(w32))
        assert np.array_equal(host(w.dequantize()).view(np.uint32), oracle.w4_dequant(packed, gs).view(np.uint32))
        y_ref = oracle.w4_matvec(packed, gs, x)
    h_ref = oracle.rmsnorm(oracle.add(y_ref, r), gamma, 1e-6)
    s = ops.linear_residual(dev(x), w, dev(r))
    h = ops.rmsnorm(s, bf16_dev(gamma), 1e-6)
    assert_close(host(s), oracle.add(y_ref, r), 4096, "y + r")
    rel = np.max(np.abs(host(h) - h_ref) / np.maximum(np.abs(h_ref), 1e-3))
    assert rel <= 1e-2 and np.max(np.abs(host(h) - h_ref)) <= 1e-4


@pytest.mark.parametrize("fmt", ["i8", "w4"])
def test_fused_linear_forms(cuda, fmt):
    rng = np.random.default_rng(11)
    dim, qr, kvr, hid = 512, 512, 128, 1376
    mk = i8_weight if fmt == "i8" else w4_weight
    mv = (lambda a, b, c, x: oracle.rs_i8_matvec(b, c, x)) if fmt == "i8" else (lambda a, b, c, x: oracle.w4_matvec(b, c, x))
    x = rng.normal(0, 1, dim).astype(F)
    gamma = oracle.bf16_from_f32(rng.uniform(0.5, 1.5, dim).astype(F))
    wq, wk, wv = mk(rng, qr, dim), mk(rng, kvr, dim), mk(rng, kvr, dim)
    # triple, plain and with fused RMSNorm
    q, k, v = ops.linear_triple(dev(x), wq[3], wk[3], wv[3])
    for got, w in ((q, wq), (k, wk), (v, wv)):
        assert_close(host(got), mv(*w[:3], x), dim, "triple")
    xn = oracle.rmsnorm(x, gamma, 1e-5)
    q, k, v = ops.linear_triple(dev(x), wq[3], wk[3], wv[3], norm_weight=bf16_dev(gamma), eps=1e-5)
    for got, w in ((q, wq), (k, wk), (v, wv)):
        assert_close(host(got), mv(*w[:3], xn), dim, "norm+triple")
    # pair (two matrices of one shape, one launch)
    a, b = ops.linear_pair(dev(x), wk[3], wv[3])
    assert_close(host(a), mv(*wk[:3], x), dim, "pair a")
    assert_close(host(b), mv(*wv[:3], x), dim, "pair b")
    with pytest.raises(ops.KmllError):
        ops.linear_pair(dev(x), wq[3], wk[3])
    # residual
    res = rng.normal(0, 1, qr).astype(F)
    assert_close(host(ops.linear_residual(dev(x), wq[3], dev(res))), oracle.add(res, mv(*wq[:3], x)), dim, "residual")
    # silu gate/up, plain and with fused RMSNorm
    wg, wu = mk(rng, hid, dim, 0.05), mk(rng, hid, dim, 0.05)
    ref = oracle.silu_mul(mv(*wg[:3], x), mv(*wu[:3], x))
    assert_close(host(ops.silu_gate_up(dev(x), wg[3], wu[3])), ref, dim, "silu gate up")
    ref = oracle.silu_mul(mv(*wg[:3], xn), mv(*wu[:3], xn))
    assert_close(host(ops.silu_gate_up(dev(x), wg[3], wu[3], norm_weight=bf16_dev(gamma), eps=1e-5)), ref, dim, "norm+silu")


def test_linear_top1_i8_reference_stress_cases(cuda, golden):
    """kmll's logit-stress scaled-i8 top-1 cases (src/main.rs:4123-4185): token must match, logit within 1e-4*sqrt(in)."""
    for idx in range(6):
        rows, cols = (int(v) for v in golden[f"top1_i8_{idx}_shape"])
        wdev = ops.DeviceRowwiseScaledI8Matrix.from_bf16_rows_symmetric(bf16_dev(golden[f"top1_i8_{idx}_wbits"]))
        packed = ops.linear_top1(dev(golden[f"top1_i8_{idx}_x"]), wdev)
        token, logit = ops.unpack_top1(int(packed.item()))
        exp_token, exp_bits = (int(v) for v in golden[f"top1_i8_{idx}_expected"])
        exp_logit = np.array([exp_bits], dtype=np.uint32).view(F)[0]
        assert token == exp_token, idx
        assert abs(logit - exp_logit) <= 1e-4 * np.sqrt(cols), idx


@pytest.mark.parametrize("fmt,rows,cols", [("i8", 4097, 96), ("i8", 8192, 128), ("w4", 8192, 128), ("w4", 32000, 512), ("i8", 1000, 64), ("w4", 33, 256)])
def test_linear_top1_vs_oracle(cuda, fmt, rows, cols):
    g = oracle.Lcg(rows * 31 + cols)
    x = g.fill_f32(cols)
    wf = g.fill_f32(rows * cols).reshape(rows, cols)
    forced = rows // 3
    wf[forced] = np.where(x >= 0, F(4.0), F(-4.0))  # planted winning row as in the reference harness
    if fmt == "i8":
        wb = oracle.bf16_from_f32(wf)
        q, sc = oracle.rs_i8_quantize(wb)
        w = ops.DeviceRowwiseScaledI8Matrix.from_parts(dev(q), dev(sc))
        logits = oracle.rs_i8_matvec(q, sc, x)
    else:
        packed, gs = oracle.w4_quantize(wf)
        w = ops.DeviceW4G128Matrix(dev(packed), dev(gs.view(np.int16), torch.float16), rows, cols)
        logits = oracle.w4_matvec(packed, gs, x)
    exp_token, exp_logit = oracle.unpack_top1(oracle.top1_packed(logits))
    token, logit = ops.unpack_top1(int(ops.linear_top1(dev(x), w).item()))
    assert token == exp_token == forced
    assert abs(logit - exp_logit) <= 1e-4 * np.sqrt(cols)


def test_linear_top1_tie_prefers_lower_token(cuda):
    rows, cols = 200, 128
    q = np.zeros((rows, cols), dtype=np.int8)
    q[150] = 5
    q[37] = 5
    q[199] = 5
    sc = np.ones(rows, dtype=F)
    w = ops.DeviceRowwiseScaledI8Matrix.from_parts(dev(q), dev(sc))
    x = np.ones(cols, dtype=F)
    token, logit = ops.unpack_top1(int(ops.linear_top1(dev(x), w).item()))
    assert token == 37 and logit == 5.0 * cols
    gamma = oracle.bf16_from_f32(np.ones(cols, dtype=F))
    token, _ = ops.unpack_top1(int(ops.linear_top1(dev(x), w, norm_weight=bf16_dev(gamma), eps=1e-6).item()))
    assert token == 37


@pytest.mark.parametrize("fmt", ["i8", "w4"])
@pytest.mark.parametrize("batch", [2, 4, 5, 8, 16, 33])
def test_linear_batched_vs_oracle(cuda, fmt, batch):
    rng = np.random.default_rng(100 + batch)
    rows, cols = 300, 512
    x = rng.normal(0, 1, (batch, cols)).astype(F)
    if fmt == "i8":
        _, q, sc, w = i8_weight(rng, rows, cols)
        ref = oracle.rs_i8_linear_batched(x, q, sc)
    else:
        _, packed, gs, w = w4_weight(rng, rows, cols)
        ref = oracle.w4_linear_batched(x, packed, gs)
    assert_close(host(ops.linear_batched(dev(x), w, batch, cols, rows)), ref, cols, f"batched {fmt} {batch}")


@pytest.mark.parametrize("batch", [9, 33])
def test_linear_batched_i8_split_k(cuda, batch):
    """Few row tiles and a long K: the tensor-core kernel splits K over several blocks per row tile and the block that
    arrives last merges the partial sums; two calls in a row check that the arrival counters are left at zero."""
    rng = np.random.default_rng(700 + batch)
    rows, cols = 700, 4096
    x = rng.normal(0, 1, (batch, cols)).astype(F)
    _, q, sc, w = i8_weight(rng, rows, cols)
    ref = oracle.rs_i8_linear_batched(x, q, sc)
    first = host(ops.linear_batched(dev(x), w, batch, cols, rows))
    second = host(ops.linear_batched(dev(x), w, batch, cols, rows))
    assert_close(first, ref, cols, f"split-k i8 {batch}")
    assert np.array_equal(first, second)


def test_linear_batched_large_k_chunks_and_qkv(cuda):
    rng = np.random.default_rng(9)
    batch, cols = 16, 4096  # 16 rows x 4096 forces several K chunks
    x = rng.normal(0, 1, (batch, cols)).astype(F)
    _, packed, gs, w = w4_weight(rng, 96, cols)
    assert_close(host(ops.linear_batched(dev(x), w, batch, cols, 96)), oracle.w4_linear_batched(x, packed, gs), cols, "chunks")
    wq, wk, wv = i8_weight(rng, 256, 512), i8_weight(rng, 64, 512), i8_weight(rng, 64, 512)
    xs = rng.normal(0, 1, (7, 512)).astype(F)
    q, k, v = ops.linear_qkv_batched(dev(xs), wq[3], wk[3], wv[3], 7, 512)
    for got, wt in ((q, wq), (k, wk), (v, wv)):
        assert_close(host(got), oracle.rs_i8_linear_batched(xs, wt[1], wt[2]), 512, "qkv batched")
    with pytest.raises(KmllError):
        ops.linear_batched(dev(xs), wq[3], 8, 512, 256)  # input shorter than batch*input_dim


# ---- row reductions / elementwise ---------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 3, 255, 256, 257, 896, 4096, 5000])
def test_rmsnorm_vs_oracle(cuda, n):
    rng = np.random.default_rng(n)
    x = rng.normal(0, 1, n).astype(F)
    w = oracle.bf16_from_f32(rng.uniform(0.5, 1.5, n).astype(F))
    got = host(ops.rmsnorm(dev(x), bf16_dev(w), 1e-6))
    ref = oracle.rmsnorm(x, w, 1e-6)
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-6)) <= 1e-5
    xb = rng.normal(0, 1, (5, n)).astype(F)
    got = host(ops.rmsnorm_batched_bf16(dev(xb), bf16_dev(w), 5, n, 1e-5))
    ref = oracle.rmsnorm(xb, w, 1e-5)
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-6)) <= 1e-5
    with pytest.raises(KmllError):
        ops.rmsnorm(dev(x), bf16_dev(w[:-1]) if n > 1 else bf16_dev(np.zeros(2, dtype=np.uint16)), 1e-6)


@pytest.mark.parametrize("n", [1, 5, 4096, 11008, 14337])
def test_add_and_silu_mul_vs_oracle(cuda, n):
    rng = np.random.default_rng(n)
    a = rng.normal(0, 3, n).astype(F)
    b = rng.normal(0, 3, n).astype(F)
    assert np.array_equal(host(ops.add(dev(a), dev(b))), oracle.add(a, b))
    got, ref = host(ops.silu_mul(dev(a), dev(b))), oracle.silu_mul(a, b)
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-6)) <= 1e-6
    out = torch.full((n + 3,), 7.0, device="cuda")
    ops.add_prefix(torch.cat([dev(a), torch.zeros(3, device="cuda")]), torch.cat([dev(b), torch.zeros(3, device="cuda")]), n, out)
    assert np.array_equal(host(out[:n]), oracle.add(a, b)) and torch.all(out[n:] == 7.0)
    out2 = torch.full((n + 3,), 7.0, device="cuda")
    ops.silu_mul_prefix(torch.cat([dev(a), torch.zeros(3, device="cuda")]), torch.cat([dev(b), torch.zeros(3, device="cuda")]), n, out2)
    assert torch.all(out2[n:] == 7.0)
    with pytest.raises(KmllError):
        ops.add(dev(a), torch.zeros(n + 1, device="cuda"))


def test_rope_known_answer_and_oracle(cuda, golden):
    out = host(ops.apply_rope(dev(golden["rope_kat_input"]), dev(golden["rope_kat_freqs"]), 1, 6))
    assert np.max(np.abs(out - golden["rope_kat_expected"])) < 1e-6  # crates/inference/src/model.rs:12227-12249
    rng = np.random.default_rng(3)
    for head_dim, rotary, n_heads, pos in [(128, 128, 32, 4095), (64, 64, 14, 511), (256, 64, 4, 1234), (128, 128, 8, 0)]:
        freqs = oracle.rope_frequencies(1e6, rotary)
        x = rng.normal(0, 1, n_heads * head_dim).astype(F)
        got = host(ops.apply_rope(dev(x), dev(freqs), pos, head_dim))
        ref = oracle.apply_rope(x, freqs, pos, head_dim)
        assert np.max(np.abs(got - ref)) <= 2e-6, (head_dim, pos)
    with pytest.raises(KmllError):
        ops.apply_rope(torch.zeros(12, device="cuda"), torch.zeros(4, device="cuda"), 0, 6)  # too many freqs
    with pytest.raises(KmllError):
        ops.apply_rope(torch.zeros(10, device="cuda"), torch.zeros(2, device="cuda"), 0, 6)  # len % head_dim


def test_kv_cache_writes_and_prepare(cuda):
    rng = np.random.default_rng(4)
    n_heads, n_kv, hd, max_seq, pos = 8, 2, 64, 16, 5
    freqs = oracle.rope_frequencies(1e6, hd)
    q = rng.normal(0, 1, n_heads * hd).astype(F)
    k = rng.normal(0, 1, n_kv * hd).astype(F)
    v = rng.normal(0, 1, n_kv * hd).astype(F)
    kc = torch.zeros(max_seq * n_kv * hd, device="cuda")
    vc = torch.zeros_like(kc)
    ops.write_kv_cache(dev(v), pos, max_seq, n_kv, hd, vc)
    ops.apply_rope_write_kv_cache(dev(k), dev(freqs), pos, max_seq, n_kv, hd, kc)
    k_rot = oracle.apply_rope(k, freqs, pos, hd)
    kc_h, vc_h = host(kc).reshape(max_seq, -1), host(vc).reshape(max_seq, -1)
    assert np.array_equal(vc_h[pos], v) and np.count_nonzero(np.delete(vc_h, pos, 0)) == 0
    assert np.max(np.abs(kc_h[pos] - k_rot)) <= 2e-6 and np.count_nonzero(np.delete(kc_h, pos, 0)) == 0
    # fused form agrees with the split form to 1e-6 (src/main.rs:4456)
    kc2, vc2, qr = torch.zeros_like(kc), torch.zeros_like(kc), torch.zeros(n_heads * hd, device="cuda")
    ops.prepare_incremental_attention(dev(q), dev(k), dev(v), dev(freqs), pos, max_seq, n_heads, n_kv, hd, qr, kc2, vc2)
    assert torch.max(torch.abs(kc2 - kc)) <= 1e-6 and torch.equal(vc2, vc)
    assert np.max(np.abs(host(qr) - oracle.apply_rope(q, freqs, pos, hd))) <= 2e-6
    with pytest.raises(KmllError):
        ops.write_kv_cache(dev(v), max_seq, max_seq, n_kv, hd, vc)  # position out of range
    # prefill staging: row i is position i
    plen = 7
    qb = rng.normal(0, 1, (plen, n_heads * hd)).astype(F)
    kb = rng.normal(0, 1, (plen, n_kv * hd)).astype(F)
    vb = rng.normal(0, 1, (plen, n_kv * hd)).astype(F)
    qrb, kc3, vc3 = torch.zeros(plen * n_heads * hd, device="cuda"), torch.zeros_like(kc), torch.zeros_like(kc)
    ops.prepare_prefill_attention_batch(dev(qb), dev(kb), dev(vb), dev(freqs), plen, n_heads * hd, n_kv * hd, hd, qrb, kc3, vc3)
    for i in range(plen):
        assert np.max(np.abs(host(qrb).reshape(plen, -1)[i] - oracle.apply_rope(qb[i], freqs, i, hd))) <= 2e-6
        assert np.max(np.abs(host(kc3).reshape(max_seq, -1)[i] - oracle.apply_rope(kb[i], freqs, i, hd))) <= 2e-6
        assert np.array_equal(host(vc3).reshape(max_seq, -1)[i], vb[i])


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 17), (32, 4096), (5, 5000), (64, 257)])
def test_softmax_rows_vs_oracle(cuda, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.normal(0, 3, (rows, cols)).astype(F)
    got, ref = host(ops.softmax_rows(dev(x))), oracle.softmax_rows(x)
    assert np.max(np.abs(got - ref) / np.maximum(ref, 1e-3)) <= 1e-5  # summation order differs
    assert np.max(np.abs(got.sum(axis=1) - 1.0)) <= 1e-5


@pytest.mark.parametrize("batch", [1, 16, 64])
def test_microsuite_bf16_io(cuda, batch):
    """RMSNorm [B,4096], SwiGLU [B,11008], RoPE [B,32,128] theta 1e6, softmax [B*32,4096]; bf16 in/out, seed 1."""
    rng = np.random.default_rng(1)

    def bf(a):
        return oracle.bf16_from_f32(a.astype(F))

    def check(got_t, ref_f32):
        got = oracle.bf16_to_f32(host(got_t.view(torch.int16)).view(np.uint16))
        ref = oracle.bf16_to_f32(bf(ref_f32))
        assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-2)) <= 1e-2
        # at most a rounding-boundary flip: the two results differ by <= 1 bf16 ulp almost everywhere
        assert np.mean(got != ref) < 0.02

    x = bf(rng.normal(0, 1, (batch, 4096)))
    gamma = bf(rng.uniform(0.5, 1.5, 4096))
    check(ops.rmsnorm_batched_bf16(bf16_dev(x), bf16_dev(gamma), batch, 4096, 1e-6), oracle.rmsnorm(oracle.bf16_to_f32(x), gamma, 1e-6))
    g, u = bf(rng.normal(0, 1, (batch, 11008))), bf(rng.normal(0, 1, (batch, 11008)))
    check(ops.silu_mul(bf16_dev(g), bf16_dev(u)), oracle.silu_mul(oracle.bf16_to_f32(g), oracle.bf16_to_f32(u)))
    xr = bf(rng.normal(0, 1, (batch, 32, 128)))
    pos = rng.integers(0, 4096, batch).astype(np.int32)
    freqs = oracle.rope_frequencies(1e6, 128)
    ref = np.stack([oracle.apply_rope(oracle.bf16_to_f32(xr[b]).reshape(-1), freqs, int(pos[b]), 128).reshape(32, 128) for b in range(batch)])
    check(ops.apply_rope_batched_bf16(bf16_dev(xr), dev(freqs), dev(pos)), ref)
    xs = bf(rng.normal(0, 1, (batch * 32, 4096)))
    check(ops.softmax_rows(bf16_dev(xs)), oracle.softmax_rows(oracle.bf16_to_f32(xs)))


# ---- attention ------------------------------------------------------------------------------------
@pytest.mark.parametrize("n_heads,n_kv,hd,seq,max_seq", [(32, 8, 128, 1, 64), (32, 8, 128, 63, 64), (32, 8, 128, 65, 2304),
                                                         (32, 8, 128, 2304, 2304), (14, 2, 64, 640, 640), (4, 4, 64, 100, 4100),
                                                         (8, 1, 128, 300, 512)])
def test_single_query_attention_vs_oracle(cuda, n_heads, n_kv, hd, seq, max_seq):
    rng = np.random.default_rng(seq + n_heads)
    q = rng.normal(0, 1, n_heads * hd).astype(F)
    kc = rng.normal(0, 1, (max_seq, n_kv, hd)).astype(F)
    vc = rng.normal(0, 1, (max_seq, n_kv, hd)).astype(F)
    ref = oracle.single_query_attention(q, kc, vc, seq, n_heads, n_kv, hd)
    ws = ops.single_query_attention_workspace(n_heads, hd, max_seq)
    got = ops.single_query_attention(dev(q), dev(kc), dev(vc), seq, max_seq, n_heads, n_kv, hd, workspace=ws)
    assert np.max(np.abs(host(got) - ref)) <= 5e-5  # kmll's fused-vs-split bound (src/main.rs:4401)
    # the workspace counters are left clean: a second call with the same workspace agrees exactly
    got2 = ops.single_query_attention(dev(q), dev(kc), dev(vc), seq, max_seq, n_heads, n_kv, hd, workspace=ws)
    assert torch.equal(got, got2)
    # split form
    sc = ops.attention_scores(dev(q), dev(kc), seq, max_seq, n_heads, n_kv, hd)
    sc_ref = oracle.attention_scores(q, kc, seq, max_seq, n_heads, n_kv, hd)
    assert np.max(np.abs(host(sc)[:, :seq] - sc_ref[:, :seq])) <= 1e-5
    out = ops.softmax_value(sc, dev(vc), seq, max_seq, n_heads, n_kv, hd)
    assert np.max(np.abs(host(out) - ref)) <= 5e-5


def test_attention_geometry_errors(cuda):
    z = torch.zeros(8 * 64, device="cuda")
    cache = torch.zeros(16 * 2 * 64, device="cuda")
    with pytest.raises(KmllError):
        ops.single_query_attention(z, cache, cache, 17, 16, 8, 2, 64)  # seq_len > max_seq_len
    with pytest.raises(KmllError):
        ops.single_query_attention(z, cache, cache, 4, 16, 8, 3, 64)  # heads not divisible
    with pytest.raises(KmllError):
        ops.single_query_attention(torch.zeros(8 * 32, device="cuda"), cache, cache, 4, 16, 8, 2, 32)  # unsupported head_dim


@pytest.mark.parametrize("n_heads,n_kv,hd,plen", [(8, 2, 128, 1), (8, 2, 128, 17), (14, 2, 64, 100), (4, 4, 64, 33)])
def test_prefill_causal_attention_vs_oracle(cuda, n_heads, n_kv, hd, plen):
    rng = np.random.default_rng(plen)
    max_seq = plen + 3
    qb = rng.normal(0, 1, (plen, n_heads * hd)).astype(F)
    kc = rng.normal(0, 1, (max_seq, n_kv, hd)).astype(F)
    vc = rng.normal(0, 1, (max_seq, n_kv, hd)).astype(F)
    ref = oracle.prefill_causal_attention(qb, kc, vc, plen, n_heads, n_kv, hd)
    got = ops.prefill_causal_attention(dev(qb), dev(kc), dev(vc), plen, max_seq, n_heads, n_kv, hd)
    assert np.max(np.abs(host(got) - ref)) <= 5e-5


# ---- embedding / logit selection --------------------------------------------------------------------
def test_embedding_vs_oracle(cuda):
    rng = np.random.default_rng(8)
    table = oracle.bf16_from_f32(rng.normal(0, 1, (100, 96)).astype(F))
    t = bf16_dev(table)
    assert np.array_equal(host(ops.embedding(t, 37, 96)), oracle.embedding(table, 37))
    toks = np.array([0, 99, 5, 5], dtype=np.int32)
    got = host(ops.embedding_tokens_bf16(t, dev(toks), 4, 96))
    for i, tok in enumerate(toks):
        assert np.array_equal(got[i], oracle.embedding(table, int(tok)))
    with pytest.raises(KmllError):
        ops.embedding(t, 100, 96)  # token out of range
    with pytest.raises(KmllError):
        ops.embedding_tokens_bf16(t, dev(toks), 5, 96)  # token buffer too short


def test_argmax_packed_reference_tie_cases(cuda, golden):
    for idx in range(8):
        logits = golden[f"argmax_{idx}_logits"]
        token, logit = ops.unpack_top1(int(ops.argmax_f32_packed(dev(logits)).item()))
        assert token == int(golden[f"argmax_{idx}_expected"][0]) and logit == 12345.0
    g = oracle.Lcg(99)
    for n in (32768, 65537, 131072):  # the long lengths of the reference list (src/main.rs:1633)
        logits = g.fill_f32(n, 10.0)
        logits[n // 3] = logits[n - 1] = F(12345.0)
        token, logit = ops.unpack_top1(int(ops.argmax_f32_packed(dev(logits)).item()))
        assert token == n // 3 and logit == 12345.0
    neg = np.full(100, -np.inf, dtype=F)
    assert ops.unpack_top1(int(ops.argmax_f32_packed(dev(neg)).item()))[0] == 0


def test_top_k_vs_oracle(cuda):
    rng = np.random.default_rng(12)
    logits = rng.normal(0, 1, 5000).astype(F)
    logits[100] = logits[4000] = 9.0
    logits[7] = -0.0
    for k in (1, 5, 16):
        tokens, values = ops.top_k_f32(dev(logits), k)
        rt, rv = oracle.top_k(logits, k)
        assert np.array_equal(host(tokens).astype(np.uint32), rt) and np.array_equal(host(values), rv)
    with pytest.raises(KmllError):
        ops.top_k_f32(dev(logits), 17)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_thread_two_devices(cuda):
    """The shared-memory opt-in of a kernel is per device: a thread that moves to a second GPU must get the same results
    there (the large-shared-memory kernels would fail to launch without it)."""
    rng = np.random.default_rng(21)
    w_host = rng.normal(0, 0.02, (512, 4096)).astype(F)
    packed, gs = oracle.w4_quantize(w_host)
    x = rng.normal(0, 1, 4096).astype(F)
    ref = oracle.w4_matvec(packed, gs, x)
    xb = rng.normal(0, 1, (16, 4096)).astype(F)
    refb = oracle.w4_linear_batched(xb, packed, gs)
    try:
        for device in (0, 1, 0):
            torch.cuda.set_device(device)
            w = ops.DeviceW4G128Matrix(torch.from_numpy(packed).cuda(), torch.from_numpy(gs.view(np.int16)).cuda().view(torch.float16), 512, 4096)
            assert_close(host(ops.linear(torch.from_numpy(x).cuda(), w)), ref, 4096, f"device {device}")
            p = ops.DeviceW4PMatrix.from_canonical(w)
            assert_close(host(ops.linear(torch.from_numpy(x).cuda(), p)), ref, 4096, f"prepared, device {device}")
            ws = ops.linear_batched_workspace(16, 4096)
            got = host(ops.linear_batched(torch.from_numpy(xb).cuda(), w, 16, 4096, 512, workspace=ws))
            assert float(np.max(np.abs(got - refb))) <= 1e-4 * np.sqrt(4096)
    finally:
        torch.cuda.set_device(0)
