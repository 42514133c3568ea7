"""W4-G128 in the prepared layout: the re-ordering is checked byte for byte against a numpy restatement of its
definition, and every operator over prepared weights against the CPU oracle working on the canonical arrays."""
import numpy as np
import pytest
import torch

import oracle
from kmll_b200 import ops
from test_ops_gpu import F, assert_close, bf16_dev, dev, host, w4_weight

pytestmark = pytest.mark.gpu
REC = 2112


def nibbles(packed, cols):
    out = np.empty((packed.shape[0], cols), dtype=np.uint8)
    out[:, 0::2] = packed & 15
    out[:, 1::2] = packed >> 4
    return out


def prepare_ref(packed_a, gs_a, rows, cols, packed_b=None, gs_b=None):
    """Definition of the prepared layout: unit u, group grp -> 2112 bytes; byte (i, l, a, e) of the first 2048 holds
    row pair g + 8 (a & 1) and column 32 t + 8 i + 4 (a >> 1) + e of the group (g = l >> 2, t = l & 3): high nibble
    two's complement q of the A row, low nibble q + 8 of the B row; then (g, which) -> scales of rows g, g + 8."""
    pair = packed_b is not None
    ng = cols // 128
    units = (rows + 15) // 16 if pair else (rows + 31) // 32
    na = nibbles(packed_a, cols)
    nb = nibbles(packed_b, cols) if pair else na
    sa, sb = gs_a, (gs_b if pair else gs_a)
    pad_rows = units * 32
    def padded(n, s):
        n2 = np.full((pad_rows, cols), 8, dtype=np.uint8)
        n2[:n.shape[0]] = n
        s2 = np.zeros((pad_rows, ng), dtype=np.uint16)
        s2[:s.shape[0]] = s
        return n2, s2
    na, sa = padded(na, sa)
    nb, sb = padded(nb, sb)
    out = np.zeros((units, ng, REC), dtype=np.uint8)
    i, l, a, e = np.meshgrid(np.arange(4), np.arange(32), np.arange(4), np.arange(4), indexing="ij")
    g, t = l >> 2, l & 3
    rp = g + 8 * (a & 1)
    c = t * 32 + i * 8 + (a >> 1) * 4 + e
    for u in range(units):
        row_a = (16 * u if pair else 32 * u) + rp
        row_b = (16 * u if pair else 32 * u + 16) + rp
        for grp in range(ng):
            qa = (na[row_a, grp * 128 + c].astype(np.int16) - 8) & 15
            byte = (qa << 4) | nb[row_b, grp * 128 + c]
            out[u, grp, :2048] = byte.astype(np.uint8).reshape(-1)
            sc = np.zeros((8, 2, 2), dtype=np.uint16)
            for gg in range(8):
                ra, rb = (16 * u if pair else 32 * u) + gg, (16 * u if pair else 32 * u + 16) + gg
                sc[gg, 0] = (sa[ra, grp], sa[ra + 8, grp])
                sc[gg, 1] = (sb[rb, grp], sb[rb + 8, grp])
            out[u, grp, 2048:] = sc.view(np.uint8).reshape(-1)
    return out.reshape(-1)


@pytest.mark.parametrize("rows,cols", [(64, 256), (17, 128), (96, 384)])
def test_prepare_matches_its_definition(cuda, rows, cols):
    rng = np.random.default_rng(rows + cols)
    _, packed, gs, w = w4_weight(rng, rows, cols)
    p = ops.DeviceW4PMatrix.from_canonical(w)
    assert np.array_equal(host(p.prepared), prepare_ref(packed, gs, rows, cols))
    _, packed2, gs2, w2 = w4_weight(rng, rows, cols)
    pp = ops.DeviceW4PMatrix.from_gate_up(w, w2)
    assert np.array_equal(host(pp.prepared), prepare_ref(packed, gs, rows, cols, packed2, gs2))


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1024, 4096), (4096, 14336), (1000, 256), (17, 128), (896, 896), (4864, 896), (33, 16384)])
def test_linear_prepared_vs_oracle(cuda, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    _, packed, gs, w = w4_weight(rng, rows, cols)
    p = ops.DeviceW4PMatrix.from_canonical(w)
    x = rng.normal(0, 1, cols).astype(F)
    ref = oracle.w4_matvec(packed, gs, x)
    assert_close(host(ops.linear(dev(x), p)), ref, cols, f"w4p {rows}x{cols}")
    r = rng.normal(0, 1, rows).astype(F)
    assert_close(host(ops.linear_residual(dev(x), p, dev(r))), oracle.add(r, ref), cols, f"w4p residual {rows}x{cols}")


def test_prepared_linear_is_deterministic_and_handles_zero(cuda):
    rng = np.random.default_rng(6)
    _, _, _, w = w4_weight(rng, 4096, 4096)
    p = ops.DeviceW4PMatrix.from_canonical(w)
    x = dev(rng.normal(0, 1, 4096).astype(F))
    a = ops.linear(x, p).clone()
    for _ in range(3):
        assert torch.equal(a, ops.linear(x, p))
    assert torch.count_nonzero(ops.linear(torch.zeros(4096, device="cuda"), p)) == 0


@pytest.mark.parametrize("dim,q_rows,kv_rows,hidden", [(4096, 4096, 1024, 14336), (896, 896, 128, 4864), (256, 200, 40, 300)])
def test_fused_forms_prepared_vs_oracle(cuda, dim, q_rows, kv_rows, hidden):
    rng = np.random.default_rng(dim + hidden)
    eps = 1e-5
    x = rng.normal(0, 1, dim).astype(F)
    gamma = oracle.bf16_from_f32(rng.uniform(0.5, 1.5, dim).astype(F))
    normed = oracle.rmsnorm(x, gamma, eps)
    mats = {}
    for name, rows in (("q", q_rows), ("k", kv_rows), ("v", kv_rows), ("g", hidden), ("u", hidden)):
        _, packed, gs, w = w4_weight(rng, rows, dim)
        mats[name] = (packed, gs, w)
    pq, pk, pv = (ops.DeviceW4PMatrix.from_canonical(mats[n][2]) for n in "qkv")
    for norm in (True, False):
        xin = normed if norm else x
        q, k, v = ops.linear_triple(dev(x), pq, pk, pv, norm_weight=bf16_dev(gamma) if norm else None, eps=eps)
        for got, n in ((q, "q"), (k, "k"), (v, "v")):
            assert_close(host(got), oracle.w4_matvec(mats[n][0], mats[n][1], xin), dim, f"triple {n} norm={norm}")
        pair = ops.DeviceW4PMatrix.from_gate_up(mats["g"][2], mats["u"][2])
        act = ops.silu_gate_up(dev(x), pair, None, norm_weight=bf16_dev(gamma) if norm else None, eps=eps)
        ref = oracle.silu_mul(oracle.w4_matvec(mats["g"][0], mats["g"][1], xin), oracle.w4_matvec(mats["u"][0], mats["u"][1], xin))
        assert_close(host(act), ref, dim, f"silu gate/up norm={norm}")


@pytest.mark.parametrize("rows,cols", [(32000, 4096), (1000, 256), (5, 128), (151936, 896)])
def test_top1_prepared(cuda, rows, cols):
    rng = np.random.default_rng(rows + cols)
    _, packed, gs, w = w4_weight(rng, rows, cols)
    p = ops.DeviceW4PMatrix.from_canonical(w)
    x = rng.normal(0, 1, cols).astype(F)
    gamma = oracle.bf16_from_f32(np.ones(cols, dtype=F))
    logits = oracle.w4_matvec(packed, gs, oracle.rmsnorm(x, gamma, 1e-5))
    for _ in range(2):  # twice: the arrival counter must be back at zero after a call
        packed_out = ops.linear_top1(dev(x), p, norm_weight=bf16_dev(gamma), eps=1e-5)
        tok, logit = ops.unpack_top1(int(packed_out.item()))
        best = float(np.max(logits))
        assert abs(logit - float(logits[tok])) <= 1e-4 * np.sqrt(cols)
        assert float(logits[tok]) >= best - 1e-4 * max(1.0, abs(best))
        second = float(np.partition(logits, -2)[-2]) if rows > 1 else -np.inf
        if best - second > 1e-3 * max(1.0, abs(best)):
            assert tok == int(np.argmax(logits))


def test_top1_prepared_tie_goes_to_the_lower_token(cuda):
    rng = np.random.default_rng(3)
    rows, cols = 640, 256
    w = rng.normal(0, 0.02, (rows, cols)).astype(F)
    w[500] = w[77]  # identical rows: identical logits
    w[77] *= 0  # make them the winners: plant a large row twice
    w[77, :] = 0.05
    w[500, :] = 0.05
    packed, gs = oracle.w4_quantize(w)
    m = ops.DeviceW4G128Matrix(dev(packed), dev(gs.view(np.int16), torch.float16), rows, cols)
    p = ops.DeviceW4PMatrix.from_canonical(m)
    x = np.abs(rng.normal(0, 1, cols)).astype(F)
    tok, _ = ops.unpack_top1(int(ops.linear_top1(dev(x), p).item()))
    assert tok == 77


@pytest.mark.parametrize("outlier", [1e3, 1e4, 1e6])
def test_activation_outlier_keeps_f32_accuracy(cuda, outlier):
    """One activation far above the rest (massive activations are normal in trained models): the digits are relative to
    the largest element, so the bound that matters is |error| <= 2^-29 max|x| sum|w| per output - far below what f32
    accumulation of the same products may lose (2^-24 of the largest product).  Checked against a float64 evaluation
    of the same quantized weights."""
    rng = np.random.default_rng(int(outlier))
    rows, cols = 256, 4096
    _, packed, gs, w = w4_weight(rng, rows, cols)
    p = ops.DeviceW4PMatrix.from_canonical(w)
    x = rng.normal(0, 1, cols).astype(F)
    x[1234] = F(outlier)
    wd = oracle.w4_dequant(packed, gs).astype(np.float64)
    exact = wd @ x.astype(np.float64)
    bound = 2.0 ** -29 * outlier * np.sum(np.abs(wd), axis=1) + 2.0 ** -22 * np.abs(wd) @ np.abs(x.astype(np.float64))
    for weight in (p, w):
        got = host(ops.linear(dev(x), weight)).astype(np.float64)
        if weight is w:  # canonical-layout kernel: three digits, 2^-22 of the largest element
            bound = bound + 2.0 ** -22 * outlier * np.sum(np.abs(wd), axis=1)
        assert np.all(np.abs(got - exact) <= bound), (outlier, float(np.max(np.abs(got - exact) / bound)))
