"""Batched quantized linear on the tensor cores (tcgen05, caller-owned workspace) against the CPU oracle: the shapes of
the quantized GEMM sweep (M = 64, 256; (N, K) = (3584, 3584), (18944, 3584), (3584, 18944), a slice of (152064, 3584)),
prefill shapes of the Mistral-7B architecture, ragged sizes, both weight formats.  Same bounds as every other linear:
kmll's max_abs <= 1e-4 sqrt(K) (src/main.rs:4306) and 1e-4 relative to the largest output."""
import numpy as np
import pytest
import torch

import oracle
from kmll_b200 import ops
from test_ops_gpu import F, assert_close, dev, host, i8_weight, w4_weight

pytestmark = pytest.mark.gpu

SHAPES = [(5, 300, 512), (16, 4096, 4096), (33, 700, 4096), (64, 3584, 3584), (256, 3584, 3584), (64, 18944, 3584),
          (256, 3584, 18944), (64, 4736, 3584), (300, 1000, 256), (2048, 1024, 4096), (128, 4096, 14336)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_w4_vs_oracle(cuda, m, n, k):
    rng = np.random.default_rng(m + n + k)
    _, packed, gs, w = w4_weight(rng, n, k)
    x = rng.normal(0, 1, (m, k)).astype(F)
    x[0, :] *= F(1e-3)  # rows of very different magnitude: the scale is per row
    x[m - 1, :] *= F(1e3)
    ref = oracle.w4_linear_batched(x, packed, gs)
    ws = ops.linear_batched_workspace(m, k)
    assert ws is not None
    got = host(ops.linear_batched(dev(x), w, m, k, n, workspace=ws))
    assert_close(got[m // 2], ref[m // 2], k, f"w4 gemm {m}x{n}x{k} row {m // 2}")  # an unscaled row: kmll's absolute bound
    scale = np.maximum(np.max(np.abs(ref), axis=1, keepdims=True), 1e-30)
    assert float(np.max(np.abs(got - ref) / scale)) <= 1e-4  # every row, relative to its own largest output


# 5 to 32 rows of x: the persistent small-batch kernel (byte digits, s8 x s8 MMAs, group scale after the MMA); shapes
# with a ragged last row tile, one row tile only, split K (few row tiles) and no split (many), 16 and 32 row blocks
SMALL = [(5, 100, 128), (16, 1024, 4096), (17, 4097, 1024), (32, 14336, 4096), (16, 4096, 14336), (8, 18944, 3584), (24, 3584, 18944),
         (16, 32000, 4096)]


@pytest.mark.parametrize("m,n,k", SMALL)
def test_small_batch_w4_vs_oracle(cuda, m, n, k):
    rng = np.random.default_rng(m * 3 + n + k)
    _, packed, gs, w = w4_weight(rng, n, k)
    x = rng.normal(0, 1, (m, k)).astype(F)
    x[0, :] *= F(1e-3)
    x[m - 1, :] *= F(1e3)
    x[1, 7] = F(300.0)  # an activation far above the rest of its row
    ref = oracle.w4_linear_batched(x, packed, gs)
    ws = ops.linear_batched_workspace(m, k)
    r = rng.normal(0, 1, (m, n)).astype(F)
    got = host(ops.linear_batched(dev(x), w, m, k, n, workspace=ws))
    assert_close(got[m // 2], ref[m // 2], k, f"small batch {m}x{n}x{k} row {m // 2}")
    scale = np.maximum(np.max(np.abs(ref), axis=1, keepdims=True), 1e-30)
    assert float(np.max(np.abs(got - ref) / scale)) <= 1e-4
    again = host(ops.linear_batched(dev(x), w, m, k, n, workspace=ws))
    assert np.array_equal(got, again)  # split-K partials are added in split order: bit-identical from call to call
    del r


@pytest.mark.parametrize("m,n,k", [(5, 100, 256), (16, 1024, 4096), (17, 4097, 1024), (32, 14336, 4096), (16, 4096, 14336), (9, 700, 320),
                                   (16, 32000, 4096)])
def test_small_batch_i8_vs_oracle(cuda, m, n, k):
    """RS-I8, 5 to 32 rows of x: the int8 rows are MMA operands as they lie (K = 320: a partial last group)."""
    rng = np.random.default_rng(m * 5 + n + k)
    _, q, sc, w = i8_weight(rng, n, k)
    x = rng.normal(0, 1, (m, k)).astype(F)
    x[0, :] *= F(1e-3)
    x[m - 1, :] *= F(1e3)
    x[1, 7] = F(300.0)
    ref = oracle.rs_i8_linear_batched(x, q, sc)
    ws = ops.linear_batched_workspace(m, k)
    got = host(ops.linear_batched(dev(x), w, m, k, n, workspace=ws))
    assert_close(got[m // 2], ref[m // 2], k, f"small batch i8 {m}x{n}x{k} row {m // 2}")
    scale = np.maximum(np.max(np.abs(ref), axis=1, keepdims=True), 1e-30)
    assert float(np.max(np.abs(got - ref) / scale)) <= 1e-4
    assert np.array_equal(got, host(ops.linear_batched(dev(x), w, m, k, n, workspace=ws)))


@pytest.mark.parametrize("m,n,k", SHAPES[:5] + [(64, 1000, 896), (2048, 1024, 4096)])
def test_gemm_i8_vs_oracle(cuda, m, n, k):
    rng = np.random.default_rng(m + n + k + 1)
    _, q, sc, w = i8_weight(rng, n, k)
    x = rng.normal(0, 1, (m, k)).astype(F)
    ref = oracle.rs_i8_linear_batched(x, q, sc)
    got = host(ops.linear_batched(dev(x), w, m, k, n))
    scale = np.maximum(np.max(np.abs(ref), axis=1, keepdims=True), 1e-30)
    assert float(np.max(np.abs(got - ref) / scale)) <= 1e-4
    assert float(np.max(np.abs(got - ref))) <= 1e-4 * np.sqrt(k)


def test_gemm_qkv_and_is_deterministic(cuda):
    rng = np.random.default_rng(9)
    m, k = 96, 4096
    mats = [w4_weight(rng, rows, k) for rows in (4096, 1024, 1024)]
    x = rng.normal(0, 1, (m, k)).astype(F)
    xd = dev(x)
    q, kk, v = ops.linear_qkv_batched(xd, mats[0][3], mats[1][3], mats[2][3], m, k)
    for got, (_, packed, gs, _) in zip((q, kk, v), mats):
        ref = oracle.w4_linear_batched(x, packed, gs)
        assert float(np.max(np.abs(host(got) - ref))) <= 1e-4 * np.sqrt(k)
    q2, _, _ = ops.linear_qkv_batched(xd, mats[0][3], mats[1][3], mats[2][3], m, k)
    assert torch.equal(q, q2)


def test_small_batch_qkv_one_launch(cuda):
    """Three matrices of different heights share the digits of x and one persistent launch; RMSNorm fused in front."""
    rng = np.random.default_rng(11)
    m, k = 16, 4096
    mats = [w4_weight(rng, rows, k) for rows in (4096, 1000, 1000)]
    x = rng.normal(0, 1, (m, k)).astype(F)
    xd = dev(x)
    q, kk, v = ops.linear_qkv_batched(xd, mats[0][3], mats[1][3], mats[2][3], m, k)
    for got, (_, packed, gs, _) in zip((q, kk, v), mats):
        ref = oracle.w4_linear_batched(x, packed, gs)
        assert float(np.max(np.abs(host(got) - ref))) <= 1e-4 * np.sqrt(k)


def test_gemm_without_workspace_still_works(cuda):
    """No workspace: the call falls back to passes of the streaming kernel (4 rows of x each) and gives the same result."""
    rng = np.random.default_rng(10)
    m, n, k = 9, 256, 512
    _, packed, gs, w = w4_weight(rng, n, k)
    x = rng.normal(0, 1, (m, k)).astype(F)
    ref = oracle.w4_linear_batched(x, packed, gs)
    from kmll_b200.lib import check, load
    out = torch.empty((m, n), device="cuda")
    xd = dev(x)
    check(load().kmll_linear_batched_w4g128(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), w.packed.data_ptr(), w.gscales.data_ptr(), m, k,
                                            n, None, out.data_ptr()))
    assert float(np.max(np.abs(host(out) - ref))) <= 1e-4 * np.sqrt(k)
