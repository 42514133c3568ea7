"""Generates tests/golden/kat.npz: known-answer vectors for the oracle and the CUDA kernels.

Everything here is computed by an INDEPENDENT pure-Python/numpy restatement (integer LCG in Python
ints, float32 numpy arithmetic applied in the reference's order) of the seeded stress cases that
kmll's own harness replays on the GPU (src/main.rs: gemm-stress :444-704, logit-stress :1614-1679)
plus the literal known-answer tests in crates/inference/src/model.rs:12216-12249.  It imports
neither the oracle library nor the product, so agreement between the three is meaningful.

Run:  python tests/golden/make_golden.py      (rewrites kat.npz next to this file)
"""
import os

import numpy as np

F = np.float32
MASK = (1 << 64) - 1


class Lcg:  # src/main.rs:4763-4769
    def __init__(self, seed):
        self.s = seed & MASK

    def next(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & MASK
        bucket = F((self.s >> 32) & 0xFFFF) / F(65535.0)
        return F(bucket * F(2.0) - F(1.0))

    def fill(self, n, scale=1.0):
        return np.array([self.next() * F(scale) for _ in range(n)], dtype=F)


def bf16_from_f32(x):  # crates/inference/src/dtypes.rs:153-157
    bits = np.asarray(x, dtype=F).view(np.uint32).astype(np.uint64)
    bias = ((bits >> 16) & 1) + 0x7FFF
    return (((bits + bias) & 0xFFFFFFFF) >> 16).astype(np.uint16)


def bf16_to_f32(b):  # crates/inference/src/dtypes.rs:148-150
    return (b.astype(np.uint32) << 16).view(F)


def round_half_away(v):
    return np.sign(v) * np.floor(np.abs(v) + F(0.5))


def rs_i8_quantize(w_bits):  # crates/inference/src/rowwise_scaled.rs:21-51
    w = bf16_to_f32(w_bits)
    max_abs = np.abs(w).max(axis=1)
    scales = np.where(max_abs == 0, F(1.0), max_abs / F(127.0)).astype(F)
    q = np.clip(round_half_away((w / scales[:, None]).astype(F)), -127, 127).astype(np.int8)
    return q, scales


def rs_i8_linear(x, q, scales):  # src/main.rs:4617-4637 == rowwise_scaled.rs:108-126 per row
    batch, k = x.shape
    n = q.shape[0]
    deq = (q.astype(F) * scales[:, None]).astype(F)
    out = np.zeros((batch, n), dtype=F)
    for kk in range(k):
        out = (out + (x[:, kk][:, None] * deq[:, kk][None, :]).astype(F)).astype(F)
    return out


def w4_quantize(w):
    rows, cols = w.shape
    g = w.reshape(rows, cols // 128, 128)
    max_abs = np.abs(g).max(axis=2)
    s32 = np.where(max_abs == 0, F(1.0), max_abs / F(7.0)).astype(F)
    s16 = s32.astype(np.float16)
    s = s16.astype(F)
    q = np.clip(round_half_away((g / s[:, :, None]).astype(F)), -7, 7).astype(np.int32) + 8
    q = q.reshape(rows, cols)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return packed, s16.view(np.uint16)


def w4_dequant(packed, gs_bits):
    rows, half = packed.shape
    q = np.empty((rows, half * 2), dtype=np.int32)
    q[:, 0::2] = packed & 0xF
    q[:, 1::2] = packed >> 4
    s = gs_bits.view(np.float16).astype(F)
    return ((q - 8).astype(F).reshape(rows, -1, 128) * s[:, :, None]).astype(F).reshape(rows, -1)


def seq_matvec(deq, x):
    out = np.zeros(deq.shape[0], dtype=F)
    for kk in range(deq.shape[1]):
        out = (out + (deq[:, kk] * x[kk]).astype(F)).astype(F)
    return out


def top1(logits):  # src/main.rs:4187-4201
    best_t, best_l = None, None
    for t, l in enumerate(logits):
        if best_t is None or l > best_l or (l == best_l and t < best_t):
            best_t, best_l = t, l
    return best_t, F(best_l)


def main():
    out = {}
    g = Lcg(0x1234)
    out["lcg_seed_0x1234_first8"] = np.array([g.next() for _ in range(8)], dtype=F)

    # crates/inference/src/model.rs:12227-12249 (cpu_rope_leaves_non_rotary_tail_unchanged)
    x = np.array([1, 2, 3, 4, 9, 10], dtype=F)
    c0, s0, c1, s1 = np.cos(F(0.5)), np.sin(F(0.5)), np.cos(F(1.0)), np.sin(F(1.0))
    out["rope_kat_input"] = x
    out["rope_kat_freqs"] = np.array([0.5, 1.0], dtype=F)
    out["rope_kat_expected"] = np.array([x[0] * c0 - x[2] * s0, x[1] * c1 - x[3] * s1, x[2] * c0 + x[0] * s0,
                                         x[3] * c1 + x[1] * s1, x[4], x[5]], dtype=F)
    # crates/inference/src/model.rs:12216-12225 (theta 1e4, rotary_dim 64): freqs[0] = 1, freqs[1] = 1/1e4^(2/64)
    out["rope_freq_kat"] = np.array([1.0, 1.0 / np.power(F(10000.0), F(2.0) / F(64.0))], dtype=F)

    # gemm-stress "linear-i8-scaled" cases, src/main.rs:463-472, seed :482 ^ 0x89 (:613-621)
    shapes = [(1, 1, 1), (3, 5, 7), (16, 16, 16), (17, 19, 23), (31, 33, 29), (64, 64, 64), (65, 33, 17), (128, 96, 64)]
    for idx, (m, n, k) in enumerate(shapes):
        seed = ((0 << 32) ^ idx ^ 0x9E3779B97F4A7C15) ^ 0x89
        lc = Lcg(seed)
        x = lc.fill(m * k).reshape(m, k)
        wb = bf16_from_f32(lc.fill(n * k)).reshape(n, k)
        q, sc = rs_i8_quantize(wb)
        out[f"gemm_i8_{idx}_shape"] = np.array([m, n, k])
        out[f"gemm_i8_{idx}_x"] = x
        out[f"gemm_i8_{idx}_wbits"] = wb
        out[f"gemm_i8_{idx}_q"] = q
        out[f"gemm_i8_{idx}_scales"] = sc
        out[f"gemm_i8_{idx}_y"] = rs_i8_linear(x, q, sc)

    # logit-stress scaled-i8 top-1 cases, src/main.rs:1646-1670 and :4123-4185
    top1_shapes = [(1, 1), (3, 5), (16, 16), (17, 31), (255, 64), (257, 65)]
    for idx, (rows, cols) in enumerate(top1_shapes):
        seed = (((0 << 32) ^ idx ^ 0xD1B54A32D192ED03) ^ 0x88)
        lc = Lcg(seed)
        x = lc.fill(cols)
        wf = lc.fill(rows * cols).reshape(rows, cols)
        wb = bf16_from_f32(wf)
        forced = 0 if rows == 1 else rows // 3
        wb[forced] = bf16_from_f32(np.where(x >= 0, F(4.0), F(-4.0)))
        q, sc = rs_i8_quantize(wb)
        logits = seq_matvec((q.astype(F) * sc[:, None]).astype(F), x)
        t, l = top1(logits)
        out[f"top1_i8_{idx}_shape"] = np.array([rows, cols])
        out[f"top1_i8_{idx}_x"] = x
        out[f"top1_i8_{idx}_wbits"] = wb
        out[f"top1_i8_{idx}_expected"] = np.array([t, np.array([l], dtype=F).view(np.uint32)[0]], dtype=np.uint64)

    # packed arg-max tie cases, src/main.rs:1633 and :4024-4054
    lengths = [1, 2, 3, 17, 255, 256, 257, 4096]
    for idx, n in enumerate(lengths):
        lc = Lcg((0 << 32) ^ idx ^ 0x6A09E667F3BCC909)
        logits = lc.fill(n, 10.0)
        exp = 0 if n == 1 else n // 3
        logits[exp] = F(12345.0)
        logits[n - 1] = F(12345.0)
        out[f"argmax_{idx}_logits"] = logits
        out[f"argmax_{idx}_expected"] = np.array([exp])

    # W4-G128 (format defined by this project; numpy restatement of the same per-group rule)
    rng = np.random.default_rng(7)
    w = rng.normal(0, 0.02, (24, 384)).astype(F)
    w[3, 128:256] = 0  # an all-zero group -> scale 1.0
    packed, gs = w4_quantize(w)
    xw = rng.normal(0, 1, 384).astype(F)
    out["w4_w"] = w
    out["w4_packed"] = packed
    out["w4_gscales"] = gs
    out["w4_dequant"] = w4_dequant(packed, gs)
    out["w4_x"] = xw
    out["w4_y"] = seq_matvec(out["w4_dequant"], xw)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kat.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
