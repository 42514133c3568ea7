"""Kernel micro-benchmark: times one quantized linear operator shape inside a CUDA graph over several
distinct weight matrices (so every launch streams cold weights from HBM) and prints achieved GB/s.

  python -m kmll_b200.microbench --op silu_gate_up --fmt w4 --rows 14336 --cols 4096
  python -m kmll_b200.microbench --op linear --fmt i8 --rows 32000 --cols 4096 --mats 8 --reps 10

ops: linear, qkv (RMSNorm + Q/K/V), linear_residual, silu_gate_up (RMSNorm prologue on), linear_top1, attention (rows =
context length).  fmt: i8 (RS-I8), w4 (W4-G128 canonical layout), w4p (W4-G128 prepared layout).  --suite decode runs every
batch-1 operator shape of a Mistral-7B-architecture decode step.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def _weight(fmt, rows, cols):
    if fmt == "w4p":
        return ops.DeviceW4PMatrix.from_canonical(_weight("w4", rows, cols))
    if fmt == "w4":
        return ops.DeviceW4G128Matrix(torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device="cuda"),
                                      (torch.rand((rows, cols // 128), device="cuda") * 0.01 + 0.001).half(), rows, cols)
    return ops.DeviceRowwiseScaledI8Matrix(torch.randint(-127, 128, (rows, cols), dtype=torch.int8, device="cuda"),
                                           torch.rand(rows, device="cuda") * 0.01, rows, cols)


def weight_bytes(fmt, rows, cols):
    return rows * cols * 0.515625 if fmt in ("w4", "w4p") else rows * cols + 4 * rows


# the batch-1 operators of one Mistral-7B-architecture decode step: (op, rows, cols, distinct matrices)
DECODE_SUITE = [("qkv", 6144, 4096, 16), ("linear_residual", 4096, 4096, 16), ("silu_gate_up", 14336, 4096, 8),
                ("linear_residual", 4096, 14336, 8), ("linear_top1", 32000, 4096, 4)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="linear", choices=["linear", "qkv", "linear_residual", "silu_gate_up", "linear_top1", "attention"])
    ap.add_argument("--fmt", default="w4", choices=["w4", "w4p", "i8"])
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--mats", type=int, default=8)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--suite", default="", choices=["", "decode"], help="decode: every batch-1 operator shape of a Mistral-7B-architecture step")
    ap.add_argument("--profile", action="store_true", help="bracket one graph replay with cudaProfilerStart/Stop")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    if a.suite == "decode":
        for op, rows, cols, mats in DECODE_SUITE:
            a.op, a.rows, a.cols, a.mats = op, rows, cols, mats
            run_one(a)
        return
    run_one(a)


def run_one(a):
    calls = []
    if a.op == "attention":
        n_heads, n_kv, hd = 32, 8, 128
        max_seq = ((a.rows + 63) // 64 + 4) * 64
        q = torch.randn(n_heads * hd, device="cuda")
        ws = ops.single_query_attention_workspace(n_heads, hd, max_seq)
        out = torch.empty(n_heads * hd, device="cuda")
        for _ in range(a.mats):
            kc, vc = torch.randn(max_seq * n_kv * hd, device="cuda"), torch.randn(max_seq * n_kv * hd, device="cuda")
            calls.append(lambda kc=kc, vc=vc: ops.single_query_attention(q, kc, vc, a.rows, max_seq, n_heads, n_kv, hd, out=out, workspace=ws))
        alg = 2 * a.rows * n_kv * hd * 4 + 2 * n_heads * hd * 4
    else:
        x = torch.randn(a.cols, device="cuda")
        gamma = torch.ones(a.cols, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(a.rows, device="cuda")
        res = torch.randn(a.rows, device="cuda")
        alg = weight_bytes(a.fmt, a.rows, a.cols) + 4 * a.cols + 4 * a.rows
        for _ in range(a.mats):
            w = _weight(a.fmt, a.rows, a.cols)
            if a.op == "linear":
                calls.append(lambda w=w: ops.linear(x, w, out=out))
            elif a.op == "qkv":  # RMSNorm + Q/K/V in one launch; rows = query rows + 2 x (rows / 6) KV rows (32q / 8kv heads)
                kv = a.rows // 6
                wk, wv = _weight(a.fmt, kv, a.cols), _weight(a.fmt, kv, a.cols)
                wq = _weight(a.fmt, a.rows - 2 * kv, a.cols)
                calls.append(lambda wq=wq, wk=wk, wv=wv: ops.linear_triple(x, wq, wk, wv, norm_weight=gamma, eps=1e-5))
            elif a.op == "linear_residual":
                calls.append(lambda w=w: ops.linear_residual(x, w, res, out=out))
            elif a.op == "linear_top1":
                calls.append(lambda w=w: ops.linear_top1(x, w))
            elif a.fmt == "w4p":
                pair = ops.DeviceW4PMatrix.from_gate_up(_weight("w4", a.rows, a.cols), _weight("w4", a.rows, a.cols))
                calls.append(lambda pair=pair: ops.silu_gate_up(x, pair, None, norm_weight=gamma, eps=1e-5, out=out))
            else:
                w2 = _weight(a.fmt, a.rows, a.cols)
                calls.append(lambda w=w, w2=w2: ops.silu_gate_up(x, w, w2, norm_weight=gamma, eps=1e-5, out=out))
        if a.op == "silu_gate_up":
            alg = 2 * weight_bytes(a.fmt, a.rows, a.cols) + 4 * a.cols + 2 * a.cols + 4 * a.rows
    for c in calls[:2]:
        c()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for c in calls:
            c()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    if a.profile:
        torch.cuda.profiler.start()
        graph.replay()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.reps * len(calls))
    print(json.dumps({"op": a.op, "fmt": a.fmt, "rows": a.rows, "cols": a.cols, "us_per_launch": us,
                      "algorithmic_bytes_per_launch": alg, "achieved_gbs": alg / us / 1e3}))


if __name__ == "__main__":
    main()
