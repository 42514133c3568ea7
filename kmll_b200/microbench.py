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
import os

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
    ap.add_argument("--op", default="linear", choices=["linear", "qkv", "linear_residual", "silu_gate_up", "linear_top1", "attention", "linear_batched",
                                                        "decode_batch", "prefill"])
    ap.add_argument("--batch", type=int, default=16, help="rows of x for --op linear_batched (5..32: small-batch kernel; more: tcgen05 f16 kernel)")
    ap.add_argument("--fmt", default="w4", choices=["w4", "w4p", "i8"])
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--mats", type=int, default=8)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--suite", default="", choices=["", "decode", "chain4096", "micro", "gemm_sweep"],
                    help="decode: every batch-1 operator shape of a Mistral-7B-architecture step; chain4096: 4096x4096 matvec + residual + "
                         "RMSNorm in both formats; micro: RMSNorm / SwiGLU / RoPE / row softmax over B in {1,16,64}, bf16; gemm_sweep: "
                         "M in {1,16,64,256,2048} x four (N,K), W4-G128")
    ap.add_argument("--shards", type=int, default=1, help="gemm_sweep: time one rank's share of every matrix when its N output rows are split over this "
                                                           "many GPUs (column-parallel: disjoint output blocks, no collective)")
    ap.add_argument("--profile", action="store_true", help="bracket one graph replay with cudaProfilerStart/Stop")
    ap.add_argument("--layers", type=int, default=2, help="decode_batch, prefill: layers of the Mistral-7B-shaped decoder (a small case for profiling)")
    ap.add_argument("--kv-bf16", action="store_true", help="decode_batch, prefill: keep the KV cache in bf16")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    if a.suite == "decode":
        for op, rows, cols, mats in DECODE_SUITE:
            a.op, a.rows, a.cols, a.mats = op, rows, cols, mats
            run_one(a)
        return
    if a.suite == "chain4096":
        return suite_chain4096(a.reps)
    if a.suite == "micro":
        return suite_micro(a.reps)
    if a.suite == "gemm_sweep":
        return suite_gemm_sweep(a.reps, shards=a.shards)
    run_one(a)


def peak_hbm_gbs():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, "fallback"


def time_graph(calls, reps):
    """Average microseconds per call: the calls are captured once each in one CUDA graph, replayed `reps` times."""
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))


def report(name, us, alg_bytes, extra=None, flops=None, cpu_us=None):
    hbm, tf, src = peak_hbm_gbs()
    line = {"op": name, "us": round(us, 2), "algorithmic_mb": round(alg_bytes / 1e6, 3), "gbs": round(alg_bytes / us / 1e3, 1),
            "frac_hbm": round(alg_bytes / us / 1e3 / hbm, 3), "peak": src}
    if flops is not None:
        line["tflops"] = round(flops / us / 1e6, 1)
        line["frac_tensor"] = round(flops / us / 1e6 / tf, 3)
    if cpu_us is not None:
        line["cpu_us"] = round(cpu_us, 1)
        line["cpu_gbs"] = round(alg_bytes / cpu_us / 1e3, 2)
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def suite_chain4096(reps, cpu=None):
    """y = dequant(W) x + r, h = RMSNorm(y): W 4096 x 4096 ~ N(0, 0.02) seed 0, x, r ~ N(0, 1), gamma ~ U(0.5, 1.5), eps 1e-6.
    `cpu(kind, **shape)`, when given, returns the microseconds a CPU implementation of the same operator takes."""
    rows = cols = 4096
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(cols, generator=gen, device="cuda")
    r = torch.randn(rows, generator=gen, device="cuda")
    gamma = (torch.rand(rows, generator=gen, device="cuda") + 0.5).to(torch.bfloat16)
    y, h = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    for fmt in ("i8", "w4", "w4p"):
        n = 24  # 24 distinct matrices: 200 to 400 MB, larger than L2
        calls = []
        for _ in range(n):
            w32 = torch.randn((rows, cols), generator=gen, device="cuda") * 0.02
            if fmt == "i8":
                w = ops.DeviceRowwiseScaledI8Matrix.from_bf16_rows_symmetric(ops.f32_to_bf16(w32))
            else:
                w = ops.DeviceW4G128Matrix.from_f32_rows(w32)
                if fmt == "w4p":
                    w = ops.DeviceW4PMatrix.from_canonical(w)
            calls.append(lambda w=w: (ops.linear_residual(x, w, r, out=y), ops.rmsnorm(y, gamma, 1e-6, out=h)))
        us = time_graph(calls, reps)
        alg = weight_bytes(fmt, rows, cols) + 4 * cols + 3 * 4 * rows + 2 * rows + 4 * rows
        report(f"matvec+residual then rmsnorm 4096x4096 [{fmt}] (2 launches)", us, alg,
               cpu_us=cpu("chain4096", fmt=fmt) if cpu else None)


def suite_micro(reps, cpu=None):
    """RMSNorm [B,4096], SwiGLU [B,11008], RoPE [B,32,128] theta 1e6 positions U[0,4096), row softmax [B*32,4096]; bf16, seed 1."""
    gen = torch.Generator(device="cuda").manual_seed(1)
    for B in (1, 16, 64):
        copies = max(2, int(300e6 // max(1, B * 32 * 4096 * 4)))  # distinct inputs so that together they exceed L2
        copies = min(copies, 64)

        def bf(*shape):
            return [torch.randn(shape, generator=gen, device="cuda").to(torch.bfloat16) for _ in range(copies)]

        xs, outs = bf(B, 4096), bf(B, 4096)
        gamma = (torch.rand(4096, generator=gen, device="cuda") + 0.5).to(torch.bfloat16)
        us = time_graph([lambda i=i: ops.rmsnorm_batched_bf16(xs[i], gamma, B, 4096, 1e-6, out=outs[i]) for i in range(copies)], reps)
        report(f"rmsnorm [{B},4096] bf16", us, B * 4096 * 4 + 2 * 4096, cpu_us=cpu("rmsnorm", batch=B) if cpu else None)
        g, u, o = bf(B, 11008), bf(B, 11008), bf(B, 11008)
        us = time_graph([lambda i=i: ops.silu_mul(g[i], u[i], out=o[i]) for i in range(copies)], reps)
        report(f"swiglu [{B},11008] bf16", us, 3 * B * 11008 * 2, cpu_us=cpu("swiglu", batch=B) if cpu else None)
        xr, orr = bf(B, 32, 128), bf(B, 32, 128)
        freqs = torch.tensor([1.0 / (1e6 ** (2 * i / 128)) for i in range(64)], dtype=torch.float32, device="cuda")
        pos = torch.randint(0, 4096, (B,), generator=gen, device="cuda", dtype=torch.int32)
        us = time_graph([lambda i=i: ops.apply_rope_batched_bf16(xr[i], freqs, pos, out=orr[i]) for i in range(copies)], reps)
        report(f"rope [{B},32,128] bf16", us, 2 * B * 32 * 128 * 2 + 4 * B, cpu_us=cpu("rope", batch=B) if cpu else None)
        sm_copies = max(2, min(copies, int(300e6 // (B * 32 * 4096 * 4))))
        sx = [torch.randn((B * 32, 4096), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(sm_copies)]
        so = [torch.empty_like(t) for t in sx]
        us = time_graph([lambda i=i: ops.softmax_rows(sx[i], out=so[i]) for i in range(sm_copies)], reps)
        report(f"softmax [{B * 32},4096] bf16", us, 2 * B * 32 * 4096 * 2, cpu_us=cpu("softmax", batch=B) if cpu else None)


def suite_gemm_sweep(reps, cpu=None, shards=1):
    """Quantized GEMM sweep, W4-G128 (seed 4): M in {1, 16, 64, 256, 2048} x (N, K) in {(3584, 3584), (18944, 3584),
    (3584, 18944), (152064, 3584)}; activations are bf16-valued N(0, 1) held as f32 (the operator API is f32)."""
    gen = torch.Generator(device="cuda").manual_seed(4)
    for n_full, k in ((3584, 3584), (18944, 3584), (3584, 18944), (152064, 3584)):
        n = n_full // shards
        wbytes = n * k * 0.515625
        for m in (1, 16, 64, 256, 2048):
            mats = 1 if m >= 256 else max(1, min(48, int(300e6 // wbytes) + 1))
            ws = [_weight("w4", n, k) for _ in range(mats)]
            x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16).float()
            out = torch.empty((m, n), device="cuda")
            if m == 1:
                if k <= 16384:
                    ws = [ops.DeviceW4PMatrix.from_canonical(w) for w in ws]
                calls = [lambda w=w: ops.linear(x[0], w, out=out[0]) for w in ws]
            else:
                scratch = ops.linear_batched_workspace(m, k)
                calls = [lambda w=w: ops.linear_batched(x, w, m, k, n, out=out, workspace=scratch) for w in ws]
            us = time_graph(calls, reps)
            report(f"gemm w4 M={m} N={n} K={k}", us, wbytes + 4 * m * k + 4 * m * n, flops=2.0 * m * n * k,
                   extra={"bound": "hbm" if m <= 16 else "tensor", "path": "stream kernel" if m == 1 else "tcgen05",
                          **({"shard_of": n_full, "shards": shards} if shards > 1 else {})},
                   cpu_us=cpu("gemm_w4", m=m, n=n, k=k) if cpu else None)
            del ws, calls
            torch.cuda.empty_cache()


def run_decode_batch(a):
    """--batch sequences in lockstep on a Mistral-7B-shaped decoder of --layers layers, each at context --rows: the whole
    step per layer (batched linears + attention over --batch caches), small enough for a profiler capture."""
    import numpy as np

    from . import runtime as rt
    ctx, B, steps = a.rows, a.batch, max(2, a.reps)
    cfg = rt.DecoderConfig(n_layers=a.layers, dim=4096, n_heads=32, n_kv_heads=8, head_dim=128, hidden_dim=14336, vocab_size=32000,
                           rope_theta=1.0e6, norm_eps=1.0e-5, max_seq_len=ctx + steps + 24,
                           format=rt.FORMAT_RS_I8 if a.fmt == "i8" else rt.FORMAT_W4G128, kv_bf16=a.kv_bf16)
    dec = rt.Decoder(cfg)
    dec.init_random(3, 0.02, False)
    dec.prefill(np.random.default_rng(3).integers(0, cfg.vocab_size, ctx))
    bd = rt.BatchDecoder(dec, B)
    for slot in range(B):
        bd.adopt(slot)
    bd.generate_greedy(3)
    torch.cuda.synchronize()
    if a.profile:
        torch.cuda.profiler.start()
        bd.enqueue_steps(1)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    bd.enqueue_steps(steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    kv_bytes = a.layers * B * 2 * (ctx + 3 + steps / 2) * 1024 * (2 if a.kv_bf16 else 4)
    print(json.dumps({"op": "decode_batch", "fmt": a.fmt, "layers": a.layers, "batch": B, "context": ctx, "kv_bf16": a.kv_bf16,
                      "ms_per_step": ms, "launches_per_step": bd.launches_per_step, "kv_bytes_per_step": kv_bytes}))
    bd.close()
    dec.close()


def run_prefill(a):
    """Batched prefill of a --rows-token prompt on the Mistral-7B-shaped decoder (--layers layers; 32 = the whole model):
    wall time of the call (host clock around a synchronised call, best of three warm calls)."""
    import time

    import numpy as np

    from . import runtime as rt
    n = a.rows
    cfg = rt.DecoderConfig(n_layers=a.layers, dim=4096, n_heads=32, n_kv_heads=8, head_dim=128, hidden_dim=14336, vocab_size=32000,
                           rope_theta=1.0e6, norm_eps=1.0e-5, max_seq_len=n + 64,
                           format=rt.FORMAT_RS_I8 if a.fmt == "i8" else rt.FORMAT_W4G128, kv_bf16=a.kv_bf16)
    dec = rt.Decoder(cfg)
    dec.init_random(3, 0.02, False)
    prompt = np.random.default_rng(3).integers(0, cfg.vocab_size, n)
    dec.prefill(prompt)  # allocates the scratch
    best = None
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dec.prefill(prompt)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    if a.profile:
        torch.cuda.profiler.start()
        dec.prefill(prompt)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    print(json.dumps({"op": "prefill", "fmt": a.fmt, "layers": a.layers, "prompt_len": n, "kv_bf16": a.kv_bf16, "seconds": best,
                      "tokens_per_s": n / best}))
    dec.close()


def run_one(a):
    if a.op == "decode_batch":
        return run_decode_batch(a)
    if a.op == "prefill":
        return run_prefill(a)
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
    elif a.op == "linear_batched":
        m = a.batch
        xb = torch.randn((m, a.cols), device="cuda")
        outb = torch.empty((m, a.rows), device="cuda")
        scratch = ops.linear_batched_workspace(m, a.cols)
        for _ in range(a.mats):
            w = _weight(a.fmt, a.rows, a.cols)
            calls.append(lambda w=w: ops.linear_batched(xb, w, m, a.cols, a.rows, out=outb, workspace=scratch))
        alg = weight_bytes(a.fmt, a.rows, a.cols) + 4 * m * a.cols + 4 * m * a.rows
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
    line = {"op": a.op, "fmt": a.fmt, "rows": a.rows, "cols": a.cols, "us_per_launch": us, "algorithmic_bytes_per_launch": alg,
            "achieved_gbs": alg / us / 1e3}
    if a.op == "linear_batched":
        line["batch"] = a.batch
        line["tflops"] = 2.0 * a.batch * a.rows * a.cols / us / 1e6
    print(json.dumps(line))


if __name__ == "__main__":
    main()
