#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s at batch 1 on a Mistral-7B-architecture model with
4-bit group-128 weights (random-init, seed 3), prompt of 2048 random token ids, one rank per GPU.

  python bench.py --gpus 1 --steps K --warmup W          single GPU
  torchrun ... bench.py --gpus N --steps K --warmup W    tensor parallel over N GPUs (NCCL)
  python bench.py --impl reference ...                   the CPU restatement of kmll's own path on the host cores

A step is one decode token: RMSNorm+QKV, RoPE/KV write, attention over the whole context, output
projection, gated MLP, residuals, and the lm_head arg-max.  Prints one JSON line (rank 0).
Beside the headline value the line carries, on one GPU: `e2e` (per-token host API), `roofline` (the gate/up kernel timed
live), `step_roofline`, `prefill_s`, `batch16` (16 sequences in lockstep), `rs_i8` (kmll's own weight format, batch 1 and
16), `kv_bf16` (the same legs with the KV cache in bf16), `cpu_baseline` (the CPU port on the host cores) and `check`
(device status, token agreement between the loops, with batch 1 and - tensor parallel - with a single-GPU decoder).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT_LEN = 2048
SEED = 3
METRIC = "decode_tokens_per_s_batch1_mistral7b_arch_w4g128"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle port of kmll's CPU path (rowwise_scaled.rs:108-126 applied to W4-G128) timed on the
# host cores over whole decode steps of the same workload (all 32 layers and the lm_head, context 2048+).
# ---------------------------------------------------------------------------------------------------
def cpu_threads(requested: int) -> int:
    """Threads for the CPU arm: an explicit request, else every core this process may run on (a launcher may have
    set OMP_NUM_THREADS=1 for its ranks; the CPU arm is one process and takes the whole host)."""
    if requested > 0:
        return requested
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class CpuModel:
    """Mistral-7B-architecture decoder with W4-G128 weights on the host, built from the oracle's C functions
    (kmll's operator order, crates/inference/src/model.rs:10102-10300).  Weight bytes are random: throughput does
    not depend on their values."""

    def __init__(self, ctx: int):
        import numpy as np

        import oracle
        self.np, self.o = np, oracle
        rng = np.random.default_rng(SEED)
        self.dim, self.q, self.kv, self.hid, self.vocab, self.hd, self.layers_n = 4096, 4096, 1024, 14336, 32000, 128, 32
        block = rng.integers(0, 256, 1 << 22, dtype=np.uint8)  # 4 MiB of random nibble pairs, tiled into every tensor
        fblock = rng.normal(0, 1, 1 << 20).astype(np.float32)

        def tiled(src, n, dtype):
            out = np.empty(n, dtype=dtype)
            full = n // src.size
            if full:
                out[:full * src.size].reshape(full, src.size)[:] = src
            out[full * src.size:] = src[:n - full * src.size]
            return out

        def qw(rows, cols):
            return (tiled(block, rows * cols // 2, np.uint8).reshape(rows, cols // 2),
                    tiled(block[:1 << 16].astype(np.uint16) % 0x800 + 0x1C00, rows * (cols // 128), np.uint16).reshape(rows, cols // 128))

        def kv():
            return tiled(fblock, ctx * 8 * self.hd, np.float32).reshape(ctx, 8, self.hd)

        self.layers = [{"wq": qw(self.q, self.dim), "wk": qw(self.kv, self.dim), "wv": qw(self.kv, self.dim), "wo": qw(self.dim, self.q),
                        "w1": qw(self.hid, self.dim), "w3": qw(self.hid, self.dim), "w2": qw(self.dim, self.hid), "k": kv(), "v": kv()}
                       for _ in range(self.layers_n)]
        self.head = qw(self.vocab, self.dim)
        self.gamma = oracle.bf16_from_f32(np.ones(self.dim, dtype=np.float32))
        self.freqs = oracle.rope_frequencies(1e6, self.hd)
        self.embedding = oracle.bf16_from_f32(rng.normal(0, 0.02, (1024, self.dim)).astype(np.float32))

    def step(self, token: int, pos: int) -> int:
        o = self.o
        h = o.embedding(self.embedding, token % 1024)
        for L in self.layers:
            n = o.rmsnorm(h, self.gamma, 1e-5)
            qv, kvv, vv = o.w4_matvec(*L["wq"], n), o.w4_matvec(*L["wk"], n), o.w4_matvec(*L["wv"], n)
            qr = o.apply_rope(qv, self.freqs, pos, self.hd)
            L["k"][pos] = o.apply_rope(kvv, self.freqs, pos, self.hd).reshape(8, self.hd)
            L["v"][pos] = vv.reshape(8, self.hd)
            a = o.single_query_attention(qr, L["k"], L["v"], pos + 1, 32, 8, self.hd)
            h2 = o.add(h, o.w4_matvec(*L["wo"], a))
            n2 = o.rmsnorm(h2, self.gamma, 1e-5)
            act = o.silu_mul(o.w4_matvec(*L["w1"], n2), o.w4_matvec(*L["w3"], n2))
            h = o.add(h2, o.w4_matvec(*L["w2"], act))
        return o.unpack_top1(o.top1_packed(o.w4_matvec(*self.head, o.rmsnorm(h, self.gamma, 1e-5))))[0]


def cpu_sample(steps: int, warmup: int, threads: int, limit_s: float):
    """Whole decode steps on the host.  The number of timed steps is cut so that the run stays near limit_s."""
    import oracle
    oracle.set_threads(threads)
    cores = oracle.max_threads()
    model = CpuModel(PROMPT_LEN + warmup + steps + 2)
    pos, token = PROMPT_LEN, 1
    t0 = time.perf_counter()
    token = model.step(token, pos)
    pos += 1
    first = time.perf_counter() - t0
    for _ in range(max(0, min(warmup - 1, int(limit_s / 4 / max(first, 1e-3))))):
        token = model.step(token, pos)
        pos += 1
    run = max(1, min(steps, int(limit_s / max(first, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(run):
        token = model.step(token, pos)
        pos += 1
    seconds = time.perf_counter() - t0
    t_token = seconds / run
    return {"value": 1.0 / t_token, "unit": "tokens/s", "cores": cores, "kind": "port", "steps_run": run, "seconds_measured": seconds,
            "extrapolated": False,
            "sample": f"{run} whole decode steps (32 layers of W4-G128 matvecs, RMSNorm, RoPE, attention over {PROMPT_LEN}+ positions, SwiGLU, "
                      f"and the lm_head arg-max) in {seconds:.1f} s; oracle C code, OpenMP over rows, {cores} threads",
            "ms_per_token": t_token * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_sample(args.steps, args.warmup, cpu_threads(args.cpu_threads), 40.0)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "steps_run": cb["steps_run"], "warmup": args.warmup, "ms_per_step": cb["ms_per_token"], "seconds_measured": cb["seconds_measured"],
            "extrapolated": False, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 weights x f32 activations, f32 accumulate (CPU)", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def cpu_operator_us(kind, **shape):
    """Microseconds the CPU port of one micro-suite operator takes on every host core (the GEMM on a bounded slice of
    its output rows, scaled by the rows left out: its cost is linear in them)."""
    import numpy as np

    import oracle
    oracle.set_threads(cpu_threads(0))
    rng = np.random.default_rng(0)

    def timed(fn, min_s=0.3):
        fn()
        n, t0 = 0, time.perf_counter()
        while n == 0 or time.perf_counter() - t0 < min_s:
            fn()
            n += 1
        return (time.perf_counter() - t0) / n * 1e6

    if kind == "chain4096":
        rows = cols = 4096
        x, r = rng.normal(0, 1, cols).astype(np.float32), rng.normal(0, 1, rows).astype(np.float32)
        gamma = oracle.bf16_from_f32(rng.uniform(0.5, 1.5, rows).astype(np.float32))
        w = rng.normal(0, 0.02, (rows, cols)).astype(np.float32)
        if shape["fmt"] == "i8":
            q, sc = oracle.rs_i8_quantize(oracle.bf16_from_f32(w))
            return timed(lambda: oracle.rmsnorm(oracle.add(oracle.rs_i8_matvec(q, sc, x), r), gamma, 1e-6))
        pk, gs = oracle.w4_quantize(w)
        return timed(lambda: oracle.rmsnorm(oracle.add(oracle.w4_matvec(pk, gs, x), r), gamma, 1e-6))
    if kind == "gemm_w4":
        m, n, k = shape["m"], shape["n"], shape["k"]
        n_s = int(min(n, max(64, 2e10 // (2 * m * k)) // 64 * 64))
        pk = rng.integers(0, 256, (n_s, k // 2), dtype=np.uint8)
        gs = np.full((n_s, k // 128), 0x2000, dtype=np.uint16)  # f16 bits of 2^-7; timing only
        x = rng.normal(0, 1, (m, k)).astype(np.float32)
        if m == 1:
            return timed(lambda: oracle.w4_matvec(pk, gs, x[0])) * n / n_s
        return timed(lambda: oracle.w4_linear_batched(x, pk, gs)) * n / n_s
    B = shape["batch"]
    if kind == "rmsnorm":
        x, gamma = rng.normal(0, 1, (B, 4096)).astype(np.float32), oracle.bf16_from_f32(np.ones(4096, dtype=np.float32))
        return timed(lambda: [oracle.rmsnorm(x[b], gamma, 1e-6) for b in range(B)])
    if kind == "swiglu":
        g, u = (rng.normal(0, 1, B * 11008).astype(np.float32) for _ in range(2))
        return timed(lambda: oracle.silu_mul(g, u))
    if kind == "rope":
        x, f = rng.normal(0, 1, (B, 32 * 128)).astype(np.float32), oracle.rope_frequencies(1e6, 128)
        return timed(lambda: [oracle.apply_rope(x[b], f, 1234 + b, 128) for b in range(B)])
    if kind == "softmax":
        x = rng.normal(0, 1, (B * 32, 4096)).astype(np.float32)
        return timed(lambda: oracle.softmax_rows(x))
    raise ValueError(kind)


def run_suite(args):
    """The operator suites of kmll_b200.microbench with the CPU port of each operator timed beside it."""
    from kmll_b200 import microbench as mb
    cpu = None if args.no_cpu else cpu_operator_us
    {"chain4096": mb.suite_chain4096, "micro": mb.suite_micro, "gemm_sweep": mb.suite_gemm_sweep}[args.suite](args.suite_reps, cpu)


def workload_config(n_gpus):
    return {"workload": "Mistral-7B-architecture decode, batch 1, W4-G128 weights (random-init seed 3), prompt 2048 random token ids, "
                        "f32 KV cache, full causal attention (window 4096 never truncates)",
            "layers": 32, "dim": 4096, "heads": "32q/8kv x128", "hidden": 14336, "vocab": 32000, "prompt_len": PROMPT_LEN,
            "parallelism": f"tp{n_gpus}", "l2_policy": "inputs larger than L2 (3.67 GB of weights per step vs 126 MB L2)"}


def device_status() -> int:
    """0 unless a bounded wait inside a kernel gave up (1) or a tensor-parallel peer did not deliver in time (2)."""
    import ctypes as C

    from kmll_b200 import lib as klib
    status = C.c_int(-1)
    klib.check(klib.load().kmll_device_status(C.byref(status)))
    return int(status.value)


def same_greedy_run(tokens, logits, ref_tokens, ref_logits, rel_tol=1e-3):
    """(ok, step of a near-tie or None).  Two greedy runs of the same model agree when their tokens are identical, or
    differ for the first time at a step where both chosen logits lie within rel_tol of each other (a near-tie: either
    token is a faithful arg-max; later steps then legitimately diverge)."""
    for i, (a, b) in enumerate(zip(tokens, ref_tokens)):
        la, lb = float(logits[i]), float(ref_logits[i])
        if int(a) != int(b):
            return abs(la - lb) <= rel_tol * max(1.0, abs(lb)), i
        if abs(la - lb) > rel_tol * max(1.0, abs(lb)):
            return False, i
    return True, None


def run_ours(args):
    import numpy as np
    import torch

    from kmll_b200 import ops
    from kmll_b200 import runtime as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    K, W = args.steps, args.warmup
    max_seq = PROMPT_LEN + W + K + 16
    cfg = rt.DecoderConfig.mistral_7b(max_seq_len=max_seq, format=rt.FORMAT_W4G128, tp_rank=rank, tp_size=world)
    dec = rt.Decoder(cfg)
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(rt.Decoder.tp_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        dec.tp_init(bytes(uid.cpu().numpy().tobytes()))
    dec.init_random(SEED, 0.02, False)
    prompt = np.random.default_rng(SEED).integers(0, cfg.vocab_size, PROMPT_LEN)
    dec.prefill(prompt)  # untimed: the first prefill allocates its scratch and encodes its tensor maps
    torch.cuda.synchronize()
    prefill_s = None
    for _ in range(2):  # host wall clock around a synchronised call: the shorter of two (a host hiccup once read 0.8 s for 0.2)
        t0 = time.perf_counter()
        dec.prefill(prompt)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        prefill_s = dt if prefill_s is None else min(prefill_s, dt)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident loop: K graph replays, token fed back on the device -------------------------
    dec.enqueue_steps(W)
    start_pos = dec.position
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.profile == "decode":
        torch.cuda.profiler.start()
    e0.record()
    dec.enqueue_steps(K)
    e1.record()
    barrier()
    if args.profile == "decode":
        torch.cuda.profiler.stop()
    clocks = sampler.stop()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    # what the loop generated: entry i = (token, logit) consumed by step i since the prefill
    dev_tokens, dev_logits = dec.history(0, W + K)

    # ---- end to end through the public per-token API: token from host memory, packed result back ----
    first_packed = (int(dev_logits[:1].view(np.uint32)[0]) << 32) | int(dev_tokens[0])
    dec.rewind(start_pos - W)
    dec.set_pending(first_packed)
    packed = dec.next_top()
    host_tokens = []
    for _ in range(W):
        host_tokens.append(packed & 0xFFFFFFFF)
        packed = dec.step_host(packed & 0xFFFFFFFF)
    barrier()
    e0.record()
    for _ in range(K):
        host_tokens.append(packed & 0xFFFFFFFF)
        packed = dec.step_host(packed & 0xFFFFFFFF)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = dec.launches_per_step * K
    check = {"device_status": device_status(), "first_tokens": [int(t) for t in dev_tokens[W:W + 8]],
             "host_loop_tokens_match_device_loop": [int(t) for t in dev_tokens] == [int(t) for t in host_tokens]}

    # ---- batch 16 (one GPU): 16 sequences in lockstep share every weight read.  The prefilled sequence is adopted
    # into all 16 slots (identical prompts: throughput does not depend on the token values) -----------------------
    batch16 = None
    if world == 1 and not args.no_batch16:
        B = 16
        steps16 = max(2, min(K, 32))
        dec.rewind(start_pos - W)
        dec.set_pending(first_packed)
        bd = rt.BatchDecoder(dec, B)
        for slot in range(B):
            bd.adopt(slot)
        t16, l16 = bd.generate_greedy(3)  # warm-up steps, also a check: every slot holds the batch-1 sequence
        check["batch16_tokens_match_batch1"] = all(same_greedy_run(t16[slot], l16[slot], dev_tokens[:3], dev_logits[:3])[0] for slot in range(B))
        torch.cuda.synchronize()
        if args.profile == "batch16":
            torch.cuda.profiler.start()
        e0.record()
        bd.enqueue_steps(steps16)
        e1.record()
        torch.cuda.synchronize()
        if args.profile == "batch16":
            torch.cuda.profiler.stop()
        ms16 = e0.elapsed_time(e1) / steps16
        batch16 = {"metric": "decode_tokens_per_s_batch16_mistral7b_arch_w4g128", "value": B * 1e3 / ms16, "unit": "tokens/s", "batch": B,
                   "steps": steps16, "ms_per_step": ms16, "launches_per_step": bd.launches_per_step,
                   "context_at_start": start_pos - W + 3}
        bd.close()

    # ---- RS-I8 (the reference's own format) on the same architecture and prompt: 7.25 GB of weights per step ------
    rs_i8 = None
    if world == 1 and not args.no_rsi8:
        steps8 = max(8, min(K, 64))
        dec8 = rt.Decoder(rt.DecoderConfig.mistral_7b(max_seq_len=PROMPT_LEN + steps8 + 64, format=rt.FORMAT_RS_I8))
        dec8.init_random(SEED, 0.02, False)
        dec8.prefill(prompt)
        dec8.enqueue_steps(3)
        torch.cuda.synchronize()
        e0.record()
        dec8.enqueue_steps(steps8)
        e1.record()
        torch.cuda.synchronize()
        ms8 = e0.elapsed_time(e1) / steps8
        bytes8 = cfg.linear_elements() + 32 * 2 * (PROMPT_LEN + 3 + steps8 / 2) * 1024 * 4
        rs_i8 = {"metric": "decode_tokens_per_s_batch1_mistral7b_arch_rs_i8", "value": 1e3 / ms8, "unit": "tokens/s", "steps": steps8,
                 "ms_per_step": ms8, "launches_per_step": dec8.launches_per_step, "algorithmic_bytes_per_step": bytes8,
                 "frac_of_peak": bytes8 / ms8 / 1e6 / peaks()[0]}
        if not args.no_batch16:  # the same 16-sequence lockstep leg in the reference's own format
            first8, logits8 = dec8.history(0, 1)
            dec8.rewind(PROMPT_LEN)
            dec8.set_pending((int(logits8[:1].view(np.uint32)[0]) << 32) | int(first8[0]))
            bd8 = rt.BatchDecoder(dec8, 16)
            for slot in range(16):
                bd8.adopt(slot)
            bd8.generate_greedy(3)
            torch.cuda.synchronize()
            n16 = max(2, min(K, 16))
            e0.record()
            bd8.enqueue_steps(n16)
            e1.record()
            torch.cuda.synchronize()
            rs_i8["batch16"] = {"value": 16 * 1e3 / (e0.elapsed_time(e1) / n16), "unit": "tokens/s", "ms_per_step": e0.elapsed_time(e1) / n16,
                                "steps": n16, "launches_per_step": bd8.launches_per_step}
            bd8.close()
        dec8.close()

    # ---- the same W4-G128 decode with the KV cache kept in bf16 (an option kmll does not have: its cache is f32) -------
    kv_bf16 = None
    if world == 1 and not args.no_kvbf16:
        steps_h = max(8, min(K, 64))
        dech = rt.Decoder(rt.DecoderConfig.mistral_7b(max_seq_len=PROMPT_LEN + steps_h + 64, format=rt.FORMAT_W4G128, kv_bf16=True))
        dech.init_random(SEED, 0.02, False)
        dech.prefill(prompt)
        dech.enqueue_steps(3)
        torch.cuda.synchronize()
        e0.record()
        dech.enqueue_steps(steps_h)
        e1.record()
        torch.cuda.synchronize()
        ms_h = e0.elapsed_time(e1) / steps_h
        tok_h, log_h = dech.history(0, 3 + steps_h)
        n_same = 0
        while n_same < min(len(tok_h), len(dev_tokens)) and int(tok_h[n_same]) == int(dev_tokens[n_same]):
            n_same += 1
        kv_bf16 = {"metric": "decode_tokens_per_s_batch1_mistral7b_arch_w4g128_kv_bf16", "value": 1e3 / ms_h, "unit": "tokens/s",
                   "steps": steps_h, "ms_per_step": ms_h, "launches_per_step": dech.launches_per_step, "kv_cache_bytes": dech.kv_bytes,
                   "leading_tokens_equal_to_f32_cache_run": n_same, "of": min(len(tok_h), len(dev_tokens))}
        if not args.no_batch16:
            dech.rewind(PROMPT_LEN)
            dech.set_pending((int(log_h[:1].view(np.uint32)[0]) << 32) | int(tok_h[0]))
            bdh = rt.BatchDecoder(dech, 16)
            for slot in range(16):
                bdh.adopt(slot)
            bdh.generate_greedy(3)
            torch.cuda.synchronize()
            n16 = max(2, min(K, 16))
            e0.record()
            bdh.enqueue_steps(n16)
            e1.record()
            torch.cuda.synchronize()
            kv_bf16["batch16"] = {"value": 16 * 1e3 / (e0.elapsed_time(e1) / n16), "unit": "tokens/s", "ms_per_step": e0.elapsed_time(e1) / n16,
                                  "steps": n16, "launches_per_step": bdh.launches_per_step}
            bdh.close()
        dech.close()
        if not args.no_batch16 and not args.no_rsi8:  # the same 16-sequence leg with RS-I8 weights and the bf16 cache
            dec8h = rt.Decoder(rt.DecoderConfig.mistral_7b(max_seq_len=PROMPT_LEN + 64, format=rt.FORMAT_RS_I8, kv_bf16=True))
            dec8h.init_random(SEED, 0.02, False)
            dec8h.prefill(prompt)
            bd8h = rt.BatchDecoder(dec8h, 16)
            for slot in range(16):
                bd8h.adopt(slot)
            bd8h.generate_greedy(3)
            torch.cuda.synchronize()
            n16 = max(2, min(K, 16))
            e0.record()
            bd8h.enqueue_steps(n16)
            e1.record()
            torch.cuda.synchronize()
            kv_bf16["rs_i8_batch16"] = {"value": 16 * 1e3 / (e0.elapsed_time(e1) / n16), "unit": "tokens/s",
                                        "ms_per_step": e0.elapsed_time(e1) / n16, "steps": n16, "launches_per_step": bd8h.launches_per_step}
            bd8h.close()
            dec8h.close()

    # ---- roofline of the dominant kernel: the fused RMSNorm + gate/up + SiLU kernel over prepared-layout weights (the
    # one the decode step above launches 32 times), timed live over 8 layers' worth of distinct weights (1.9 GB per
    # pass) on the launching stream ----------------------------------------------------------------------
    roofline = None
    if world == 1:
        hid, dim = cfg.hidden_dim, cfg.dim
        n_mats = 8

        def canonical():
            return ops.DeviceW4G128Matrix(torch.randint(0, 256, (hid, dim // 2), dtype=torch.uint8, device="cuda"),
                                          (torch.rand((hid, dim // 128), device="cuda") * 0.01 + 0.001).half(), hid, dim)
        mats = [ops.DeviceW4PMatrix.from_gate_up(canonical(), canonical()) for _ in range(n_mats)]
        x = torch.randn(dim, device="cuda")
        gamma = torch.ones(dim, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(hid, device="cuda")
        for pair in mats[:2]:
            ops.silu_gate_up(x, pair, None, norm_weight=gamma, eps=1e-5, out=out)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for pair in mats:
                ops.silu_gate_up(x, pair, None, norm_weight=gamma, eps=1e-5, out=out)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        reps = 10
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        per_launch_us = e0.elapsed_time(e1) * 1e3 / (reps * n_mats)
        alg_bytes = 2 * hid * dim * 0.515625 + dim * 4 + dim * 2 + hid * 4
        peak, peak_src = peaks()
        achieved = alg_bytes / per_launch_us / 1e3
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                traffic = json.load(f).get("silu_gate_up_w4p_bytes_per_launch")
        roofline = {"bound": "hbm", "kernel": "linear_chain_kernel, one phase: RMSNorm + gate/up pair records + SiLU, 2x[14336x4096] W4-G128 prepared",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "of": peak_src, "traffic": traffic,
                    "algorithmic_bytes_per_launch": alg_bytes, "us_per_launch": per_launch_us}
        del mats, graph

    tok_s = K / (dev_ms / 1e3)
    e2e_tok_s = K / (e2e_ms / 1e3)
    weight_bytes = cfg.linear_elements() * 0.515625
    kv_bytes = 32 * 2 * (start_pos + K / 2) * 1024 * 4
    step_bytes = (weight_bytes + kv_bytes) / world
    peak, peak_src = peaks()
    line = {"metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": dev_ms / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 weights, s8 x u8 tensor-core MMA on four byte digits of the f32 activations (30-bit fixed point), s32 then f32 accumulate",
            "data": "synthetic", "config": workload_config(world), "clocks": clocks,
            "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8,
                    "ms_per_step": e2e_ms / K, "api": "kmll_decoder_step_host (token from pinned host memory, packed result read back, stream sync)"},
            "gpu_launches": launches, "launches_per_step": dec.launches_per_step,
            "step_roofline": {"algorithmic_bytes_per_step_per_gpu": step_bytes, "achieved_gbs_per_gpu": step_bytes / (dev_ms / K) / 1e6,
                              "frac_of_peak": step_bytes / (dev_ms / K) / 1e6 / peak, "peak": peak, "of": peak_src},
            "prefill_s": prefill_s, "context_at_start": start_pos}
    if roofline is not None:
        line["roofline"] = roofline
    if batch16 is not None:
        line["batch16"] = batch16
    if rs_i8 is not None:
        line["rs_i8"] = rs_i8
    if kv_bf16 is not None:
        line["kv_bf16"] = kv_bf16
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_sample(8, 1, cpu_threads(args.cpu_threads), 12.0)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    # ---- tensor parallel: rank 0 decodes the same prompt once more on a single-GPU decoder (same seed, so the same
    # quantized tensors; untimed) and the generated tokens must agree -----------------------------------------
    if world > 1:
        statuses = [None] * world
        dist.all_gather_object(statuses, check["device_status"])
        check["device_status"] = max(statuses)
        if rank == 0:
            ref = rt.Decoder(rt.DecoderConfig.mistral_7b(max_seq_len=max_seq, format=rt.FORMAT_W4G128))
            ref.init_random(SEED, 0.02, False)
            ref.prefill(prompt)
            ref_tokens, ref_logits = ref.generate_greedy(W + K)
            ref.close()
            same, where = same_greedy_run(dev_tokens, dev_logits, ref_tokens, ref_logits)
            check["tokens_match_tp1"] = same
            check["near_tie_at_step"] = where
    line["check"] = check
    ok = check["device_status"] == 0 and check["host_loop_tokens_match_device_loop"] and check.get("tokens_match_tp1", True)
    if rank == 0:
        print(json.dumps(line))
    dec.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("bench: the generated tokens failed their check (see \"check\" in the line above)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-threads", type=int, default=0, help="threads of the CPU arm (default: every core of the host)")
    ap.add_argument("--no-batch16", action="store_true", help="skip the batch-16 leg")
    ap.add_argument("--no-rsi8", action="store_true", help="skip the RS-I8 (the reference's own format) decode leg")
    ap.add_argument("--no-kvbf16", action="store_true", help="skip the leg that keeps the KV cache in bf16")
    ap.add_argument("--suite", default="", choices=["", "chain4096", "micro", "gemm_sweep"],
                    help="instead of the decode bench: one operator suite of kmll_b200.microbench, CPU port timed beside each line")
    ap.add_argument("--suite-reps", type=int, default=20)
    ap.add_argument("--profile", nargs="?", const="decode", default=None, choices=["decode", "batch16"],
                    help="bracket the timed batch-1 decode loop (default) or the timed batch-16 loop with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.suite:
        run_suite(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
