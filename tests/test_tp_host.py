"""CPU tests of the tensor-parallel path: two gloo ranks shard the weights the way the runtime does,
compute their partial results with the oracle, and meet in an all-reduce / all-gather; the result
must equal the single-rank oracle (bit-exact weights slices, f32 tolerance on the re-associated sum)."""
import os
import socket
import struct

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
import tp_rules as tp

F = np.float32


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _pack(logit, token):
    return (struct.unpack("<I", struct.pack("<f", logit))[0] << 32) | token


def _worker(rank, world, port, fmt, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)  # same seed on every rank: full tensors are identical, shards are slices
        dim, hid, vocab = 256, 512, 384
        x = rng.normal(0, 1, dim).astype(F)
        w1f, w2f, outf = (rng.normal(0, 0.05, s).astype(F) for s in ((hid, dim), (dim, hid), (vocab, dim)))
        if fmt == "w4":
            quant = lambda w: oracle.w4_quantize(w)
            matvec = lambda q, v: oracle.w4_matvec(q[0], q[1], v)
            group = 128
            cols_of = lambda q, lo, hi: (np.ascontiguousarray(q[0][:, lo // 2:hi // 2]), np.ascontiguousarray(q[1][:, lo // 128:hi // 128]))
        else:
            quant = lambda w: oracle.rs_i8_quantize(oracle.bf16_from_f32(w))
            matvec = lambda q, v: oracle.rs_i8_matvec(q[0], q[1], v)
            group = 64
            cols_of = lambda q, lo, hi: (np.ascontiguousarray(q[0][:, lo:hi]), q[1])  # row scales are replicated
        rows_of = lambda q, lo, hi: (np.ascontiguousarray(q[0][lo:hi]), np.ascontiguousarray(q[1][lo:hi]))
        w1, w2, wout = quant(w1f), quant(w2f), quant(outf)  # quantize BEFORE sharding
        # column-parallel up projection, row-parallel down projection, all-reduce of the partial sums
        (r0, r1), _ = tp.shard_shape("w1", hid, dim, rank, world)
        act_local = matvec(rows_of(w1, r0, r1), x)
        _, (c0, c1) = tp.shard_shape("w2", dim, hid, rank, world, group)
        partial = matvec(cols_of(w2, c0, c1), act_local)
        t = torch.from_numpy(partial.copy())
        dist.all_reduce(t)
        y = t.numpy()
        y_ref = matvec(w2, matvec(w1, x))
        # vocabulary-parallel arg-max: local packed result with global token ids, all-gather, deterministic merge
        (v0, v1), _ = tp.shard_shape("output", vocab, dim, rank, world)
        logits_local = matvec(rows_of(wout, v0, v1), x)
        tok, logit = oracle.unpack_top1(oracle.top1_packed(logits_local))
        mine = torch.tensor([_pack(logit, tok + v0)], dtype=torch.int64)
        gathered = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, mine)
        merged = tp.merge_top1([int(g.item()) & 0xFFFFFFFFFFFFFFFF for g in gathered])
        ref_tok, ref_logit = oracle.unpack_top1(oracle.top1_packed(matvec(wout, x)))
        if rank == 0:
            out.put((float(np.max(np.abs(y - y_ref))), float(np.max(np.abs(y_ref))), tp.unpack(merged), (ref_tok, ref_logit)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt", ["i8", "w4"])
def test_two_rank_tensor_parallel_matches_single_rank(fmt):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fmt, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    diff, scale, merged, ref = out.get(timeout=10)
    assert diff <= 1e-5 * max(scale, 1.0)
    assert merged[0] == ref[0] and merged[1] == ref[1]


def test_shard_rules_and_merge():
    assert tp.shard_bounds(4096, 3, 8) == (1536, 2048)
    with pytest.raises(ValueError):
        tp.shard_bounds(10, 0, 4)
    assert tp.shard_shape("wo", 4096, 4096, 1, 8, 128) == ((0, 4096), (512, 1024))
    assert tp.shard_shape("w2", 4096, 14336, 7, 8, 128) == ((0, 4096), (12544, 14336))
    with pytest.raises(ValueError):
        tp.shard_shape("w2", 64, 896, 1, 2, 128)  # 448 is not a multiple of the group size
    assert tp.shard_shape("wk", 1024, 4096, 2, 8) == ((256, 384), (0, 4096))
    # merge: negative logits must not win through their larger unsigned bit pattern; ties -> lower token
    a, b, c = _pack(-1.0, 5), _pack(-3.0, 2), _pack(-1.0, 9)
    assert tp.unpack(tp.merge_top1([b, c, a])) == (5, -1.0)
    assert max(a, b, c) == b  # what an unsigned max would have picked
