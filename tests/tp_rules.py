"""Host-side rules of the tensor-parallel layout used by the decode runtime (pure Python, no GPU):
which slice of each weight a rank owns and how per-rank arg-max results are merged.  The C++
runtime applies the same rules on the device (copy_shard / merge_packed_kernel)."""
from __future__ import annotations

import struct

ROW_PARALLEL = ("wo", "w2")            # split the input (K) dimension; partial outputs are all-reduced
COLUMN_PARALLEL = ("wq", "wk", "wv", "w1", "w3", "output")  # split the output rows


def shard_bounds(total: int, rank: int, size: int) -> tuple[int, int]:
    if total % size:
        raise ValueError(f"{total} is not divisible by tp_size {size}")
    per = total // size
    return rank * per, (rank + 1) * per


def shard_shape(name: str, rows: int, cols: int, rank: int, size: int, group: int = 1):
    """((row_lo, row_hi), (col_lo, col_hi)) of the shard of a [rows, cols] weight."""
    if name in ROW_PARALLEL:
        lo, hi = shard_bounds(cols, rank, size)
        if lo % group or hi % group:
            raise ValueError(f"column shard [{lo}, {hi}) of {name} does not start on a multiple of {group}")
        return (0, rows), (lo, hi)
    if name in COLUMN_PARALLEL:
        return shard_bounds(rows, rank, size), (0, cols)
    raise ValueError(f"unknown weight {name}")


def unpack(packed: int) -> tuple[int, float]:
    token = packed & 0xFFFFFFFF
    logit = struct.unpack("<f", struct.pack("<I", (packed >> 32) & 0xFFFFFFFF))[0]
    return token, logit


def merge_top1(packed_per_rank) -> int:
    """Higher logit wins, equal logits -> lower token id (the arg-max rule of kmll,
    crates/inference/src/kernels/inference.rs:402-404).  An unsigned max over the packed words would
    be wrong: negative f32 bit patterns order backwards."""
    best = None
    for p in packed_per_rank:
        tok, logit = unpack(int(p))
        if best is None or logit > best[1] or (logit == best[1] and tok < best[0]):
            best = (tok, logit, int(p))
    return best[2]
