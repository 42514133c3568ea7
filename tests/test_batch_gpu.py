"""Lockstep batch decode: every sequence of the batch must produce the greedy tokens it produces alone in the
single-sequence decoder (which the runtime tests pin against the CPU oracle)."""
import numpy as np
import pytest

from kmll_b200 import runtime as rt
from kmll_b200.lib import KmllError

pytestmark = pytest.mark.gpu


def _cfg(fmt, **kw):
    base = dict(n_layers=2, dim=256, n_heads=4, n_kv_heads=2, head_dim=64, hidden_dim=512, vocab_size=640, rope_theta=1e6, norm_eps=1e-6,
                max_seq_len=48, format=fmt, fused=True)
    base.update(kw)
    return rt.DecoderConfig(**base)


@pytest.mark.parametrize("fmt", [rt.FORMAT_RS_I8, rt.FORMAT_W4G128])
@pytest.mark.parametrize("batch", [3, 16])
def test_batch_matches_single_sequence(cuda, fmt, batch):
    cfg = _cfg(fmt)
    dec = rt.Decoder(cfg)
    dec.init_random(7, 0.05, False)
    rng = np.random.default_rng(batch)
    prompts = [rng.integers(0, cfg.vocab_size, 10) for _ in range(batch)]
    n_steps = 6
    singles = []
    for p in prompts:
        dec.prefill(p)
        t, l = dec.generate_greedy(n_steps)
        singles.append((t.copy(), l.copy()))
    bd = rt.BatchDecoder(dec, batch)
    for slot, p in enumerate(prompts):
        dec.prefill(p)
        bd.adopt(slot)
    tokens, logits = bd.generate_greedy(n_steps)
    assert bd.position == len(prompts[0]) + n_steps
    assert bd.launches_per_step >= 5 * cfg.n_layers + 3  # the batched linear forms issue one or more kernels each
    for slot in range(batch):
        ref_t, ref_l = singles[slot]
        for i in range(n_steps):
            # the batched linear kernel rounds differently from the batch-1 kernel: identical tokens unless the step is a
            # near-tie, after which the sequence may legitimately diverge
            if int(tokens[slot, i]) != int(ref_t[i]):
                assert i > 0 and abs(float(logits[slot, i]) - float(ref_l[i])) <= 2e-3 * max(1.0, abs(float(ref_l[i]))), (slot, i)
                break
            assert abs(float(logits[slot, i]) - float(ref_l[i])) <= 2e-3 * max(1.0, abs(float(ref_l[i]))), (slot, i)
    bd.close()
    dec.close()


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_batch_gqa_head_dim_128(cuda, kv_bf16):
    cfg = _cfg(rt.FORMAT_W4G128, n_heads=8, n_kv_heads=2, head_dim=128, dim=256, max_seq_len=96, kv_bf16=kv_bf16)
    dec = rt.Decoder(cfg)
    dec.init_random(9, 0.05, False)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab_size, 70) for _ in range(4)]  # longer than one 64-position attention tile
    singles = []
    for p in prompts:
        dec.prefill(p)
        singles.append(dec.generate_greedy(5)[0].copy())
    bd = rt.BatchDecoder(dec, 4)
    for slot, p in enumerate(prompts):
        dec.prefill(p)
        bd.adopt(slot)
    tokens, _ = bd.generate_greedy(5)
    for slot in range(4):
        assert tokens[slot].tolist() == singles[slot].tolist()
    bd.close()
    dec.close()


@pytest.mark.parametrize("kv_bf16,window,head_dim,n_heads,n_kv", [(False, 0, 64, 8, 8), (True, 0, 64, 8, 8), (False, 90, 64, 8, 8), (True, 0, 128, 32, 8),
                                                                  (True, 150, 128, 16, 8), (False, 0, 128, 32, 8), (False, 0, 64, 16, 2),
                                                                  (True, 0, 128, 16, 2)])
def test_batch_attention_with_several_tiles_per_block(cuda, kv_bf16, window, head_dim, n_heads, n_kv):
    """16 sequences x 8 KV heads fill the GPU along the batch axis, so the attention plan gives every block a long slice
    of the sequence (here 256 positions: several 64-position tiles of the f32 kernel, several 16-position stages per
    warp of the bf16-cache kernel); with 200-token prompts the position being written lies deep inside its block's slice.
    The single-sequence runs they are compared with use one block per 64 positions: a different partition of the same
    sums.  Head dimensions 64 and 128 with 1, 2, 4 and 8 query heads per KV head cover the fragment layouts of the tensor-core
    kernel."""
    cfg = _cfg(rt.FORMAT_W4G128, n_heads=n_heads, n_kv_heads=n_kv, head_dim=head_dim, dim=512, max_seq_len=400, kv_bf16=kv_bf16,
               sliding_window=window)
    dec = rt.Decoder(cfg)
    dec.init_random(11, 0.05, False)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab_size, 200) for _ in range(16)]
    singles = []
    for p in prompts[:4]:
        dec.prefill(p)
        singles.append(dec.generate_greedy(6)[0].copy())
    bd = rt.BatchDecoder(dec, 16)
    for slot, p in enumerate(prompts):
        dec.prefill(p)
        bd.adopt(slot)
    tokens, _ = bd.generate_greedy(6)
    for slot in range(4):
        assert tokens[slot].tolist() == singles[slot].tolist()
    bd.close()
    dec.close()


def test_batch_errors(cuda):
    cfg = _cfg(rt.FORMAT_RS_I8)
    dec = rt.Decoder(cfg)
    dec.init_random(7, 0.05, False)
    with pytest.raises(KmllError):
        rt.BatchDecoder(dec, 17)
    bd = rt.BatchDecoder(dec, 2)
    with pytest.raises(KmllError):  # nothing prefilled yet
        bd.adopt(0)
    dec.prefill(np.arange(5))
    bd.adopt(0)
    with pytest.raises(KmllError):  # slot 1 is empty
        bd.generate_greedy(2)
    dec.prefill(np.arange(7))
    with pytest.raises(KmllError):  # different position
        bd.adopt(1)
    bd.close()
    dec.close()
