"""CPU oracle of the whole decoder forward, composed from the C oracle ops in kmll's own order
(single block: crates/inference/src/model.rs:8425-8467; FFN: :11658-11669; logits + top-1:
:10511-10657).  Weights are the quantized tensors downloaded from the device runtime, so the two
sides multiply exactly the same bytes."""
import numpy as np

import oracle
from kmll_b200 import runtime as rt

F = np.float32


class OracleDecoder:
    def __init__(self, cfg: rt.DecoderConfig, dec: rt.Decoder, freqs=None):
        self.cfg = cfg
        self.w4 = cfg.format == rt.FORMAT_W4G128
        g = dec.get_tensor
        self.layers = []
        for l in range(cfg.n_layers):
            self.layers.append({name: g(l, tid) for name, tid in (("attention_norm", rt.T_ATTENTION_NORM), ("wq", rt.T_WQ), ("wk", rt.T_WK),
                                                                   ("wv", rt.T_WV), ("wo", rt.T_WO), ("ffn_norm", rt.T_FFN_NORM),
                                                                   ("w1", rt.T_W1), ("w3", rt.T_W3), ("w2", rt.T_W2))})
        self.qk_norm = []
        for l in range(cfg.n_layers):
            try:
                self.qk_norm.append((g(l, rt.T_Q_NORM), g(l, rt.T_K_NORM)))
            except rt.KmllError:
                self.qk_norm.append(None)
        self.final_norm = g(-1, rt.T_FINAL_NORM)
        self.embedding = g(-1, rt.T_EMBEDDING)
        self.output = g(-1, rt.T_OUTPUT)
        kv = cfg.n_kv_heads * cfg.head_dim
        self.key = [np.zeros((cfg.max_seq_len, kv), dtype=F) for _ in range(cfg.n_layers)]
        self.value = [np.zeros((cfg.max_seq_len, kv), dtype=F) for _ in range(cfg.n_layers)]
        self.freqs = oracle.rope_frequencies(cfg.rope_theta, cfg.rotary_dim or cfg.head_dim) if freqs is None else np.asarray(freqs, dtype=F)
        self.position = 0
        self.hidden = None

    def matvec(self, w, x):
        return oracle.w4_matvec(w[0], w[1], x) if self.w4 else oracle.rs_i8_matvec(w[0], w[1], x)

    def forward(self, token: int) -> np.ndarray:
        c = self.cfg
        pos = self.position
        hidden = oracle.embedding(self.embedding, token)
        for l, L in enumerate(self.layers):
            normed = oracle.rmsnorm(hidden, L["attention_norm"], c.norm_eps)
            q, k, v = self.matvec(L["wq"], normed), self.matvec(L["wk"], normed), self.matvec(L["wv"], normed)
            if self.qk_norm[l] is not None:  # per-head RMSNorm before RoPE (model.rs:10165-10194)
                hd = c.head_dim
                q = np.concatenate([oracle.rmsnorm(q[h * hd:(h + 1) * hd], self.qk_norm[l][0], c.norm_eps) for h in range(c.n_heads)])
                k = np.concatenate([oracle.rmsnorm(k[h * hd:(h + 1) * hd], self.qk_norm[l][1], c.norm_eps) for h in range(c.n_kv_heads)])
            q_rot = oracle.apply_rope(q, self.freqs, pos, c.head_dim)
            k_row = oracle.apply_rope(k, self.freqs, pos, c.head_dim)
            if c.kv_bf16:  # the cache keeps bf16: rows rounded to nearest-even once, when they are written
                k_row, v = oracle.bf16_to_f32(oracle.bf16_from_f32(k_row)), oracle.bf16_to_f32(oracle.bf16_from_f32(v))
            self.key[l][pos] = k_row
            self.value[l][pos] = v
            lo = max(0, pos + 1 - c.sliding_window) if c.sliding_window > 0 else 0  # sliding window: the last rows only
            attn = oracle.single_query_attention(q_rot, self.key[l][lo:pos + 1], self.value[l][lo:pos + 1], pos + 1 - lo, c.n_heads,
                                                 c.n_kv_heads, c.head_dim)
            hidden = oracle.add(hidden, self.matvec(L["wo"], attn))
            normed = oracle.rmsnorm(hidden, L["ffn_norm"], c.norm_eps)
            act = oracle.silu_mul(self.matvec(L["w1"], normed), self.matvec(L["w3"], normed))
            hidden = oracle.add(hidden, self.matvec(L["w2"], act))
        self.position += 1
        self.hidden = hidden
        return hidden

    def logits(self) -> np.ndarray:
        return self.matvec(self.output, oracle.rmsnorm(self.hidden, self.final_norm, self.cfg.norm_eps))

    def prefill(self, tokens):
        self.position = 0
        for t in tokens:
            self.forward(int(t))
        return self.logits()

    def generate_greedy(self, logits, n_steps):
        """Returns [(token, logit, margin)] - margin = gap between the best and second best logit."""
        out = []
        for _ in range(n_steps):
            token, logit = oracle.unpack_top1(oracle.top1_packed(logits))
            second = np.partition(logits, -2)[-2] if logits.size > 1 else -np.inf
            out.append((token, logit, float(logit - second)))
            self.forward(token)
            logits = self.logits()
        return out, logits
