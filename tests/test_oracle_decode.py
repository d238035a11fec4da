"""Pins of the decode-loop restatement (oracle/decode.py) against the reference's own tests.

model/decode_golden_test.go:94-130 freezes the 12 tokens the sequential decode loop emits for small
synthetic models whose weights come from a linear congruential generator
(model/cpu_prefill_test.go:10-28, :33-100).  The models are rebuilt here by the same formula and the
restatement must emit the same tokens; that pins RMSNorm, QK-norm, RoPE, grouped-query attention,
SiLU and the residual order at the token level."""
import json
import os

import numpy as np
import pytest

from oracle import decode as od

F = np.float32


class LCG:
    """lcg.f of model/cpu_prefill_test.go:13-18, in uint32 / float32 arithmetic."""

    def __init__(self, seed):
        self.s = np.uint32(seed)

    def tensor(self, *shape):
        n = int(np.prod(shape))
        out = np.empty(n, dtype=F)
        s = int(self.s)
        for i in range(n):
            s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
            out[i] = (F(s >> 8) / F(1 << 24) - F(0.5)) * F(0.2)
        self.s = np.uint32(s)
        return out.reshape(shape)


def build_prefill_test_model(qk_norm):
    """buildPrefillTestModel(modelType, large=false, qkNorm, preFFN=false): generation order matters."""
    h, heads, kv, inter, vocab, layers = 16, 2, 1, 32, 32, 2
    hd = h // heads
    g = LCG(12345)
    embed, norm, lm = g.tensor(vocab, h), g.tensor(h), g.tensor(vocab, h)
    L = []
    for _ in range(layers):
        d = {"input_norm": g.tensor(h), "post_norm": g.tensor(h)}
        d["q"], d["k"], d["v"] = g.tensor(h, heads * hd), g.tensor(h, kv * hd), g.tensor(h, kv * hd)
        d["o"] = g.tensor(heads * hd, h)
        d["gate"], d["up"], d["down"] = g.tensor(h, inter), g.tensor(h, inter), g.tensor(inter, h)
        if qk_norm:
            d["q_norm"], d["k_norm"] = g.tensor(hd), g.tensor(hd)
        L.append(d)
    cfg = od.DecodeConfig(hidden=h, layers=layers, heads=heads, kv_heads=kv, head_dim=hd, inter=inter, vocab=vocab,
                          eps=1e-6, theta=10000.0, qk_norm=qk_norm, max_seq=64)
    return cfg, od.DenseWeights(embed, norm, lm, L)


GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_golden_tokens.json")))


@pytest.mark.parametrize("qk_norm,name", [(False, "llama_plain"), (True, "qwen3_qknorm")])
def test_decode_loop_golden_tokens(qk_norm, name):
    cfg, w = build_prefill_test_model(qk_norm)
    got = od.OracleDecoder(cfg, w).generate(GOLDEN["prompt"], 6)
    assert got == GOLDEN[name]


def test_rope_table_and_rotation():
    t = od.rope_table(8, 8, 10000.0)
    assert np.all(t[0, :, 0] == 1) and np.all(t[0, :, 1] == 0)            # position 0 rotates nothing
    assert t[3, 0, 0] == F(np.cos(3.0)) and t[3, 0, 1] == F(np.sin(3.0))   # pair 0 turns by pos radians
    assert t[5, 2, 0] == F(np.cos(5.0 / 10000.0 ** 0.5))
    x = np.arange(16, dtype=F)
    y = x.copy()
    od.apply_rope(y, t, 0, 2, 8)
    assert np.array_equal(x, y)
    od.apply_rope(y, t, 3, 2, 8)
    c, s = t[3, 1, 0], t[3, 1, 1]
    assert y[1] == x[1] * c - x[5] * s and y[5] == x[1] * s + x[5] * c     # pairs are (i, i + d/2)
    assert y[9] == x[9] * c - x[13] * s


def test_rmsnorm_attention_silu_closed_forms():
    x = np.full(8, 2.0, dtype=F)
    assert np.allclose(od.rmsnorm(x, np.full(8, 3.0, dtype=F), 0.0), 3.0)
    q = np.ones(4, dtype=F)
    kc = np.ones((3, 4), dtype=F)
    vc = np.stack([np.full(4, v, dtype=F) for v in (1.0, 2.0, 6.0)])
    # one position: the output is that position's value; equal scores: the mean of the values
    assert np.array_equal(od.attention(q, kc, vc, 1, 1, 1, 4, 0.5), vc[0])
    assert np.allclose(od.attention(q, kc, vc, 3, 1, 1, 4, 0.5), 3.0)
    g = np.array([0.0, 1.0, -1.0], dtype=F)
    assert np.allclose(od.silu_mul(g, np.full(3, 2.0, dtype=F)), 2 * g / (1 + np.exp(-g.astype(np.float64))), rtol=1e-6)
    assert od.argmax_first(np.array([1.0, 5.0, 5.0, 2.0], dtype=F)) == 1
