"""CPU restatement of the reference's sequential decode loop (test infrastructure, not product).

Follows LlamaModel.runLegacyCPUToken (model/llama.go:899-1441) for the llama / qwen3 families at
the level of operations and their order:
  embed -> per layer [residual; RMSNorm; q,k,v projections; per-head QK RMSNorm (qwen3); RoPE on
  q and k; KV append; grouped-query attention; output projection; residual add; RMSNorm; gate, up
  projections; SiLU(gate)*up; down projection; residual add] -> final RMSNorm -> LM head -> argmax.
Per-op arithmetic follows the scalar Go definitions:
  RMSNorm   x = (x * inv) * w, inv = 1/sqrt(sum(x^2)/n + eps) in f32   (backends/simd/runtime/vec_amd64.s:280-375)
  RoPE      table = f32(cos/sin(f64(pos) / theta^(2i/d))); pairs (i, i + d/2): x0*c - x1*s, x0*s + x1*c
            (backends/simd/runtime/rope_freqs.go:11-30, backends/simd/kernels/rope.go:29-44)
  attention scores = (q . k_t) * scale; softmax with f64 exp; out = sum_t p_t v_t
            (backends/simd/runtime/attention.go:82-113, softmax.go:9-30)
  SiLU      x / (1 + f32(exp(f64(-x))))                                  (backends/simd/kernels/activation.go:15-24)
  argmax    first maximum wins                                            (model/inference_helpers.go:248-261)
The MLX projections go through the oracle's mlx.GemvTo restatement (bit-exact order).  What is NOT
reproduced is the lane order of the amd64 assembly reductions (Sdot, RMSNorm's sum of squares, the
LM-head row dots, which in the reference even depend on GOMAXPROCS): numpy's f32 reductions are
used instead, so logits agree with the reference binary to rounding, not bit for bit — parity of
the decode gate is pinned at the token level by the reference's frozen sequences
(model/decode_golden_test.go:94-130, reproduced in tests/test_oracle_decode.py), unpinned at the ulp level.
"""
import math
from dataclasses import dataclass

import numpy as np

F = np.float32


@dataclass
class DecodeConfig:
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    inter: int
    vocab: int
    eps: float = 1e-6
    theta: float = 1e6
    qk_norm: bool = True
    max_seq: int = 256


def rope_table(max_seq, head_dim, theta):
    """simd.BuildRoPEFreqs: [max_seq][head_dim/2][cos, sin], angles in f64, stored as f32."""
    half = head_dim // 2
    t = np.empty((max_seq, half, 2), dtype=F)
    for i in range(half):
        freq = 1.0 / math.pow(theta, float(2 * i) / float(head_dim))
        ang = np.arange(max_seq, dtype=np.float64) * freq
        t[:, i, 0] = np.cos(ang).astype(F)
        t[:, i, 1] = np.sin(ang).astype(F)
    return t


def rmsnorm(x, w, eps):
    x = np.asarray(x, dtype=F)
    ss = F(np.dot(x, x))
    inv = F(1.0) / F(np.sqrt(F(ss / F(x.size)) + F(eps)))
    return (x * inv) * w


def apply_rope(x, table, pos, heads, head_dim):
    """kernels.ApplyRoPE in place on x [heads*head_dim]."""
    half = head_dim // 2
    xv = x.reshape(heads, head_dim)
    c, s = table[pos, :, 0], table[pos, :, 1]
    x0, x1 = xv[:, :half].copy(), xv[:, half:].copy()
    xv[:, :half] = x0 * c - x1 * s
    xv[:, half:] = x0 * s + x1 * c


def softmax(v):
    mx = v.max()
    e = np.exp((v - mx).astype(np.float64)).astype(F)
    return e * (F(1.0) / e.sum(dtype=F))


def attention(q, kc, vc, seq, heads, kv_heads, head_dim, scale):
    """simd.GQAAttentionScaleInto: kc, vc are [seq][kv_heads*head_dim]."""
    out = np.zeros(heads * head_dim, dtype=F)
    per = heads // kv_heads
    K = kc[:seq].reshape(seq, kv_heads, head_dim)
    V = vc[:seq].reshape(seq, kv_heads, head_dim)
    for h in range(heads):
        kv = h // per
        scores = (K[:, kv, :] @ q[h * head_dim:(h + 1) * head_dim]) * F(scale)
        p = softmax(scores.astype(F))
        out[h * head_dim:(h + 1) * head_dim] = p @ V[:, kv, :]
    return out


def silu_mul(gate, up):
    g = np.asarray(gate, dtype=F)
    s = g / (F(1.0) + np.exp((-g).astype(np.float64)).astype(F))
    return s * up


def argmax_first(logits):
    return int(np.argmax(logits))  # numpy returns the first maximum, as ArgmaxLogits does


class DenseWeights:
    """f32 weights as the reference's small test models hold them (non-Large layout [in, out])."""

    def __init__(self, embed, final_norm, lm_head, layers):
        self.embed, self.final_norm, self.lm_head, self.layers = embed, final_norm, lm_head, layers

    def embedding(self, tok):
        return self.embed[tok].copy()

    def proj(self, l, name, x):
        return (x @ self.layers[l][name]).astype(F)

    def norm(self, l, name):
        return self.layers[l][name]

    def logits(self, h):
        return (self.lm_head @ h).astype(F)


class MLXWeights:
    """MLX 4-bit g64 projections (through the oracle's GemvTo), tied LM head used as embedding and,
    dequantised to f32, as the LM head (what the reference does for MLX checkpoints)."""

    def __init__(self, orc, cfg, layers, lm_head, final_norm, nthreads=8, gs=64):
        self.orc, self.cfg, self.layers, self.lm, self.final_norm = orc, cfg, layers, lm_head, final_norm
        self.nthreads, self.gs = nthreads, gs
        w, s, b = lm_head
        self.lm_dense = orc.mlx_dequant(w, s, b, cfg.vocab, cfg.hidden, gs, nthreads=nthreads).reshape(cfg.vocab, cfg.hidden)

    def embedding(self, tok):
        return self.lm_dense[tok].copy()

    def proj(self, l, name, x):
        (w, s, b), out_dim, in_dim = self.layers[l][name]
        return self.orc.mlx_gemv(x, w, s, b, out_dim, in_dim, self.gs, nthreads=self.nthreads)

    def norm(self, l, name):
        return self.layers[l][name]

    def logits(self, h):
        return self.lm_dense @ h


class OracleDecoder:
    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights
        self.table = rope_table(cfg.max_seq, cfg.head_dim, cfg.theta)
        kvd = cfg.kv_heads * cfg.head_dim
        self.kc = [np.zeros((cfg.max_seq, kvd), dtype=F) for _ in range(cfg.layers)]
        self.vc = [np.zeros((cfg.max_seq, kvd), dtype=F) for _ in range(cfg.layers)]
        self.scale = F(1.0 / math.sqrt(cfg.head_dim))

    def step(self, tok, pos, dump=None):
        """One token through the stack; returns the logits.  dump: optional list that receives
        (label, f32 array) after every layer, the labelled-tensor hook of the reference's loop
        (debugLayerHook, model/llama.go:933-1437)."""
        c, w = self.cfg, self.w
        hidden = w.embedding(tok).astype(F)
        for l in range(c.layers):
            residual = hidden.copy()
            hidden = rmsnorm(hidden, w.norm(l, "input_norm"), c.eps)
            q, k, v = w.proj(l, "q", hidden), w.proj(l, "k", hidden), w.proj(l, "v", hidden)
            if c.qk_norm:
                qn, kn = w.norm(l, "q_norm"), w.norm(l, "k_norm")
                q = np.concatenate([rmsnorm(q[h * c.head_dim:(h + 1) * c.head_dim], qn, c.eps) for h in range(c.heads)])
                k = np.concatenate([rmsnorm(k[h * c.head_dim:(h + 1) * c.head_dim], kn, c.eps) for h in range(c.kv_heads)])
            q, k = q.astype(F).copy(), k.astype(F).copy()
            apply_rope(q, self.table, pos, c.heads, c.head_dim)
            apply_rope(k, self.table, pos, c.kv_heads, c.head_dim)
            self.kc[l][pos], self.vc[l][pos] = k, v
            attn = attention(q, self.kc[l], self.vc[l], pos + 1, c.heads, c.kv_heads, c.head_dim, self.scale)
            hidden = residual + w.proj(l, "o", attn)
            residual = hidden.copy()
            hidden = rmsnorm(hidden, w.norm(l, "post_norm"), c.eps)
            act = silu_mul(w.proj(l, "gate", hidden), w.proj(l, "up", hidden))
            hidden = residual + w.proj(l, "down", act.astype(F))
            if dump is not None:
                dump.append(("layer%d.hidden" % l, hidden.astype(F).copy()))
        hidden = rmsnorm(hidden, w.final_norm, c.eps)
        return w.logits(hidden.astype(F))

    def generate(self, prompt, max_new, trace=None, all_logits=None):
        """LlamaModel.Generate with Tok == nil: prompt tokens one by one, then greedy tokens.
        all_logits: optional list that receives the logits of every position, prompt included."""
        out = list(prompt)
        logits = None
        for pos, tok in enumerate(prompt):
            logits = self.step(tok, pos)
            if all_logits is not None:
                all_logits.append(logits.copy())
        for i in range(max_new):
            nxt = argmax_first(logits)
            if trace is not None:
                top2 = np.partition(logits, -2)[-2:]
                trace.append((nxt, float(top2[1] - top2[0]), logits.copy() if trace is not None and getattr(trace, "keep_logits", False) else None))
            out.append(nxt)
            if i + 1 < max_new:
                logits = self.step(nxt, len(out) - 1)
                if all_logits is not None:
                    all_logits.append(logits.copy())
        return out
