"""Seeded synthetic tensors in the reference's in-memory layouts.

Real checkpoints are not available, so every test and benchmark input is generated here:
MLX 4-bit words with bf16-valued scales/biases, GGUF Q8_0 / Q4_K block streams, FP8 E4M3
bytes with per-row scales, and bf16- or f32-valued activations.  One seed per tensor; the
generator is numpy's Philox, whose stream is stable across numpy versions.
"""
import zlib

import numpy as np

F = np.float32


def rng(*key):
    """Generator keyed by (config id, tensor name, ...)."""
    seed = zlib.crc32(repr(key).encode()) | (len(key) << 32)
    return np.random.Generator(np.random.Philox(seed))


def bf16_round(a):
    """Round f32 to the nearest bf16 (ties to even) and widen back; the result is exact in f32."""
    b = np.ascontiguousarray(a, dtype=F).view(np.uint32)
    r = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(F)


def mlx_weight(key, out_dim, in_dim, gs=64):
    """uint32 words of 8 uniform nibbles; scale = bf16(|N(0,1)|*0.02 + 1e-3); bias = bf16(-8*scale)."""
    g = rng("mlx", key, out_dim, in_dim, gs)
    w = g.integers(0, 2**32, size=out_dim * (in_dim // 8), dtype=np.uint32)
    n = out_dim * (in_dim // gs)
    scales = bf16_round(np.abs(g.standard_normal(n, dtype=F)) * F(0.02) + F(1e-3))
    biases = bf16_round(F(-8) * scales)
    return w, scales, biases


def activations(key, n, bf16=True):
    x = rng("x", key, n).standard_normal(n, dtype=F)
    return bf16_round(x) if bf16 else x


def q8_0_matrix(key, out_dim, in_dim):
    """34-byte blocks: f16 d ~ U(0.001,0.02), 32 int8 ~ U[-127,127]."""
    g = rng("q8_0", key, out_dim, in_dim)
    nb = out_dim * (in_dim // 32)
    raw = np.empty((nb, 34), dtype=np.uint8)
    raw[:, 0:2] = g.uniform(0.001, 0.02, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    raw[:, 2:] = g.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    return raw.reshape(-1)


def q4k_matrix(key, out_dim, in_dim):
    """144-byte super-blocks: f16 d, dmin ~ U(0.001,0.02); 12 scale bytes and 128 quant bytes uniform bits."""
    g = rng("q4_k", key, out_dim, in_dim)
    nb = out_dim * (in_dim // 256)
    raw = np.empty((nb, 144), dtype=np.uint8)
    raw[:, 0:4] = g.uniform(0.001, 0.02, (nb, 2)).astype(np.float16).view(np.uint8).reshape(nb, 4)
    raw[:, 4:] = g.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    return raw.reshape(-1)


def q5k_matrix(key, out_dim, in_dim):
    """176-byte super-blocks: f16 d, dmin ~ U(0.001,0.02); 12 scale bytes, 32 fifth-bit bytes and 128 nibble bytes uniform bits."""
    g = rng("q5_k", key, out_dim, in_dim)
    nb = out_dim * (in_dim // 256)
    raw = np.empty((nb, 176), dtype=np.uint8)
    raw[:, 0:4] = g.uniform(0.001, 0.02, (nb, 2)).astype(np.float16).view(np.uint8).reshape(nb, 4)
    raw[:, 4:] = g.integers(0, 256, size=(nb, 172), dtype=np.uint8)
    return raw.reshape(-1)


def q6k_matrix(key, out_dim, in_dim):
    """210-byte super-blocks: 128 nibble bytes and 64 two-bit bytes uniform bits, 16 int8 scales ~ U[-127,127],
    f16 d ~ U(0.0005,0.005)."""
    g = rng("q6_k", key, out_dim, in_dim)
    nb = out_dim * (in_dim // 256)
    raw = np.empty((nb, 210), dtype=np.uint8)
    raw[:, 0:192] = g.integers(0, 256, size=(nb, 192), dtype=np.uint8)
    raw[:, 192:208] = g.integers(-127, 128, size=(nb, 16), dtype=np.int8).view(np.uint8)
    raw[:, 208:210] = g.uniform(0.0005, 0.005, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return raw.reshape(-1)


def gptq_weight(key, out_dim, in_dim, gs=128, act_order=False, f16_scales=True):
    """GPTQ symmetric INT4 in checkpoint layout: qweight [in/8][out] int32 of uniform nibbles, scales
    [in/gs][out] ~ U(0.002,0.02) (rounded to f16 as checkpoints store them unless f16_scales is False),
    g_idx = i // gs, or under act_order that pattern scattered by a random permutation of the inputs."""
    g = rng("gptq", key, out_dim, in_dim, gs, act_order)
    qw = g.integers(0, 2 ** 32, size=(in_dim // 8) * out_dim, dtype=np.uint64).astype(np.uint32).view(np.int32)
    sc = g.uniform(0.002, 0.02, (in_dim // gs) * out_dim).astype(np.float32)
    if f16_scales:
        sc = sc.astype(np.float16).astype(np.float32)
    gidx = (np.arange(in_dim) // gs).astype(np.int32)
    if act_order:
        gidx = gidx[g.permutation(in_dim)]
    return qw, gidx, sc


def e4m3_table():
    """Value of every E4M3FN code (bias 7, subnormals, 0x7f/0xff NaN)."""
    t = np.zeros(256, dtype=F)
    for c in range(256):
        e, m = (c >> 3) & 0xF, c & 7
        if e == 0:
            v = m / 8.0 * 2.0 ** -6
        elif e == 0xF and m == 7:
            v = float("nan")
        else:
            v = (1 + m / 8.0) * 2.0 ** (e - 7)
        t[c] = -v if c & 0x80 else v
    return t


def e4m3_encode(a):
    """Nearest finite E4M3FN code of each value (never a NaN code)."""
    t = e4m3_table()
    codes = np.array([c for c in range(256) if not np.isnan(t[c]) and c != 0x80], dtype=np.uint8)
    order = np.argsort(t[codes], kind="stable")
    codes, vals = codes[order], t[codes][order]
    a = np.clip(np.asarray(a, dtype=F), -448, 448)
    hi = np.clip(np.searchsorted(vals, a), 1, len(vals) - 1)
    lo = hi - 1
    pick_hi = (vals[hi] - a) < (a - vals[lo])
    return np.where(pick_hi, codes[hi], codes[lo]).astype(np.uint8)


def fp8_linear(key, out_dim, in_dim, bias=False):
    """E4M3 bytes of clip(N(0,1), ±448); row scale ~ U(0.5,2)/sqrt(in_dim); optional N(0,1) bias."""
    g = rng("fp8", key, out_dim, in_dim)
    w = e4m3_encode(g.standard_normal(out_dim * in_dim, dtype=F))
    scale = (g.uniform(0.5, 2.0, out_dim) / np.sqrt(in_dim)).astype(F)
    b = g.standard_normal(out_dim, dtype=F) if bias else None
    return w, scale, b


def rel_err(got, ref):
    """max_i |got-ref| / max(|ref_i|, 1e-3*max|ref|): rows that cancel to ~0 are floored."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    floor = 1e-3 * np.max(np.abs(ref)) if ref.size else 0.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), max(floor, 1e-30)))) if ref.size else 0.0
