"""GPU parity of the decode-step operations and of greedy decoding against the CPU restatement
(oracle/decode.py, pinned by the reference's frozen token sequences), through the C ABI.

Operations are compared within f32 rounding of the restatement; the decode gate is token identity
over the generated sequence on random-init models (the reference's gate for MLX checkpoints)."""
import numpy as np
import pytest

from gpu_util import F
from oracle import binding as orc
from oracle import decode as od

pytestmark = pytest.mark.gpu


def test_add_rmsnorm(gpu, pkg):
    g = pkg.synth.rng("rms")
    n = 1024
    a, b, w = (g.standard_normal(n, dtype=F) for _ in range(3))
    A, B, W = gpu.from_numpy(a), gpu.from_numpy(b), gpu.from_numpy(w)
    hid, nrm = gpu.Malloc(n), gpu.Malloc(n)
    gpu.AddRMSNorm(hid, nrm, A, B, W, n, 1, 1e-6)
    gpu.Sync()
    assert np.array_equal(hid.Download(), a + b)
    assert np.allclose(nrm.Download(), od.rmsnorm(a + b, w, 1e-6), rtol=2e-6, atol=1e-7)
    gpu.AddRMSNorm(None, nrm, A, None, W, n, 1, 1e-6)      # no residual, no hidden output
    gpu.Sync()
    assert np.allclose(nrm.Download(), od.rmsnorm(a, w, 1e-6), rtol=2e-6, atol=1e-7)
    gpu.AddRMSNorm(A, nrm, A, B, W, n, 1, 1e-6)            # in place on the residual stream
    gpu.Sync()
    assert np.array_equal(A.Download(), a + b)
    assert np.allclose(nrm.Download(), od.rmsnorm(a + b, w, 1e-6), rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("heads,kv_heads,head_dim,qk_norm,max_seq,steps", [
    (16, 8, 128, True, 96, 70), (4, 2, 64, False, 96, 70), (8, 8, 128, True, 96, 70), (4, 1, 256, True, 96, 40),
    (8, 4, 128, True, 1024, 600),     # long cache: CTAs of 32 warps, the positions split over several per head
    (8, 4, 128, True, 256, 250),      # the longest cache the 4-warp CTAs take (16 splits of 16 positions)
    (4, 2, 64, True, 272, 270),       # the shortest the 32-warp CTAs take
])
def test_qk_norm_rope_append_and_attention(gpu, pkg, heads, kv_heads, head_dim, qk_norm, max_seq, steps, fused):
    g = pkg.synth.rng("attn", heads, head_dim)
    kvd = kv_heads * head_dim
    table = od.rope_table(max_seq, head_dim, 1e6)
    T = gpu.from_numpy(table.reshape(-1))
    qn = g.standard_normal(head_dim, dtype=F) if qk_norm else None
    kn = g.standard_normal(head_dim, dtype=F) if qk_norm else None
    QN = gpu.from_numpy(qn) if qk_norm else None
    KN = gpu.from_numpy(kn) if qk_norm else None
    kc, vc = gpu.Malloc(max_seq * kvd), gpu.Malloc(max_seq * kvd)
    kc.Zero(); vc.Zero()
    ref_k, ref_v = np.zeros((max_seq, kvd), dtype=F), np.zeros((max_seq, kvd), dtype=F)
    pos_buf = gpu.MallocBytes(4)
    out = gpu.Malloc(heads * head_dim)
    scale = 1.0 / np.sqrt(head_dim)
    checks = {0, 1, 31, 32, 127, 128, 129, 255, 256, 257, steps - 1}
    for pos in range(steps):
        q = g.standard_normal(heads * head_dim, dtype=F)
        k = g.standard_normal(kvd, dtype=F)
        v = g.standard_normal(kvd, dtype=F)
        pos_buf.UploadBytes(np.array([pos], dtype=np.int32).view(np.uint8))
        Q, K, V = gpu.from_numpy(q), gpu.from_numpy(k), gpu.from_numpy(v)
        if fused:
            gpu.AttnDecodeFused(out, Q, K, V, QN, KN, T, pos_buf, kc, vc, max_seq, heads, kv_heads, head_dim, scale, 1e-6)
        else:
            gpu.QKNormRoPEAppend(Q, K, V, QN, KN, T, pos_buf, kc, vc, max_seq, heads, kv_heads, head_dim, 1e-6)
            gpu.AttnDecode(out, Q, kc, vc, pos_buf, max_seq, heads, kv_heads, head_dim, scale)
        if pos in checks:
            gpu.Sync()
        rq, rk = q.copy(), k.copy()
        if qk_norm:
            rq = np.concatenate([od.rmsnorm(rq[h * head_dim:(h + 1) * head_dim], qn, 1e-6) for h in range(heads)]).astype(F)
            rk = np.concatenate([od.rmsnorm(rk[h * head_dim:(h + 1) * head_dim], kn, 1e-6) for h in range(kv_heads)]).astype(F)
        od.apply_rope(rq, table, pos, heads, head_dim)
        od.apply_rope(rk, table, pos, kv_heads, head_dim)
        ref_k[pos], ref_v[pos] = rk, v
        if pos in checks:
            if not fused:
                assert np.allclose(Q.Download(), rq, rtol=1e-5, atol=1e-6)
            assert np.allclose(kc.Download()[pos * kvd:(pos + 1) * kvd], rk, rtol=1e-5, atol=1e-6)
            assert np.array_equal(vc.Download()[pos * kvd:(pos + 1) * kvd], v)
            want = od.attention(rq, ref_k, ref_v, pos + 1, heads, kv_heads, head_dim, scale)
            assert np.allclose(out.Download(), want, rtol=1e-4, atol=2e-5)
        for t in (Q, K, V):
            t.Free()


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("bad_pos", [16, -1, 1 << 20])
def test_position_outside_the_cache_is_refused(gpu, pkg, fused, bad_pos):
    """A step replayed once more than the cache holds (or a stale position word) must not write out of
    bounds: the kernels leave q, the caches and out untouched and record 401 / 402 in the status word."""
    heads, kv_heads, head_dim, max_seq = 4, 2, 64, 16
    kvd = kv_heads * head_dim
    g = pkg.synth.rng("badpos")
    T = gpu.from_numpy(od.rope_table(max_seq, head_dim, 1e6).reshape(-1))
    kc, vc = gpu.Malloc(max_seq * kvd + 64), gpu.Malloc(max_seq * kvd + 64)
    sentinel = np.full(max_seq * kvd + 64, 123.0, dtype=F)
    kc.Upload(sentinel); vc.Upload(sentinel)
    q = g.standard_normal(heads * head_dim, dtype=F)
    Q, K, V = gpu.from_numpy(q), gpu.from_numpy(g.standard_normal(kvd, dtype=F)), gpu.from_numpy(g.standard_normal(kvd, dtype=F))
    out = gpu.Malloc(heads * head_dim)
    out.Upload(np.full(heads * head_dim, 7.0, dtype=F))
    pos_buf = gpu.from_numpy(np.array([bad_pos], dtype=np.int32))
    assert gpu.KernelStatus() == 0
    try:
        if fused:
            gpu.AttnDecodeFused(out, Q, K, V, None, None, T, pos_buf, kc, vc, max_seq, heads, kv_heads, head_dim, 0.125, 1e-6)
        else:
            gpu.QKNormRoPEAppend(Q, K, V, None, None, T, pos_buf, kc, vc, max_seq, heads, kv_heads, head_dim, 1e-6)
            gpu.AttnDecode(out, Q, kc, vc, pos_buf, max_seq, heads, kv_heads, head_dim, 0.125)
        gpu.Sync()
        assert gpu.KernelStatus() == (402 if fused else 401)
        assert np.array_equal(kc.Download(), sentinel) and np.array_equal(vc.Download(), sentinel)
        assert np.array_equal(Q.Download(), q) and np.all(out.Download() == 7.0)
    finally:
        gpu.KernelStatusClear()
    assert gpu.KernelStatus() == 0
    for t in (T, kc, vc, Q, K, V, out, pos_buf):
        t.Free()


def test_silu_mul_argmax_embed(gpu, pkg):
    g = pkg.synth.rng("misc")
    n = 3072
    a, b = g.standard_normal(n, dtype=F) * F(3), g.standard_normal(n, dtype=F)
    out = gpu.Malloc(n)
    gpu.SiLUMul(out, gpu.from_numpy(a), gpu.from_numpy(b), n)
    gpu.Sync()
    assert np.allclose(out.Download(), od.silu_mul(a, b), rtol=2e-6, atol=1e-7)
    # argmax: first maximum, history and position bookkeeping, forced tokens
    logits = g.standard_normal(151936, dtype=F)
    logits[[77, 5000, 150000]] = logits.max() + F(1)
    ints = gpu.MallocBytes(8 + 8 * 16)
    host = np.full(2 + 32, -1, dtype=np.int32)
    host[0], host[1] = 3, 4
    host[2 + 16 + 6] = 999                                     # forced[6]
    ints.UploadBytes(host.view(np.uint8))
    tok, pos = gpu.wrap(ints.Ptr, 4), gpu.wrap(ints.Ptr + 4, 4)
    hist, forced = gpu.wrap(ints.Ptr + 8, 64), gpu.wrap(ints.Ptr + 8 + 64, 64)
    L = gpu.from_numpy(logits)
    gpu.ArgmaxAdvance(L, logits.size, tok, pos, hist, forced, 16)
    gpu.ArgmaxAdvance(L, logits.size, tok, pos, hist, forced, 16)
    gpu.Sync()
    got = ints.Download(2 + 32, dtype=np.int32)
    assert got[0] == 999 and got[1] == 6 and got[2 + 5] == 77 and got[2 + 6] == 999
    # embedding = dequantised row of the tied LM head, both layouts
    for layout, (rows, cols) in ((1, (300, 256)), (2, (300, 256)), (0, (8192, 1024))):
        w, s, b2 = pkg.synth.mlx_weight(("emb", layout), rows, cols, 64)
        gpu.SetOption("mlx_layout", layout)
        h = gpu.UploadMLXWeight(w, s, b2, cols, rows, 64, True)
        gpu.SetOption("mlx_layout", 0)
        want = orc.mlx_dequant(w, s, b2, rows, cols, 64).reshape(rows, cols)
        e = gpu.Malloc(cols)
        for t in (0, 129, rows - 1):
            ints.UploadBytes(np.array([t], dtype=np.int32).view(np.uint8))
            gpu.EmbedMLX(e, h, tok)
            gpu.Sync()
            assert np.array_equal(e.Download().view(np.uint32), want[t].view(np.uint32))
        h.Free()


def build_model(pkg, cfg, key, centred=False):
    syn = pkg.synth
    g = syn.rng("decode", key)
    shapes = {"q": (cfg.heads * cfg.head_dim, cfg.hidden), "k": (cfg.kv_heads * cfg.head_dim, cfg.hidden),
              "v": (cfg.kv_heads * cfg.head_dim, cfg.hidden), "o": (cfg.hidden, cfg.heads * cfg.head_dim),
              "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden), "down": (cfg.hidden, cfg.inter)}
    def mlx(wsb):
        # centred: bias = -7.5 * scale (bf16) instead of -8 * scale, i.e. weights of zero mean
        return (wsb[0], wsb[1], syn.bf16_round(F(-7.5) * wsb[1])) if centred else wsb

    layers_gpu, layers_orc = [], []
    for l in range(cfg.layers):
        dg, do = {}, {}
        for name, (o, i) in shapes.items():
            w = mlx(syn.mlx_weight((key, name, l % 4), o, i, 64))   # four distinct sets of layer weights
            dg[name] = w
            do[name] = (w, o, i)
        for name, n in (("input_norm", cfg.hidden), ("post_norm", cfg.hidden), ("q_norm", cfg.head_dim), ("k_norm", cfg.head_dim)):
            v = (F(1) + F(0.1) * g.standard_normal(n, dtype=F)).astype(F)   # norm weights 1 + small noise
            dg[name] = do[name] = v
        layers_gpu.append(dg)
        layers_orc.append(do)
    lm = mlx(syn.mlx_weight((key, "lm"), cfg.vocab, cfg.hidden, 64))
    final_norm = (F(1) + F(0.1) * g.standard_normal(cfg.hidden, dtype=F)).astype(F)
    return layers_gpu, layers_orc, lm, final_norm


LOGIT_TOL = 2e-4   # (measured 1.2e-5) max |logit_gpu - logit_oracle| / max |logit_oracle| allowed at any position


def run_gate(gpu, pkg, cfg, key, prompt_len, max_new, centred=False):
    """Greedy decode on the GPU against the restated CPU loop: tokens, and the logits of EVERY
    position (prompt positions included).  Returns the statistics the assertions and the report use."""
    layers_gpu, layers_orc, lm, final_norm = build_model(pkg, cfg, key, centred)
    prompt = [int(t) for t in pkg.synth.rng("prompt", key).integers(0, cfg.vocab, prompt_len)]
    oracle = od.OracleDecoder(cfg, od.MLXWeights(orc, cfg, layers_orc, lm, final_norm, nthreads=16))
    trace, ref_logits, got_logits = [], [], []
    want = oracle.generate(prompt, max_new, trace=trace, all_logits=ref_logits)
    dec = pkg.decode.MLXDecoder(gpu, cfg, layers_gpu, lm, final_norm, od.rope_table(cfg.max_seq, cfg.head_dim, cfg.theta))
    got = dec.generate(prompt, max_new, logits_all=got_logits)
    assert gpu.KernelStatus() == 0
    assert len(got_logits) == len(ref_logits) == prompt_len + max_new - 1
    margins = [m for _, m, _ in trace]
    # positions whose inputs are the same on both sides: everything up to the first differing token
    same = next((i for i, (x, y) in enumerate(zip(got, want)) if x != y), len(want))
    npos = min(len(ref_logits), same)
    errs, top5_bad = [], 0
    for p in range(npos):
        r, g = ref_logits[p], got_logits[p]
        d = float(np.max(np.abs(g - r)))
        errs.append(d / float(np.max(np.abs(r))))
        t6 = np.sort(np.partition(r, -6)[-6:])
        if t6[1] - t6[0] > 4 * d:   # the 5th and 6th largest are further apart than the error
            top5_bad += set(np.argpartition(r, -5)[-5:].tolist()) != set(np.argpartition(g, -5)[-5:].tolist())
    stats = {"positions_compared": npos, "max_logit_err": max(errs), "min_margin": min(margins),
             "median_margin": float(np.median(margins)), "distinct_generated": len(set(want[prompt_len:])),
             "first_difference": None if same == len(want) else same, "top5_mismatches": top5_bad}
    print("decode gate %s%s: %s" % (key, " (centred)" if centred else "", stats))
    assert stats["max_logit_err"] <= LOGIT_TOL, stats
    assert top5_bad == 0, stats
    if same < len(want):
        # a different token is only acceptable at a near tie: the oracle's margin at that step within
        # four times the logit error measured there
        step = same - prompt_len
        r, g = ref_logits[same - 1], got_logits[same - 1]
        assert margins[step] <= 4 * float(np.max(np.abs(g - r))), (stats, margins[step])
    return want, got, stats, dec


def layer_states(gpu, pkg, cfg, key, prompt_len, pos, centred=False):
    """The residual stream after every layer at position `pos` of the prompt, GPU against the restated
    CPU loop: the layer-by-layer comparison the reference does with its labelled-tensor hooks."""
    layers_gpu, layers_orc, lm, final_norm = build_model(pkg, cfg, key, centred)
    prompt = [int(t) for t in pkg.synth.rng("prompt", key).integers(0, cfg.vocab, prompt_len)]
    oracle = od.OracleDecoder(cfg, od.MLXWeights(orc, cfg, layers_orc, lm, final_norm, nthreads=16))
    ref = []
    for p in range(pos + 1):
        oracle.step(prompt[p], p, dump=ref if p == pos else None)
    dec = pkg.decode.MLXDecoder(gpu, cfg, layers_gpu, lm, final_norm, od.rope_table(cfg.max_seq, cfg.head_dim, cfg.theta))
    dec.reset(prompt)
    got = []
    for p in range(pos + 1):
        dec.step(None, dump=got if p == pos else None)
    gpu.Sync()
    assert [n for n, _ in got] == [n for n, _ in ref] and len(ref) == cfg.layers
    return [float(np.max(np.abs(g - r)) / np.max(np.abs(r))) for (_, g), (_, r) in zip(got, ref)]


def test_greedy_tokens_small_model(gpu, pkg):
    cfg = od.DecodeConfig(hidden=512, layers=3, heads=8, kv_heads=4, head_dim=64, inter=1024, vocab=4096, max_seq=64)
    want, got, stats, dec = run_gate(gpu, pkg, cfg, "small", 12, 40)
    assert got == want, stats
    again = dec.generate(want[:12], 40, use_graph=False)     # plain launches give the same tokens as the graph
    assert again == want
    # the same model with norm / activation as separate launches instead of inside the products
    layers_gpu, _, lm, final_norm = build_model(pkg, cfg, "small")
    plain = pkg.decode.MLXDecoder(gpu, cfg, layers_gpu, lm, final_norm, od.rope_table(cfg.max_seq, cfg.head_dim, cfg.theta), fuse=False)
    assert dec.fused and not plain.fused and plain.launches_per_step == 0
    assert plain.generate(want[:12], 40) == want
    assert plain.launches_per_step > dec.launches_per_step


def test_greedy_tokens_vary_small_model(gpu, pkg):
    """Biases of -7.5 * scale centre the weights, and the greedy sequence then changes from step to step
    with top-2 margins of a few hundredths: a decoder that is off by more than rounding fails here."""
    cfg = od.DecodeConfig(hidden=512, layers=3, heads=8, kv_heads=4, head_dim=64, inter=1024, vocab=4096, max_seq=64)
    want, got, stats, _ = run_gate(gpu, pkg, cfg, "small", 12, 40, centred=True)
    assert stats["distinct_generated"] >= 16, stats
    assert got == want or stats["first_difference"] is not None
    errs = layer_states(gpu, pkg, cfg, "small", 12, 9, centred=True)
    print("residual stream after each layer at position 9, max relative difference:", ["%.2e" % e for e in errs])
    assert max(errs) <= 1e-3, errs


def test_gemv_with_operation_in_front(gpu, pkg):
    """goph_mlx_gemv_pre against the separate operations of the oracle."""
    out_dim, in_dim = 768, 1024
    w, s, b = pkg.synth.mlx_weight("pre", out_dim, in_dim, 64)
    gpu.SetOption("mlx_layout", 1)
    h = gpu.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
    gpu.SetOption("mlx_layout", 0)
    g = pkg.synth.rng("pre")
    x, r, nw = (g.standard_normal(in_dim, dtype=F) for _ in range(3))
    X, R, NW = gpu.from_numpy(x), gpu.from_numpy(r), gpu.from_numpy(nw)
    out, hid = gpu.Malloc(out_dim), gpu.Malloc(in_dim)
    gpu.GemvMLXPre(out, h, 1, X, R, NW, hid, 1e-6)
    gpu.Sync()
    assert np.array_equal(hid.Download(), x + r)
    want = orc.mlx_gemv(od.rmsnorm(x + r, nw, 1e-6).astype(F), w, s, b, out_dim, in_dim, 64)
    assert pkg.synth.rel_err(out.Download(), want) <= 2e-3
    gpu.GemvMLXPre(out, h, 1, X, None, NW, None, 1e-6)           # no residual, no hidden output
    gpu.Sync()
    assert pkg.synth.rel_err(out.Download(), orc.mlx_gemv(od.rmsnorm(x, nw, 1e-6).astype(F), w, s, b, out_dim, in_dim, 64)) <= 2e-3
    gpu.GemvMLXPre(out, h, 2, X, R, None, None)                   # silu(x) * r
    gpu.Sync()
    assert pkg.synth.rel_err(out.Download(), orc.mlx_gemv(od.silu_mul(x, r).astype(F), w, s, b, out_dim, in_dim, 64)) <= 2e-3
    with pytest.raises(gpu.GophError):
        gpu.GemvMLXPre(out, h, 1, X, R, NW, X)                    # hidden_out aliasing an input
    with pytest.raises(gpu.GophError):
        gpu.GemvMLXPre(out, h, 3, X, R, NW, None)
    gpu.SetOption("mlx_layout", 2)
    ht = gpu.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
    gpu.SetOption("mlx_layout", 0)
    with pytest.raises(gpu.GophError):
        gpu.GemvMLXPre(out, ht, 1, X, R, NW, hid)                 # tiled weights: not supported, the caller splits
    h.Free(); ht.Free()


QWEN3_0_6B = dict(hidden=1024, layers=28, heads=16, kv_heads=8, head_dim=128, inter=3072, vocab=151936,
                  eps=1e-6, theta=1e6, qk_norm=True, max_seq=192)


def test_greedy_tokens_qwen3_0_6b(gpu, pkg):
    """Random-init Qwen3-0.6B architecture in MLX 4-bit g64 (bias = -8 * scale), 128-token random
    prompt, 64 greedy tokens: identical to the restatement of the reference's CPU loop, and the logits
    of all 191 positions within LOGIT_TOL of its logits."""
    cfg = od.DecodeConfig(**QWEN3_0_6B)
    want, got, stats, _ = run_gate(gpu, pkg, cfg, "qwen3-0.6b", 128, 64)
    assert got == want, stats
    assert stats["positions_compared"] == 191


def test_greedy_tokens_vary_qwen3_0_6b(gpu, pkg):
    """The same architecture with centred weights (bias = -7.5 * scale): the 64 greedy tokens vary, the
    logits of every position are compared, and the residual stream after each of the 28 layers at a
    mid-prompt position is compared layer by layer."""
    cfg = od.DecodeConfig(**QWEN3_0_6B)
    want, got, stats, _ = run_gate(gpu, pkg, cfg, "qwen3-0.6b", 128, 64, centred=True)
    assert stats["distinct_generated"] >= 16, stats
    errs = layer_states(gpu, pkg, cfg, "qwen3-0.6b", 128, 40, centred=True)
    print("residual stream after each layer at position 40, max relative difference: first %.2e last %.2e max %.2e"
          % (errs[0], errs[-1], max(errs)))
    assert max(errs) <= 1e-3, errs


def test_product_lists_change_nothing(gpu, pkg):
    """The step with everything between two attentions as one cooperative launch (two launches per
    layer) against the same step as five launches per layer: same tokens, same logits bit for bit."""
    cfg = od.DecodeConfig(hidden=512, layers=3, heads=8, kv_heads=4, head_dim=64, inter=1024, vocab=4096, max_seq=40)
    layers_gpu, _, lm, final_norm = build_model(pkg, cfg, "lists")
    table = od.rope_table(cfg.max_seq, cfg.head_dim, cfg.theta)
    with_lists = pkg.decode.MLXDecoder(gpu, cfg, layers_gpu, lm, final_norm, table, lists=True)
    without = pkg.decode.MLXDecoder(gpu, cfg, layers_gpu, lm, final_norm, table)
    assert with_lists.lists is not None and len(with_lists.lists) == cfg.layers + 1 and without.lists is None
    prompt = [5, 17, 3, 99, 1024, 7]
    la, lb = [], []
    a = with_lists.generate(prompt, 12, use_graph=True, logits_at=la)
    b = without.generate(prompt, 12, use_graph=True, logits_at=lb)
    assert a == b
    for x, y in zip(la, lb):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))
    assert with_lists.launches_per_step < without.launches_per_step
    assert all(p.Status() == 0 for p in with_lists.lists)
    assert with_lists.generate(prompt, 12, use_graph=False) == a
