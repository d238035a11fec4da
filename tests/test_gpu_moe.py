"""GPU parity of the mixture-of-experts selected-expert path against the CPU oracle, through the C ABI.

Routing from supplied logits is compared exactly (ids and weights bit for bit); the expert
projections within max relative error 2e-3 of the oracle (floor 1e-3 of the largest output)."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def no_wait_gave_up(gpu):
    yield
    assert gpu.KernelStatus() == 0


class Layer:
    """Synthetic MoE layer resident on the GPU plus the stacked host arrays the oracle takes."""

    def __init__(self, rt, syn, key, experts, hidden, inter, gs=64, top_k=8, norm=True, max_tokens=32, resident=None,
                 layout=1):
        # layout: 1 = experts row-major (CUDA-core expert kernels), 2 = tiled (grouped tensor-core launches)
        self.rt, self.E, self.hidden, self.inter, self.gs = rt, experts, hidden, inter, gs
        self.top_k, self.norm = top_k, norm
        g = syn.rng("moe", key, experts, hidden, inter, gs)

        def stack(out_dim, in_dim):
            w = g.integers(0, 2**32, size=(experts, out_dim * (in_dim // 8)), dtype=np.uint32)
            s = syn.bf16_round(np.abs(g.standard_normal((experts, out_dim * (in_dim // gs)), dtype=F)) * F(0.02) + F(1e-3))
            return w, s, syn.bf16_round(F(-8) * s)

        self.gate, self.up, self.down = stack(inter, hidden), stack(inter, hidden), stack(hidden, inter)
        self.router = syn.mlx_weight(("router", key), experts, hidden, gs)
        rt.SetOption("mlx_layout", 1)
        try:
            self.layer = rt.GPUMoELayer(experts, hidden, inter, gs, top_k, norm, max_tokens)
            self.rw = rt.UploadMLXWeight(*self.router, hidden, experts, gs, True)
            self.layer.SetRouter(self.rw)
            self.handles = []
            rt.SetOption("mlx_layout", layout)
            for e in range(experts):
                if resident is not None and e not in resident:
                    continue
                hs = [rt.UploadMLXWeight(t[0][e], t[1][e], t[2][e], i, o, gs, True)
                      for t, o, i in ((self.gate, inter, hidden), (self.up, inter, hidden), (self.down, hidden, inter))]
                self.layer.SetExpert(e, *hs)
                self.handles += hs
        finally:
            rt.SetOption("mlx_layout", 0)

    def oracle_logits(self, x):
        return orc.mlx_gemv(x, *self.router, self.E, self.hidden, self.gs)

    def oracle(self, x, ids, wts):
        return orc.moe_experts(x, self.hidden, self.inter, self.gs, self.gate, self.up, self.down, ids, wts)

    def free(self):
        self.layer.Free()
        self.rw.Free()
        for h in self.handles:
            h.Free()


def run_forward(L, x, tokens, logits=None):
    rt = L.rt
    xb = rt.from_numpy(x)
    out = out_with_canary(rt, tokens * L.hidden)
    if logits is None:
        L.layer.Forward(out, xb, tokens)
    else:
        lb = rt.from_numpy(logits)
        L.layer.ForwardLogits(out, xb, lb, tokens)
    rt.Sync()
    got = read_and_check_canary(out, tokens * L.hidden).reshape(tokens, L.hidden)
    ids, wts = L.layer.LastRouting(tokens)
    xb.Free(); out.Free()
    return got, ids, wts


@pytest.mark.parametrize("experts,hidden,inter,top_k,norm,tokens", [
    (6, 128, 256, 2, True, 1),      # the reference's own MoE test shape (model/moe_mlx_test.go:10-40)
    (16, 512, 256, 4, True, 3),
    (16, 512, 256, 4, False, 5),
    (8, 1024, 768, 8, True, 2),     # every expert selected
    (5, 256, 128, 9, True, 2),      # top_k above the expert count is clamped
    (8, 512, 256, 8, True, 6),      # every expert has six tokens: two passes over its rows
    (4, 256, 128, 2, True, 13),     # ragged passes (4 + 4 + ...)
    (128, 2048, 768, 8, True, 1),   # Qwen3-30B-A3B layer, decode
    (128, 2048, 768, 8, True, 8),
    (128, 2048, 768, 8, True, 32),
])
def test_forward_parity(gpu, pkg, experts, hidden, inter, top_k, norm, tokens):
    L = Layer(gpu, pkg.synth, "fw", experts, hidden, inter, 64, top_k, norm, max_tokens=32)
    x = pkg.synth.activations(("moe", experts, tokens), tokens * hidden).reshape(tokens, hidden)
    got, ids, wts = run_forward(L, x, tokens)
    k = min(top_k, experts)
    for t in range(tokens):
        want_ids, want_w = orc.moe_route(L.oracle_logits(x[t]), top_k, norm)
        assert len(want_ids) == k
        # the device's logits differ from the oracle's in the last bits; a flip needs a near tie
        p = np.sort(orc.softmax(L.oracle_logits(x[t])))[::-1]
        near_tie = k < experts and (p[k - 1] - p[k]) < 1e-4 * p[k - 1]
        if not near_tie:
            assert set(ids[t].tolist()) == set(want_ids.tolist())
        if list(ids[t]) == list(want_ids):
            assert np.allclose(wts[t], want_w, rtol=1e-4, atol=1e-7)
        want = L.oracle(x[t], ids[t], wts[t])
        assert pkg.synth.rel_err(got[t], want) <= TOL, (t, pkg.synth.rel_err(got[t], want))
    L.free()


@pytest.mark.parametrize("experts,hidden,inter,top_k,norm,tokens", [
    (16, 512, 256, 4, True, 3),
    (16, 512, 256, 4, False, 5),
    (8, 1024, 768, 8, True, 2),     # every expert selected, two items each
    (8, 512, 256, 8, True, 6),      # six items per expert: entries of four and two
    (4, 256, 256, 2, True, 13),     # ragged entries (4 + 4 + ...)
    (3, 256, 256, 3, True, 32),     # 32 items per expert: eight full entries each
    (128, 2048, 768, 8, True, 1),   # Qwen3-30B-A3B layer, decode
    (128, 2048, 768, 8, True, 8),
    (128, 2048, 768, 8, True, 32),
])
def test_forward_parity_tiled_experts(gpu, pkg, experts, hidden, inter, top_k, norm, tokens):
    # experts uploaded in the tiled layout run as grouped launches of the tensor-core kernel
    L = Layer(gpu, pkg.synth, "fw", experts, hidden, inter, 64, top_k, norm, max_tokens=32, layout=2)
    x = pkg.synth.activations(("moe", experts, tokens), tokens * hidden).reshape(tokens, hidden)
    got, ids, wts = run_forward(L, x, tokens)
    for t in range(tokens):
        want = L.oracle(x[t], ids[t], wts[t])
        assert pkg.synth.rel_err(got[t], want) <= TOL, (t, pkg.synth.rel_err(got[t], want))
    # the same tokens one at a time and in another order: a token's result does not depend on its batch
    if tokens > 1:
        order = list(range(tokens))[::-1]
        again, _, _ = run_forward(L, x[order].copy(), tokens)
        assert np.array_equal(again[::-1].view(np.uint32), got.view(np.uint32))
        one, _, _ = run_forward(L, x[tokens - 1:tokens].copy(), 1)
        assert np.array_equal(one[0].view(np.uint32), got[tokens - 1].view(np.uint32))
    L.free()


@pytest.mark.parametrize("layout", [1, 2])
def test_many_tokens_per_call(gpu, pkg, layout):
    # 96 tokens on 16 experts with top-4: 24 items per expert on average (tiled: six work entries each)
    experts, hidden, inter, top_k, tokens = 16, 512, 256, 4, 96
    L = Layer(gpu, pkg.synth, "many", experts, hidden, inter, 64, top_k, True, max_tokens=tokens, layout=layout)
    x = pkg.synth.activations(("many", tokens), tokens * hidden).reshape(tokens, hidden)
    got, ids, wts = run_forward(L, x, tokens)
    for t in range(0, tokens, 7):
        assert pkg.synth.rel_err(got[t], L.oracle(x[t], ids[t], wts[t])) <= TOL, t
    one, _, _ = run_forward(L, x[50:51].copy(), 1)
    assert np.array_equal(one[0].view(np.uint32), got[50].view(np.uint32))
    L.free()


def test_tiled_expert_placement_and_layout_rules(gpu, pkg):
    experts, hidden, inter, top_k, tokens = 32, 512, 256, 8, 4
    full = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True, layout=2)
    lo = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True, resident=set(range(16)), layout=2)
    hi = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True, resident=set(range(16, 32)), layout=2)
    rowmajor = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True, layout=1)
    x = pkg.synth.activations("place", tokens * hidden).reshape(tokens, hidden)
    a, ids, wts = run_forward(full, x, tokens)
    b, ids_lo, _ = run_forward(lo, x, tokens)
    c, ids_hi, _ = run_forward(hi, x, tokens)
    d, ids_rm, _ = run_forward(rowmajor, x, tokens)
    assert np.array_equal(ids, ids_lo) and np.array_equal(ids, ids_hi) and np.array_equal(ids, ids_rm)
    for t in range(tokens):
        assert pkg.synth.rel_err(b[t] + c[t], a[t]) <= 1e-4
        assert pkg.synth.rel_err(a[t], full.oracle(x[t], ids[t], wts[t])) <= TOL
        assert pkg.synth.rel_err(a[t], d[t]) <= 1e-3              # the two expert paths agree (each within 2e-3 of the oracle)
    # a layer's experts share one layout
    with pytest.raises(gpu.GophError):
        full.layer.SetExpert(0, *rowmajor.handles[:3])
    with pytest.raises(gpu.GophError):
        rowmajor.layer.SetExpert(0, *full.handles[:3])
    for L in (full, lo, hi, rowmajor):
        L.free()


@pytest.mark.parametrize("norm", [True, False])
def test_routing_from_logits_is_exact(gpu, pkg, norm):
    experts, hidden, inter, top_k, tokens = 128, 256, 128, 8, 16
    L = Layer(gpu, pkg.synth, "route", experts, hidden, inter, 64, top_k, norm, resident=set(range(4)))
    g = pkg.synth.rng("logits", norm)
    logits = (g.standard_normal((tokens, experts), dtype=F) * F(3)).astype(F)
    logits[1, 5] = logits[1, 77] = logits[1].max() + F(1)      # exact tie: the lower id first
    logits[2, :] = F(0.25)                                      # all equal: ids 0..7
    logits[3, 9] = -np.inf
    x = pkg.synth.activations("route", tokens * hidden).reshape(tokens, hidden)
    _, ids, wts = run_forward(L, x, tokens, logits)
    for t in range(tokens):
        want_ids, want_w = orc.moe_route(logits[t], top_k, norm)
        assert list(ids[t]) == list(want_ids), t
        assert np.array_equal(wts[t].view(np.uint32), want_w.view(np.uint32)), t
    assert list(ids[1][:2]) == [5, 77] and list(ids[2]) == list(range(8))
    L.free()


@pytest.mark.parametrize("layout", [1, 2])
def test_failed_softmax_runs_no_expert(gpu, pkg, layout):
    # simd.SoftmaxInPlace reports failure on a NaN/Inf sum and moeForward then adds nothing
    # (backends/simd/runtime/softmax.go:20-24; model/moe.go:230-233)
    experts, hidden, inter = 8, 256, 256
    L = Layer(gpu, pkg.synth, "nan", experts, hidden, inter, 64, 2, True, layout=layout)
    logits = np.zeros((2, experts), dtype=F)
    logits[0, 3] = np.nan
    logits[1, 2] = 1.0
    x = pkg.synth.activations("nan", 2 * hidden).reshape(2, hidden)
    got, ids, wts = run_forward(L, x, 2, logits)
    assert list(ids[0]) == [-1, -1] and np.all(got[0] == 0)
    want_ids, want_w = orc.moe_route(logits[1], 2, True)
    assert list(ids[1]) == list(want_ids)
    assert pkg.synth.rel_err(got[1], L.oracle(x[1], want_ids, want_w)) <= TOL
    # every token fails: no work entry at all, the output is zero
    logits[1, 5] = np.inf
    got, ids, _ = run_forward(L, x, 2, logits)
    assert np.all(ids == -1) and np.all(got == 0)
    # and the layer still works afterwards
    logits[:] = 0
    logits[0, 1] = logits[1, 6] = 2.0
    got, ids, wts = run_forward(L, x, 2, logits)
    for t in range(2):
        assert pkg.synth.rel_err(got[t], L.oracle(x[t], ids[t], wts[t])) <= TOL
    L.free()


def test_expert_placement_partials_add_up(gpu, pkg):
    # experts split over two "GPUs" (16 + 16): the partial outputs sum to the full result
    experts, hidden, inter, top_k, tokens = 32, 512, 256, 8, 4
    full = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True)
    lo = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True, resident=set(range(16)))
    hi = Layer(gpu, pkg.synth, "place", experts, hidden, inter, 64, top_k, True, resident=set(range(16, 32)))
    x = pkg.synth.activations("place", tokens * hidden).reshape(tokens, hidden)
    a, ids, wts = run_forward(full, x, tokens)
    b, ids_lo, _ = run_forward(lo, x, tokens)
    c, ids_hi, _ = run_forward(hi, x, tokens)
    assert np.array_equal(ids, ids_lo) and np.array_equal(ids, ids_hi)
    for t in range(tokens):
        assert pkg.synth.rel_err(b[t] + c[t], a[t]) <= 1e-4   # f32 sums associated differently
        assert pkg.synth.rel_err(a[t], full.oracle(x[t], ids[t], wts[t])) <= TOL
    for L in (full, lo, hi):
        L.free()


def test_results_do_not_depend_on_scheduling(gpu, pkg):
    L = Layer(gpu, pkg.synth, "det", 16, 512, 256, 64, 4, True)
    x = pkg.synth.activations("det", 8 * 512).reshape(8, 512)
    a, _, _ = run_forward(L, x, 8)
    b, _, _ = run_forward(L, x, 8)
    one, _, _ = run_forward(L, x[5:6].copy(), 1)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.array_equal(a[5].view(np.uint32), one[0].view(np.uint32))   # a token's result does not depend on the batch
    L.free()


@pytest.mark.parametrize("experts,hidden,inter,top_k,resident", [
    (6, 128, 256, 2, None),
    (16, 512, 256, 4, None),
    (128, 2048, 768, 8, None),
    (32, 512, 256, 8, set(range(0, 32, 2))),    # half of the experts live elsewhere
    (5, 256, 128, 9, None),                      # top_k clamped to the expert count
])
def test_one_token_single_launch_form(gpu, pkg, experts, hidden, inter, top_k, resident):
    # a call of one token runs as one cooperative launch; option moe_fused = 0 keeps the five launches.
    # Same bits, call after call (the grid barrier's counter carries over), with and without the router.
    L = Layer(gpu, pkg.synth, "one", experts, hidden, inter, 64, top_k, True, resident=resident)
    g = pkg.synth.rng("one-token", experts)
    for rep in range(3):
        x = pkg.synth.activations(("one", experts, rep), hidden).reshape(1, hidden)
        n0 = gpu.LaunchCount()
        got, ids, wts = run_forward(L, x, 1)
        assert gpu.LaunchCount() - n0 == 1
        gpu.SetOption("moe_fused", 0)
        try:
            n0 = gpu.LaunchCount()
            ref, ids2, wts2 = run_forward(L, x, 1)
            assert gpu.LaunchCount() - n0 == 5
        finally:
            gpu.SetOption("moe_fused", 1)
        assert np.array_equal(ids, ids2) and np.array_equal(wts.view(np.uint32), wts2.view(np.uint32))
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
        res = [e for e in ids[0] if e >= 0 and (resident is None or e in resident)]
        keep = np.array([k for k, e in enumerate(ids[0]) if e in res], dtype=np.int64)
        want = L.oracle(x[0], ids[0][keep], wts[0][keep]) if len(keep) else np.zeros(hidden, dtype=F)
        assert pkg.synth.rel_err(got[0], want) <= TOL
        # routing supplied by the caller (two barriers instead of three in the same launch)
        logits = (g.standard_normal((1, experts), dtype=F) * F(2)).astype(F)
        got_l, ids_l, wts_l = run_forward(L, x, 1, logits)
        want_ids, want_w = orc.moe_route(logits[0], top_k, True)
        assert list(ids_l[0]) == list(want_ids)
        assert np.array_equal(wts_l[0].view(np.uint32), want_w.view(np.uint32))
    logits = np.zeros((1, experts), dtype=F)
    logits[0, 1] = np.nan                       # the softmax fails: no expert runs, the output is zero
    got, ids, _ = run_forward(L, x, 1, logits)
    assert np.all(ids[0] == -1) and np.all(got[0] == 0)
    L.free()


def test_malformed(gpu, pkg):
    rt = gpu
    with pytest.raises(rt.GophError):
        rt.GPUMoELayer(0, 128, 64)
    with pytest.raises(rt.GophError):
        rt.GPUMoELayer(4, 100, 64)                  # hidden not a multiple of the group size
    L = Layer(rt, pkg.synth, "bad", 4, 128, 64, 64, 2, True, max_tokens=2)
    x = rt.Malloc(4 * 128); out = rt.Malloc(4 * 128)
    with pytest.raises(rt.GophError):
        L.layer.Forward(out, x, 3)                  # above max_tokens
    with pytest.raises(rt.GophError):
        L.layer.Forward(rt.Malloc(100), x, 1)       # short out
    wrong = rt.UploadMLXWeight(*pkg.synth.mlx_weight("wrong", 64, 64), 64, 64, 64, True)
    with pytest.raises(rt.GophError):
        L.layer.SetExpert(0, wrong, wrong, wrong)   # wrong shapes
    with pytest.raises(rt.GophError):
        L.layer.SetExpert(9, None, None, None)      # id out of range
    with pytest.raises(rt.GophError):
        L.layer.SetRouter(wrong)
    L.free()
