"""GPU parity of the work-list GGUF products (fused gate/up + GELU, weighted scatter-add) through the C ABI.

The cases follow the reference's own tests for these operators (backends/nvidia/runtime/q4k_gateup_test.go,
q4k_bywork_test.go, q8_test.go:60-100, q8_work_test.go:11-104): experts stacked in one matrix, a short work
list, every item checked against the single-expert product."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc

pytestmark = pytest.mark.gpu
Q8_0, Q4_K = orc.Q8_0, orc.Q4_K


def make(pkg, qtype, key, out_dim, in_dim):
    gen = {Q8_0: pkg.synth.q8_0_matrix, Q4_K: pkg.synth.q4k_matrix}[qtype]
    return gen(key, out_dim, in_dim)


def gelu_tanh(g):
    g = g.astype(np.float64)
    return 0.5 * g * (1.0 + np.tanh(0.7978845608 * (g + 0.044715 * g ** 3)))


@pytest.mark.parametrize("layout", [1, 2])
@pytest.mark.parametrize("qtype", [Q4_K, Q8_0])
def test_gate_up_gelu_batch(gpu, pkg, qtype, layout):
    inter, in_dim, batch = 96, 512, 3
    raw = make(pkg, qtype, ("gu", layout), 2 * inter, in_dim)
    gpu.SetOption("gguf_layout", layout)
    try:
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, 2 * inter)
    finally:
        gpu.SetOption("gguf_layout", 0)
    x = pkg.synth.activations(("gu", batch), batch * in_dim, bf16=False)
    xo, out = gpu.from_numpy(x), out_with_canary(gpu, batch * inter)
    gpu.GateUpGELUQ4KBatchToBuffer(out, xo, batch, inter, m)
    gpu.Sync()
    got = read_and_check_canary(out, batch * inter).reshape(batch, inter)
    y = orc.gguf_gemv(x, raw, qtype, in_dim, 2 * inter, batch, nthreads=4).reshape(batch, 2 * inter)
    want = (gelu_tanh(y[:, :inter]) * y[:, inter:].astype(np.float64)).astype(F)
    assert pkg.synth.rel_err(got.reshape(-1), want.reshape(-1)) <= TOL
    with pytest.raises(gpu.GophError):   # the matrix must hold exactly gate and up
        gpu.GateUpGELUQ4KBatchToBuffer(out, xo, batch, inter - 1, m)
    for t in (m, xo, out):
        t.Free()


@pytest.mark.parametrize("layout", [1, 2])
@pytest.mark.parametrize("qtype", [Q4_K, Q8_0])
def test_gate_up_gelu_by_work(gpu, pkg, qtype, layout):
    inter, in_dim, active = 64, 256, 3
    experts = [0, 2, 0, 1, 2]
    raw = make(pkg, qtype, ("guw", layout), active * 2 * inter, in_dim)
    gpu.SetOption("gguf_layout", layout)
    try:
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, active * 2 * inter)
    finally:
        gpu.SetOption("gguf_layout", 0)
    n = len(experts)
    x = pkg.synth.activations(("guw", n), n * in_dim, bf16=False)
    xo, we, out = gpu.from_numpy(x), gpu.from_numpy(np.array(experts, dtype=np.uint32)), out_with_canary(gpu, n * inter)
    gpu.GateUpGELUQ4KByWorkToBuffer(out, xo, we, n, inter, active, m)
    gpu.Sync()
    got = read_and_check_canary(out, n * inter).reshape(n, inter)
    row_bytes = raw.size // (active * 2 * inter)
    for w, e in enumerate(experts):   # every item against the single-expert product, as the reference's test does
        slab = raw[e * 2 * inter * row_bytes:(e + 1) * 2 * inter * row_bytes]
        y = orc.gguf_gemv(x[w * in_dim:(w + 1) * in_dim], slab, qtype, in_dim, 2 * inter, nthreads=4)
        want = (gelu_tanh(y[:inter]) * y[inter:].astype(np.float64)).astype(F)
        assert pkg.synth.rel_err(got[w], want) <= TOL, (w, e)
    assert gpu.KernelStatus() == 0
    # an expert index outside the matrix: the item is skipped, the others are computed, the status says so
    bad = gpu.from_numpy(np.array([0, 7, 1, 1, 2], dtype=np.uint32))
    out2 = out_with_canary(gpu, n * inter)
    gpu.GateUpGELUQ4KByWorkToBuffer(out2, xo, bad, n, inter, active, m)
    gpu.Sync()
    got2 = read_and_check_canary(out2, n * inter).reshape(n, inter)
    assert np.all(got2[1] == F(123.0)) and np.array_equal(got2[0], got[0])
    assert gpu.KernelStatus() == 601
    gpu.KernelStatusClear()
    for t in (m, xo, we, bad, out, out2):
        t.Free()


@pytest.mark.parametrize("layout", [1, 2])
@pytest.mark.parametrize("qtype", [Q8_0, Q4_K])
def test_scatter_by_work_and_batch_scatter(gpu, pkg, qtype, layout):
    expert_out, in_dim, active, tokens = 80, 512, 3, 4
    work_active, work_pos, work_weight = [0, 1, 0, 2, 1], [2, 0, 1, 2, 3], [0.5, 0.25, 1.0, -0.75, 2.0]
    raw = make(pkg, qtype, ("sc", layout), active * expert_out, in_dim)
    gpu.SetOption("gguf_layout", layout)
    try:
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, active * expert_out)
    finally:
        gpu.SetOption("gguf_layout", 0)
    n = len(work_active)
    x = pkg.synth.activations(("sc", n), n * in_dim, bf16=False)
    xo = gpu.from_numpy(x)
    wa, wp = gpu.from_numpy(np.array(work_active, dtype=np.uint32)), gpu.from_numpy(np.array(work_pos, dtype=np.uint32))
    ww = gpu.from_numpy(np.array(work_weight, dtype=F))
    base = pkg.synth.activations("sc-dst", tokens * expert_out, bf16=False)   # dst is added to, not overwritten
    dst = gpu.from_numpy(np.concatenate([base, np.full(64, 123.0, dtype=F)]))
    gpu.GemvQ8_0ScatterByWork(gpu.wrap(dst.Ptr, tokens * expert_out * 4), xo, wa, wp, ww, n, active, m)
    gpu.Sync()
    got = dst.Download()
    assert np.all(got[tokens * expert_out:] == F(123.0))
    want = base.astype(np.float64).reshape(tokens, expert_out).copy()
    row_bytes = raw.size // (active * expert_out)
    for w in range(n):   # two items share destination row 2
        slab = raw[work_active[w] * expert_out * row_bytes:(work_active[w] + 1) * expert_out * row_bytes]
        y = orc.gguf_gemv(x[w * in_dim:(w + 1) * in_dim], slab, qtype, in_dim, expert_out, nthreads=4)
        want[work_pos[w]] += np.float64(work_weight[w]) * y
    assert pkg.synth.rel_err(got[:tokens * expert_out], want.reshape(-1).astype(F)) <= TOL
    # a destination past the end of dst: skipped, status 602
    far = gpu.from_numpy(np.array([2, 0, 1, 99, 3], dtype=np.uint32))
    gpu.GemvQ8_0ScatterByWork(gpu.wrap(dst.Ptr, tokens * expert_out * 4), xo, wa, far, ww, n, active, m)
    gpu.Sync()
    assert np.all(dst.Download()[tokens * expert_out:] == F(123.0)) and gpu.KernelStatus() == 602
    gpu.KernelStatusClear()
    # the whole matrix as one expert: GemvQ8_0BatchScatter (runtime/q8_test.go:60-100)
    dst2 = gpu.from_numpy(np.zeros(3 * active * expert_out, dtype=F))
    pos2, w2 = gpu.from_numpy(np.array([2, 0], dtype=np.uint32)), gpu.from_numpy(np.array([0.5, 0.25], dtype=F))
    gpu.GemvQ8_0BatchScatter(dst2, xo, pos2, w2, 2, m)
    gpu.Sync()
    got2 = dst2.Download().reshape(3, active * expert_out)
    y = orc.gguf_gemv(x[:2 * in_dim], raw, qtype, in_dim, active * expert_out, 2, nthreads=4).reshape(2, -1)
    assert pkg.synth.rel_err(got2[2], (0.5 * y[0]).astype(F)) <= TOL and pkg.synth.rel_err(got2[0], (0.25 * y[1]).astype(F)) <= TOL
    assert np.all(got2[1] == 0)
    for t in (m, xo, wa, wp, ww, far, dst, dst2, pos2, w2):
        t.Free()


@pytest.mark.parametrize("layout", [1, 2])
@pytest.mark.parametrize("qtype", [Q4_K, Q8_0])
@pytest.mark.parametrize("active,experts", [
    (3, [0, 2, 0, 1, 2, 0, 0, 2, 1, 0, 2, 1, 1]),   # five, four and four items: passes of four and one
    (8, [3, 1, 3, 7, 1]),                            # fewer items than experts: the grid goes by item
    (2, [1] * 9),                                    # one expert with nine items
])
def test_long_and_short_work_lists(gpu, pkg, qtype, layout, active, experts):
    # both products on one list: every item against the single-expert products, as the reference's tests do
    inter, hidden, tokens = 64, 256, 4
    n = len(experts)
    raw_gu = make(pkg, qtype, ("lgu", layout, active), active * 2 * inter, hidden)
    raw_dn = make(pkg, qtype, ("ldn", layout, active), active * hidden, inter * 4)     # down: in_dim 256
    gpu.SetOption("gguf_layout", layout)
    try:
        gu = gpu.UploadGGUFMatrix(qtype, raw_gu, hidden, active * 2 * inter)
        dn = gpu.UploadGGUFMatrix(qtype, raw_dn, inter * 4, active * hidden)
    finally:
        gpu.SetOption("gguf_layout", 0)
    x = pkg.synth.activations(("long", n), n * hidden, bf16=False)
    xo, we, out = gpu.from_numpy(x), gpu.from_numpy(np.array(experts, dtype=np.uint32)), out_with_canary(gpu, n * inter)
    gpu.GateUpGELUQ4KByWorkToBuffer(out, xo, we, n, inter, active, gu)
    gpu.Sync()
    got = read_and_check_canary(out, n * inter).reshape(n, inter)
    rb = raw_gu.size // (active * 2 * inter)
    for w, e in enumerate(experts):
        y = orc.gguf_gemv(x[w * hidden:(w + 1) * hidden], raw_gu[e * 2 * inter * rb:(e + 1) * 2 * inter * rb], qtype, hidden, 2 * inter, nthreads=4)
        want = (gelu_tanh(y[:inter]) * y[inter:].astype(np.float64)).astype(F)
        assert pkg.synth.rel_err(got[w], want) <= TOL, (w, e)
    # scatter-add of the down products into four destination rows
    pos = np.arange(n, dtype=np.uint32) % tokens
    wt = pkg.synth.rng("long-w", n).uniform(0.1, 0.5, n).astype(F)
    h = pkg.synth.activations(("long-h", n), n * inter * 4, bf16=False)
    ho, po, wo = gpu.from_numpy(h), gpu.from_numpy(pos), gpu.from_numpy(wt)
    base = pkg.synth.activations("long-dst", tokens * hidden, bf16=False)
    dst = gpu.from_numpy(np.concatenate([base, np.full(64, 123.0, dtype=F)]))
    gpu.GemvQ8_0ScatterByWork(gpu.wrap(dst.Ptr, tokens * hidden * 4), ho, we, po, wo, n, active, dn)
    gpu.Sync()
    res = dst.Download()
    assert np.all(res[tokens * hidden:] == F(123.0))
    want = base.astype(np.float64).reshape(tokens, hidden).copy()
    rb = raw_dn.size // (active * hidden)
    for w, e in enumerate(experts):
        y = orc.gguf_gemv(h[w * inter * 4:(w + 1) * inter * 4], raw_dn[e * hidden * rb:(e + 1) * hidden * rb], qtype, inter * 4, hidden, nthreads=4)
        want[pos[w]] += np.float64(wt[w]) * y
    assert pkg.synth.rel_err(res[:tokens * hidden], want.reshape(-1).astype(F)) <= TOL
    assert gpu.KernelStatus() == 0
    for t in (gu, dn, xo, we, out, ho, po, wo, dst):
        t.Free()


def test_work_calls_reject_malformed_arguments(gpu, pkg):
    raw = make(pkg, Q4_K, "bad", 128, 256)
    m = gpu.UploadGGUFMatrix(Q4_K, raw, 256, 128)
    x, out, we = gpu.Malloc(256), gpu.Malloc(64), gpu.from_numpy(np.zeros(1, dtype=np.uint32))
    with pytest.raises(gpu.GophError):
        gpu.GateUpGELUQ4KByWorkToBuffer(out, x, we, 1, 64, 2, m)        # 2 experts x 128 rows do not fit 128 rows
    with pytest.raises(gpu.GophError):
        gpu.GateUpGELUQ4KByWorkToBuffer(gpu.wrap(out.Ptr, 63 * 4), x, we, 1, 64, 1, m)   # short out
    with pytest.raises(gpu.GophError):
        gpu.GemvQ8_0ScatterByWork(out, x, we, we, out, 1, 3, m)          # 128 rows do not divide into 3 experts
    gpu.GateUpGELUQ4KByWorkToBuffer(out, x, we, 0, 64, 1, m)             # an empty work list is a no-op, as in the reference
    for t in (m, x, out, we):
        t.Free()
