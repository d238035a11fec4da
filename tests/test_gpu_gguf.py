"""GPU parity of the GGUF Q8_0 / Q4_K / Q5_K / Q6_K path against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc
from test_oracle_pins import q4k_test_rows, q8_0_test_rows, qk_test_rows

pytestmark = pytest.mark.gpu

Q8_0, Q4_K, Q5_K, Q6_K = orc.Q8_0, orc.Q4_K, orc.Q5_K, orc.Q6_K


def make(pkg, qtype, key, out_dim, in_dim):
    gen = {Q8_0: pkg.synth.q8_0_matrix, Q4_K: pkg.synth.q4k_matrix, Q5_K: pkg.synth.q5k_matrix,
           Q6_K: pkg.synth.q6k_matrix}[qtype]
    return gen(key, out_dim, in_dim)


@pytest.mark.parametrize("qtype,out_dim,in_dim", [(Q8_0, 64, 4096), (Q8_0, 3, 32), (Q8_0, 17, 96),
                                                   (Q4_K, 64, 4096), (Q4_K, 2, 256), (Q4_K, 9, 2816),
                                                   (Q5_K, 64, 4096), (Q5_K, 2, 256), (Q5_K, 9, 2816),
                                                   (Q6_K, 64, 4096), (Q6_K, 2, 256), (Q6_K, 9, 2816)])
def test_dequant_bit_exact(gpu, pkg, qtype, out_dim, in_dim):
    raw = make(pkg, qtype, "deq", out_dim, in_dim)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    assert m.ResidentBytes() == raw.size  # the device layout costs what the GGUF stream costs
    out = out_with_canary(gpu, out_dim * in_dim)
    m.Dequant(out)
    gpu.Sync()
    got = read_and_check_canary(out, out_dim * in_dim)
    want = orc.gguf_dequant(raw, qtype, in_dim, out_dim, nthreads=8).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    m.Free(); out.Free()


def test_q4k_reference_formula_blocks(gpu, pkg):
    # backends/nvidia/runtime/q4k_test.go:11-59: GemvQ4K and GemvQ4KBatch vs dequant·x, abs 1e-3
    raw, x, in_dim, out_dim = q4k_test_rows()
    m = gpu.UploadQ4KMatrixRows(raw, in_dim, out_dim)
    got = gpu.GemvQ4K(x, m)
    got2 = gpu.GemvQ4KBatch(np.concatenate([x, x]), 2, m)
    want = orc.gguf_gemv(x, raw, Q4_K, in_dim, out_dim)
    assert np.max(np.abs(got - want)) <= 1e-3
    assert np.max(np.abs(got2[:out_dim] - want)) <= 1e-3 and np.max(np.abs(got2[out_dim:] - want)) <= 1e-3
    m.Free()


def test_q8_0_reference_formula_blocks(gpu, pkg):
    # backends/nvidia/runtime/q8_test.go:25-104: GemvQ8_0 and GemvQ8_0Batch, abs 1e-3
    raw, x, in_dim, out_dim = q8_0_test_rows()
    m = gpu.UploadQ8_0MatrixRows(raw, in_dim, out_dim)
    got = gpu.GemvQ8_0(x, m)
    got2 = gpu.GemvQ8_0Batch(np.concatenate([x, x]), 2, m)
    want = orc.gguf_gemv(x, raw, Q8_0, in_dim, out_dim)
    assert np.max(np.abs(got - want)) <= 1e-3
    assert np.max(np.abs(got2[:out_dim] - want)) <= 1e-3 and np.max(np.abs(got2[out_dim:] - want)) <= 1e-3
    m.Free()


@pytest.mark.parametrize("kind", [5, 6])
def test_q5k_q6k_reference_formula_blocks(gpu, pkg, kind):
    # backends/nvidia/runtime/qk_test.go:11-75: GemvQ5KBatch / GemvQ6KBatch at batch 3 vs the indexed
    # dequantisation times x, within 2e-4 * max(1, |want|); the device dequantisation bit for bit
    raw, x, in_dim, out_dim = qk_test_rows(kind)
    qtype = Q5_K if kind == 5 else Q6_K
    m = (gpu.UploadQ5KMatrixRows if kind == 5 else gpu.UploadQ6KMatrixRows)(raw, in_dim, out_dim)
    assert m.ResidentBytes() == raw.size
    got = (gpu.GemvQ5KBatch if kind == 5 else gpu.GemvQ6KBatch)(x, 3, m).reshape(3, out_dim)
    deq = orc.gguf_dequant(raw, qtype, in_dim, out_dim)
    for b in range(3):
        want = deq.astype(np.float64) @ x[b * in_dim:(b + 1) * in_dim].astype(np.float64)
        assert np.all(np.abs(got[b] - want) <= 2e-4 * np.maximum(1.0, np.abs(want)))
    out = out_with_canary(gpu, out_dim * in_dim)
    m.Dequant(out)
    gpu.Sync()
    assert np.array_equal(read_and_check_canary(out, out_dim * in_dim).view(np.uint32), deq.reshape(-1).view(np.uint32))
    with pytest.raises(gpu.GophError):  # the other kind's entry point refuses this matrix (qk.go:403-405)
        (gpu.GemvQ6KBatch if kind == 5 else gpu.GemvQ5KBatch)(x, 3, m)
    m.Free(); out.Free()


@pytest.mark.parametrize("rows", [0, 1, 2, 4])
@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("out_dim,in_dim", [(1024, 4096), (4096, 4096), (259, 2816), (2048, 768)])
def test_gemv_parity(gpu, pkg, qtype, out_dim, in_dim, rows):
    gpu.SetOption("gguf_rows", rows)
    gpu.SetOption("gguf_layout", 1)   # the CUDA-core streaming kernels
    try:
        raw = make(pkg, qtype, ("gemv", out_dim, in_dim), out_dim, in_dim)
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
        x = pkg.synth.activations(("gemv", in_dim), in_dim, bf16=False)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        m.ProjectBatchToBuffer(out, xo, 1)
        gpu.Sync()
        got = read_and_check_canary(out, out_dim)
        want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL
        for t in (m, xo, out):
            t.Free()
    finally:
        gpu.SetOption("gguf_rows", 0)
        gpu.SetOption("gguf_layout", 0)


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("batch", [2, 3, 4, 5, 8, 11])
def test_batched_projection(gpu, pkg, qtype, batch):
    out_dim, in_dim = 1024, 2048
    raw = make(pkg, qtype, "batch", out_dim, in_dim)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    x = pkg.synth.activations(("batch", batch), batch * in_dim, bf16=False)
    xo = gpu.from_numpy(x)
    out = out_with_canary(gpu, batch * out_dim)
    gpu.GemvQ4KBatchToBuffer(out, xo, batch, m)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, batch=batch, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    for t in (m, xo, out):
        t.Free()


def test_malformed_calls_raise(gpu, pkg):
    raw = make(pkg, Q4_K, "bad", 4, 256)
    with pytest.raises(gpu.GophError):
        gpu.UploadQ4KMatrixRaw(raw, 255, 4)
    with pytest.raises(gpu.GophError):
        gpu.UploadQ4KMatrixRaw(raw[:-1], 256, 4)
    with pytest.raises(gpu.GophError):
        gpu.UploadGGUFMatrix(10, raw, 256, 4)  # Q2_K is not on this path
    with pytest.raises(gpu.GophError):
        gpu.UploadQ5KMatrixRows(raw, 256, 4)   # 144-byte blocks where 176 are due
    with pytest.raises(gpu.GophError):
        gpu.UploadQ6KMatrixRows(make(pkg, Q6_K, "bad", 4, 256), 128, 4)
    m = gpu.UploadQ4KMatrixRaw(raw, 256, 4)
    x = gpu.Malloc(256); out = out_with_canary(gpu, 4)
    with pytest.raises(gpu.GophError):
        m.ProjectBatchToBuffer(out, x, 2)
    with pytest.raises(gpu.GophError):
        m.ProjectBatchToBuffer(out, x, 0)
    gpu.Sync()
    assert np.all(out.Download() == F(123.0))
    m.Free(); m.Free()
    with pytest.raises(gpu.GophError):
        m.ProjectBatchToBuffer(out, x, 1)
    x.Free(); out.Free()


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("out_dim,in_dim", [(14336, 4096), (4096, 14336), (128256, 4096)])
def test_full_size_against_device_dequant(gpu, pkg, qtype, out_dim, in_dim):
    """Llama-3-8B shapes: fused projection vs bit-exact device dequantisation and an f64 product."""
    import torch
    raw = make(pkg, qtype, ("full", out_dim, in_dim), out_dim, in_dim)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    x = pkg.synth.activations(("full", in_dim), in_dim, bf16=False)
    xt = torch.from_numpy(x).cuda()
    deq = torch.empty(out_dim * in_dim, dtype=torch.float32, device="cuda")
    m.Dequant(gpu.wrap(deq.data_ptr(), deq.numel() * 4))
    out = torch.empty(out_dim, dtype=torch.float32, device="cuda")
    m.ProjectBatchToBuffer(gpu.wrap(out.data_ptr(), out_dim * 4), gpu.wrap(xt.data_ptr(), in_dim * 4), 1)
    gpu.Sync()
    ref = deq.view(out_dim, in_dim).double() @ xt.double()
    assert pkg.synth.rel_err(out.cpu().numpy(), ref.cpu().numpy()) <= TOL
    # spot-check the dequantised rows against the oracle (first and last 8 rows)
    rb = orc.gguf_row_bytes(qtype, in_dim)
    for r0 in (0, out_dim - 8):
        want = orc.gguf_dequant(raw[r0 * rb:(r0 + 8) * rb], qtype, in_dim, 8).reshape(-1)
        got = deq[r0 * in_dim:(r0 + 8) * in_dim].cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    m.Free()


# ---- the tensor-core layout (gguf_layout=2: every matrix whose in_dim is a multiple of 256) ----

@pytest.fixture
def tiled_layout(gpu):
    gpu.SetOption("gguf_layout", 2)
    yield
    gpu.SetOption("gguf_layout", 0)
    assert gpu.KernelStatus() == 0   # no bounded wait gave up


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("out_dim,in_dim", [(128, 256), (64, 4096), (300, 512), (259, 2816)])
def test_tiled_dequant_bit_exact(gpu, pkg, tiled_layout, qtype, out_dim, in_dim):
    raw = make(pkg, qtype, "deq-t", out_dim, in_dim)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    padded = (out_dim + 127) // 128 * 128
    # bytes per row and 256 elements, rows padded to the 128-row tile: the file's for Q8_0 and Q4_K; Q5_K and
    # Q6_K are written out as one byte per weight (+ 16 / 32 bytes of scales) for the tensor cores
    per_chunk = {Q8_0: 272, Q4_K: 144, Q5_K: 272, Q6_K: 288}[qtype]
    assert m.ResidentBytes() == padded * (in_dim // 256) * per_chunk
    out = out_with_canary(gpu, out_dim * in_dim)
    m.Dequant(out)
    gpu.Sync()
    got = read_and_check_canary(out, out_dim * in_dim)
    want = orc.gguf_dequant(raw, qtype, in_dim, out_dim, nthreads=8).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    m.Free(); out.Free()


@pytest.mark.parametrize("digits", [4, 3])
@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("out_dim,in_dim", [(1024, 4096), (4096, 4096), (259, 2816), (2048, 768), (64, 256), (19000, 1024)])
def test_tiled_gemv_parity(gpu, pkg, tiled_layout, qtype, out_dim, in_dim, digits):
    gpu.SetOption("mlx_digits", digits)
    try:
        raw = make(pkg, qtype, ("gemv-t", out_dim, in_dim), out_dim, in_dim)
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
        # three digits carry 20 bits under the block maximum: meant for bf16-valued activations
        x = pkg.synth.activations(("gemv-t", in_dim), in_dim, bf16=(digits == 3))
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        m.ProjectBatchToBuffer(out, xo, 1)
        gpu.Sync()
        got = read_and_check_canary(out, out_dim)
        want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL, pkg.synth.rel_err(got, want)
        out2 = out_with_canary(gpu, out_dim)
        m.ProjectBatchToBuffer(out2, xo, 1)
        gpu.Sync()
        assert np.array_equal(read_and_check_canary(out2, out_dim).view(np.uint32), got.view(np.uint32))  # run-to-run identical
        for t in (m, xo, out, out2):
            t.Free()
    finally:
        gpu.SetOption("mlx_digits", 4)


@pytest.mark.parametrize("splits", [1, 2, 3, 16])
@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
def test_tiled_k_splits(gpu, pkg, tiled_layout, qtype, splits):
    out_dim, in_dim = 700, 4096
    gpu.SetOption("mlx_splits", splits)
    try:
        raw = make(pkg, qtype, "split-t", out_dim, in_dim)
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
        x = pkg.synth.activations("split-t", in_dim, bf16=False)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        m.ProjectBatchToBuffer(out, xo, 1)
        gpu.Sync()
        want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, nthreads=8)
        assert pkg.synth.rel_err(read_and_check_canary(out, out_dim), want) <= TOL
        for t in (m, xo, out):
            t.Free()
    finally:
        gpu.SetOption("mlx_splits", 0)


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("batch", [2, 3, 4, 5, 8, 11])
def test_tiled_batched_projection(gpu, pkg, tiled_layout, qtype, batch):
    out_dim, in_dim = 777, 2048
    raw = make(pkg, qtype, "batch-t", out_dim, in_dim)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    x = pkg.synth.activations(("batch-t", batch), batch * in_dim, bf16=False)
    xo = gpu.from_numpy(x)
    out = out_with_canary(gpu, batch * out_dim)
    m.ProjectBatchToBuffer(out, xo, batch)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, batch, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    for t in (m, xo, out):
        t.Free()


def test_tiled_wide_dynamic_range(gpu, pkg, tiled_layout):
    # activations spanning 2^-20 .. 2^10 inside one block: the integer digits keep 26 bits under the block maximum
    out_dim, in_dim = 256, 1024
    rng = pkg.synth.rng("range-t")
    x = (rng.standard_normal(in_dim) * np.exp2(rng.integers(-20, 11, in_dim))).astype(F)
    for qtype in (Q8_0, Q4_K):
        raw = make(pkg, qtype, "range-t", out_dim, in_dim)
        m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
        xo = gpu.from_numpy(x)
        out = gpu.Malloc(out_dim)
        m.ProjectBatchToBuffer(out, xo, 1)
        gpu.Sync()
        want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim)
        assert pkg.synth.rel_err(out.Download(), want) <= TOL
        for t in (m, xo, out):
            t.Free()


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K])
def test_tiled_product_while_l2_writes_back(gpu, pkg, qtype):
    """Loads arrive late and out of order when the L2 is full of dirty lines (here: a 600 MB memset
    right before the launch); the pipeline's waits must hold under that timing too."""
    out_dim, in_dim = 128256, 4096
    raw = make(pkg, qtype, ("wb", out_dim), out_dim, in_dim)
    x = pkg.synth.activations(("wb", in_dim), in_dim, bf16=False)
    want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, nthreads=16)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    xo, out, junk = gpu.from_numpy(x), gpu.Malloc(out_dim), gpu.Malloc(150_000_000)
    for _ in range(4):
        junk.Zero()
        m.ProjectBatchToBuffer(out, xo, 1)
        gpu.Sync()
        assert pkg.synth.rel_err(out.Download(), want) <= TOL
    assert gpu.KernelStatus() == 0
    for t in (m, xo, out, junk):
        t.Free()


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("out_dim,in_dim", [(1024, 4096), (300, 256), (2048, 8192), (640, 14336)])
def test_tiled_fused_and_separate_preparation_agree(gpu, pkg, tiled_layout, qtype, out_dim, in_dim, batch):
    raw = make(pkg, qtype, ("fuse-t", out_dim, in_dim), out_dim, in_dim)
    m = gpu.UploadGGUFMatrix(qtype, raw, in_dim, out_dim)
    x = pkg.synth.activations(("fuse-t", in_dim, batch), batch * in_dim, bf16=False)
    xo = gpu.from_numpy(x)
    want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, batch, nthreads=8)
    got = []
    try:
        for fuse in (1, 0):
            gpu.SetOption("mlx_fuse", fuse)
            out = out_with_canary(gpu, batch * out_dim)
            m.ProjectBatchToBuffer(out, xo, batch)
            gpu.Sync()
            got.append(read_and_check_canary(out, batch * out_dim))
            out.Free()
    finally:
        gpu.SetOption("mlx_fuse", 1)
    assert pkg.synth.rel_err(got[0], want) <= TOL
    assert np.array_equal(got[0].view(np.uint32), got[1].view(np.uint32))
    m.Free(); xo.Free()


@pytest.mark.parametrize("qname,layout", [("q4k", 2), ("q4k", 1), ("q8_0", 2)])
@pytest.mark.parametrize("batch", [1, 3])
def test_pair_projection_shares_x(gpu, pkg, qname, layout, batch):
    # nvidia.ProjectQ4PairToBuffers (runtime/gguf_matrix.go:82-111): gate and up on one x equal two
    # single projections bit for bit, and the oracle within the product tolerance
    in_dim, out_a, out_b = 1024, 768, 512
    qt = gpu.GGUF_Q4_K if qname == "q4k" else gpu.GGUF_Q8_0
    gen = pkg.synth.q4k_matrix if qname == "q4k" else pkg.synth.q8_0_matrix
    ra, rb = gen(("pair", "a"), out_a, in_dim), gen(("pair", "b"), out_b, in_dim)
    gpu.SetOption("gguf_layout", layout)
    try:
        ma, mb = gpu.UploadGGUFMatrix(qt, ra, in_dim, out_a), gpu.UploadGGUFMatrix(qt, rb, in_dim, out_b)
    finally:
        gpu.SetOption("gguf_layout", 0)
    x = pkg.synth.activations(("pair", batch), batch * in_dim, bf16=False)
    xo = gpu.from_numpy(x)
    oa, ob = out_with_canary(gpu, batch * out_a), out_with_canary(gpu, batch * out_b)
    gpu.ProjectQ4PairToBuffers(oa, ob, xo, batch, ma, mb)
    gpu.Sync()
    ga, gb = read_and_check_canary(oa, batch * out_a), read_and_check_canary(ob, batch * out_b)
    sa, sb = out_with_canary(gpu, batch * out_a), out_with_canary(gpu, batch * out_b)
    ma.ProjectBatchToBuffer(sa, xo, batch)
    mb.ProjectBatchToBuffer(sb, xo, batch)
    gpu.Sync()
    assert np.array_equal(ga.view(np.uint32), read_and_check_canary(sa, batch * out_a).view(np.uint32))
    assert np.array_equal(gb.view(np.uint32), read_and_check_canary(sb, batch * out_b).view(np.uint32))
    assert pkg.synth.rel_err(ga, orc.gguf_gemv(x, ra, qt, in_dim, out_a, batch, nthreads=8)) <= TOL
    assert pkg.synth.rel_err(gb, orc.gguf_gemv(x, rb, qt, in_dim, out_b, batch, nthreads=8)) <= TOL
    with pytest.raises(gpu.GophError):
        gpu.ProjectQ4PairToBuffers(oa, ob, xo, batch, ma, None)
    for t_ in (ma, mb, xo, oa, ob, sa, sb):
        t_.Free()
