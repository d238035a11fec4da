"""GPU parity of the MLX 4-bit path against the CPU oracle, through the C ABI.

Dequantisation is compared bit for bit; products within max relative error 2e-3 of the
oracle's f32 accumulation (floor 1e-3 of the largest output, see synth.rel_err)."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc

pytestmark = pytest.mark.gpu

# [out x in] of one Qwen3-0.6B layer: q, k, v, o, gate, up, down
QWEN3_LAYER = [(2048, 1024), (1024, 1024), (1024, 1024), (1024, 2048), (3072, 1024), (3072, 1024), (1024, 3072)]


def upload(rt, syn, key, out_dim, in_dim, gs=64, layout=2):
    """layout 2: tiled + tensor cores whenever the shape allows, 1: row-major, 0: the library's choice by size."""
    w, s, b = syn.mlx_weight(key, out_dim, in_dim, gs)
    rt.SetOption("mlx_layout", layout)
    try:
        return rt.UploadMLXWeight(w, s, b, in_dim, out_dim, gs, True), (w, s, b)
    finally:
        rt.SetOption("mlx_layout", 0)


@pytest.fixture(autouse=True)
def no_wait_gave_up(gpu):
    """Every device-side wait is bounded; none may have given up during a test."""
    yield
    assert gpu.KernelStatus() == 0


@pytest.mark.parametrize("layout", [2, 1])
@pytest.mark.parametrize("out_dim,in_dim,gs", [(2048, 1024, 64), (1024, 3072, 64), (300, 256, 64), (37, 96, 32), (5, 64, 16), (3, 24, 4), (4, 8, 4)])
def test_dequant_bit_exact(gpu, pkg, out_dim, in_dim, gs, layout):
    h, (w, s, b) = upload(gpu, pkg.synth, "deq", out_dim, in_dim, gs, layout)
    out = out_with_canary(gpu, out_dim * in_dim)
    gpu.DequantMLX(out, h)
    gpu.Sync()
    got = read_and_check_canary(out, out_dim * in_dim)
    want = orc.mlx_dequant(w, s, b, out_dim, in_dim, gs, nthreads=8)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    h.Free(); out.Free()


def test_dequant_bit_exact_f32_scales(gpu, pkg):
    # scales that are not bf16 values take the f32 table on the device
    rng = pkg.synth.rng("f32sb")
    out_dim, in_dim, gs = 64, 256, 64
    w = rng.integers(0, 2**32, size=out_dim * in_dim // 8, dtype=np.uint32)
    s = (rng.random(out_dim * 4, dtype=F) * F(0.1) + F(0.01)).astype(F)
    b = (rng.random(out_dim * 4, dtype=F) * F(0.05)).astype(F)
    h = gpu.UploadMLXWeightNative(w, s, b, in_dim, out_dim, gs)
    out = gpu.Malloc(out_dim * in_dim)
    gpu.DequantMLX(out, h)
    want = orc.mlx_dequant(w, s, b, out_dim, in_dim, gs)
    assert np.array_equal(out.Download().view(np.uint32), want.view(np.uint32))
    x = pkg.synth.activations("f32sb", in_dim, bf16=False)
    xo = gpu.from_numpy(x); o = gpu.Malloc(out_dim)
    gpu.GemvMLX(o, xo, h); gpu.Sync()
    assert pkg.synth.rel_err(o.Download(), orc.mlx_gemv(x, w, s, b, out_dim, in_dim, gs)) <= TOL
    for t in (h, out, xo, o):
        t.Free()


@pytest.mark.parametrize("digits", [4, 3])
@pytest.mark.parametrize("out_dim,in_dim", QWEN3_LAYER)
def test_gemv_qwen3_layer_shapes_tensor_cores(gpu, pkg, out_dim, in_dim, digits):
    # the Qwen3-0.6B projection shapes on the tcgen05 path; bf16-valued activations, 4 or 3 base-128 digits
    gpu.SetOption("mlx_digits", digits)
    try:
        h, (w, s, b) = upload(gpu, pkg.synth, ("cfg0", out_dim, in_dim), out_dim, in_dim)
        x = pkg.synth.activations(("cfg0", in_dim), in_dim)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        gpu.GemvMLX(out, xo, h)
        gpu.Sync()
        got = read_and_check_canary(out, out_dim)
        want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL
        for t in (h, xo, out):
            t.Free()
    finally:
        gpu.SetOption("mlx_digits", 4)


@pytest.mark.parametrize("splits", [0, 1, 2, 3, 16])
@pytest.mark.parametrize("out_dim,in_dim", [(4096, 4096), (1000, 4096), (128, 256), (129, 768), (2048, 14336)])
def test_gemv_tensor_cores_k_splits(gpu, pkg, out_dim, in_dim, splits):
    # the K range of a tile shared by several CTAs: partials added in split order by the last arriver
    gpu.SetOption("mlx_splits", splits)
    try:
        h, (w, s, b) = upload(gpu, pkg.synth, ("split", out_dim, in_dim), out_dim, in_dim)
        x = pkg.synth.activations(("split", in_dim), 2 * in_dim, bf16=False)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, 2 * out_dim)
        gpu.GemmMLX(out, xo, h, 2)
        gpu.Sync()
        got = read_and_check_canary(out, 2 * out_dim)
        again = out_with_canary(gpu, 2 * out_dim)
        gpu.GemmMLX(again, xo, h, 2)
        gpu.Sync()
        assert np.array_equal(got, read_and_check_canary(again, 2 * out_dim))  # run-to-run identical
        want = orc.mlx_gemm(x, 2, w, s, b, out_dim, in_dim, 64, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL
        for t in (h, xo, out, again):
            t.Free()
    finally:
        gpu.SetOption("mlx_splits", 0)


def test_tensor_core_path_handles_wide_dynamic_range(gpu, pkg):
    # activations spanning 2^-20 .. 2^12 inside one group, zeros, and an all-zero group
    out_dim, in_dim = 384, 1024
    h, (w, s, b) = upload(gpu, pkg.synth, "range", out_dim, in_dim)
    rng = pkg.synth.rng("range-x")
    x = (rng.standard_normal(in_dim) * np.exp2(rng.integers(-20, 13, in_dim))).astype(F)
    x[::7] = 0
    x[64:128] = 0
    xo = gpu.from_numpy(x); out = gpu.Malloc(out_dim)
    gpu.GemvMLX(out, xo, h); gpu.Sync()
    assert pkg.synth.rel_err(out.Download(), orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64)) <= TOL
    for t in (h, xo, out):
        t.Free()


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("out_dim,in_dim", QWEN3_LAYER)
def test_gemv_qwen3_layer_shapes(gpu, pkg, out_dim, in_dim, mode):
    gpu.SetOption("mlx_unpack", mode)
    try:
        h, (w, s, b) = upload(gpu, pkg.synth, ("cfg0", out_dim, in_dim), out_dim, in_dim, layout=1)
        x = pkg.synth.activations(("cfg0", in_dim), in_dim)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        gpu.GemvMLX(out, xo, h)
        gpu.Sync()
        got = read_and_check_canary(out, out_dim)
        want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL
        for t in (h, xo, out):
            t.Free()
    finally:
        gpu.SetOption("mlx_unpack", 0)


@pytest.mark.parametrize("rows", [1, 2, 4])
@pytest.mark.parametrize("out_dim,in_dim,gs", [(4096, 4096, 64), (1000, 4096, 128), (333, 768, 32), (1, 64, 64), (7, 2080, 32)])
def test_gemv_row_tiles_and_ragged_shapes(gpu, pkg, out_dim, in_dim, gs, rows):
    gpu.SetOption("mlx_rows", rows)
    gpu.SetOption("mlx_unpack", 0)
    try:
        h, (w, s, b) = upload(gpu, pkg.synth, ("rag", out_dim, in_dim), out_dim, in_dim, gs, layout=1)
        x = pkg.synth.activations(("rag", in_dim), in_dim, bf16=False)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        gpu.GemvMLXDirect(out, xo, h)
        gpu.Sync()
        got = read_and_check_canary(out, out_dim)
        want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, gs, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL
        for t in (h, xo, out):
            t.Free()
    finally:
        gpu.SetOption("mlx_rows", 0)
        gpu.SetOption("mlx_unpack", 0)


@pytest.mark.parametrize("out_dim,in_dim,gs", [(19, 64, 16), (3, 24, 4), (40, 72, 8)])
def test_gemv_generic_group_sizes(gpu, pkg, out_dim, in_dim, gs):
    # group sizes below 32 (the reference's own test shapes) take the generic kernel
    h, (w, s, b) = upload(gpu, pkg.synth, ("gen", out_dim, in_dim), out_dim, in_dim, gs)
    for batch in (1, 3):
        x = pkg.synth.activations(("gen", in_dim, batch), batch * in_dim, bf16=False)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, batch * out_dim)
        gpu.GemmMLX(out, xo, h, batch)
        gpu.Sync()
        got = read_and_check_canary(out, batch * out_dim)
        want = orc.mlx_gemm(x, batch, w, s, b, out_dim, in_dim, gs)
        assert pkg.synth.rel_err(got, want) <= TOL
        xo.Free(); out.Free()
    h.Free()


@pytest.mark.parametrize("layout", [2, 1, 0])
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 5, 7, 8, 9, 13])
def test_gemm_batches(gpu, pkg, batch, layout):
    # backends/mlx/gemm_test.go:29-66 batches, at a projection-sized shape, both kernel families
    out_dim, in_dim, gs = 1536, 2048, 64
    h, (w, s, b) = upload(gpu, pkg.synth, "gemm", out_dim, in_dim, gs, layout)
    x = pkg.synth.activations(("gemm", batch), batch * in_dim)
    xo = gpu.from_numpy(x)
    out = out_with_canary(gpu, batch * out_dim)
    gpu.GemmMLX(out, xo, h, batch)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.mlx_gemm(x, batch, w, s, b, out_dim, in_dim, gs, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    # every batch row equals the batch-1 product of that row (Gemm == repeated GemvTo)
    one = gpu.Malloc(out_dim)
    xr = gpu.from_numpy(x[(batch - 1) * in_dim:])
    gpu.GemvMLX(one, xr, h); gpu.Sync()
    assert pkg.synth.rel_err(got[(batch - 1) * out_dim:], one.Download()) <= 1e-3
    for t in (h, xo, out, one, xr):
        t.Free()


def test_multi_weight_launch_shares_x(gpu, pkg):
    # mlx.Gemv2To (backends/mlx/gemv.go:32-60) generalised: q, k, v in one launch
    in_dim = 1024
    shapes = [2048, 1024, 1024]
    hs, hosts = zip(*[upload(gpu, pkg.synth, ("qkv", i), o, in_dim) for i, o in enumerate(shapes)])
    for batch in (1, 2):
        x = pkg.synth.activations(("qkv", batch), batch * in_dim)
        xo = gpu.from_numpy(x)
        outs = [out_with_canary(gpu, batch * o) for o in shapes]
        gpu.GemmMLXMulti(outs, xo, list(hs), batch)
        gpu.Sync()
        for o_dim, ob, (w, s, b) in zip(shapes, outs, hosts):
            got = read_and_check_canary(ob, batch * o_dim)
            want = orc.mlx_gemm(x, batch, w, s, b, o_dim, in_dim, 64, nthreads=8)
            assert pkg.synth.rel_err(got, want) <= TOL
            ob.Free()
        xo.Free()
    for h in hs:
        h.Free()


def test_host_slice_entry_point(gpu, pkg):
    out_dim, in_dim = 768, 2048  # Qwen3-30B-A3B expert gate/up shape
    h, (w, s, b) = upload(gpu, pkg.synth, "host", out_dim, in_dim)
    x = pkg.synth.activations("host", 2 * in_dim)
    got = gpu.GemmMLXHost(x, h, 2)
    assert pkg.synth.rel_err(got, orc.mlx_gemm(x, 2, w, s, b, out_dim, in_dim, 64)) <= TOL
    h.Free()


def test_reference_small_known_answer(gpu, pkg):
    # backends/mlx/quant_test.go:197-260 through the GPU path (4x8, group 4, x = 1..8)
    out_dim, in_dim, gs = 4, 8, 4
    w = np.zeros(out_dim, dtype=np.uint32)
    for row in range(out_dim):
        for i in range(in_dim):
            w[row] |= np.uint32(((row * in_dim + i) % 16) << (i * 4))
    s = np.full(out_dim * 2, 0.1, dtype=F)
    b = np.full(out_dim * 2, -0.5, dtype=F)
    x = np.arange(1, 9, dtype=F)
    h = gpu.UploadMLXWeight(w, s, b, in_dim, out_dim, gs, False)
    xo = gpu.from_numpy(x); out = gpu.Malloc(out_dim)
    gpu.GemvMLX(out, xo, h); gpu.Sync()
    want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, gs)
    assert np.max(np.abs(out.Download() - want)) <= 1e-4
    for t in (h, xo, out):
        t.Free()


def test_malformed_calls_raise_and_write_nothing(gpu, pkg):
    # backends/nvidia/runtime/mlx_test.go:5-42: short buffers and nil weights must not run
    h, _ = upload(gpu, pkg.synth, "bad", 64, 128)
    x = gpu.Malloc(128); out = out_with_canary(gpu, 64)
    short_x = gpu.Malloc(127); short_out = gpu.Malloc(63)
    with pytest.raises(gpu.GophError):
        gpu.GemvMLX(out, short_x, h)
    with pytest.raises(gpu.GophError):
        gpu.GemvMLX(short_out, x, h)
    with pytest.raises(gpu.GophError):
        gpu.GemmMLX(out, x, h, 0)
    with pytest.raises(gpu.GophError):
        gpu.GemmMLX(out, x, h, 2)
    with pytest.raises(gpu.GophError):
        gpu.GemvMLX(out, x, None)
    with pytest.raises(gpu.GophError):
        gpu.UploadMLXWeight(np.zeros(4, np.uint32), np.zeros(1, F), np.zeros(1, F), 60, 1, 64)
    gpu.Sync()
    assert np.all(out.Download() == F(123.0))
    h.Free(); h.Free()  # Free is idempotent
    with pytest.raises(gpu.GophError):
        gpu.GemvMLX(out, x, h)
    for t in (x, out, short_x, short_out):
        t.Free()


@pytest.mark.parametrize("out_dim,in_dim", [(4096, 4096), (14336, 4096), (4096, 14336), (151936, 1024)])
def test_full_size_against_device_dequant(gpu, pkg, out_dim, in_dim):
    """Llama-3-8B projection shapes and the Qwen3 LM head: the fused GEMV must agree with
    (bit-exact) device dequantisation followed by an f64 product, and be linear in x."""
    import torch
    h, _ = upload(gpu, pkg.synth, ("full", out_dim, in_dim), out_dim, in_dim)
    x = pkg.synth.activations(("full", in_dim), 2 * in_dim)
    xt = torch.from_numpy(x).cuda()
    deq = torch.empty(out_dim * in_dim, dtype=torch.float32, device="cuda")
    gpu.DequantMLX(gpu.wrap(deq.data_ptr(), deq.numel() * 4), h)
    out = torch.empty(2 * out_dim, dtype=torch.float32, device="cuda")
    gpu.GemmMLX(gpu.wrap(out.data_ptr(), out.numel() * 4), gpu.wrap(xt.data_ptr(), xt.numel() * 4), h, 2)
    gpu.Sync()
    ref = (deq.view(out_dim, in_dim).double() @ xt.view(2, in_dim).double().T).T.contiguous().view(-1)
    assert pkg.synth.rel_err(out.cpu().numpy(), ref.cpu().numpy()) <= TOL
    xs = (xt[:in_dim] + xt[in_dim:]).contiguous()
    o1 = torch.empty(out_dim, dtype=torch.float32, device="cuda")
    gpu.GemvMLX(gpu.wrap(o1.data_ptr(), out_dim * 4), gpu.wrap(xs.data_ptr(), in_dim * 4), h)
    gpu.Sync()
    lin = out[:out_dim] + out[out_dim:]
    assert pkg.synth.rel_err(o1.cpu().numpy(), lin.cpu().numpy()) <= 1e-3
    h.Free()


def test_tensor_core_product_while_l2_writes_back(gpu, pkg):
    """Loads arrive late and out of order when the L2 is full of dirty lines (a 600 MB memset right
    before each launch); the pipeline's waits must hold under that timing too."""
    out_dim, in_dim = 128256, 4096
    h, (w, s, b) = upload(gpu, pkg.synth, ("wb", out_dim, in_dim), out_dim, in_dim)
    x = pkg.synth.activations(("wb", in_dim), in_dim)
    want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64, nthreads=16)
    xo, out, junk = gpu.from_numpy(x), gpu.Malloc(out_dim), gpu.Malloc(150_000_000)
    for _ in range(4):
        junk.Zero()
        gpu.GemvMLX(out, xo, h)
        gpu.Sync()
        assert pkg.synth.rel_err(out.Download(), want) <= TOL
    for t in (h, xo, out, junk):
        t.Free()


@pytest.mark.parametrize("digits", [4, 3])
@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("out_dim,in_dim", [(1024, 4096), (300, 256), (4096, 1024), (2048, 8192), (640, 14336)])
def test_fused_and_separate_preparation_agree(gpu, pkg, out_dim, in_dim, batch, digits):
    """With option mlx_fuse narrow launches make the activation digits inside the product kernel
    (one launch instead of two).  Same arithmetic, same bits."""
    h, (w, s, b) = upload(gpu, pkg.synth, ("fuse", out_dim, in_dim), out_dim, in_dim)
    x = pkg.synth.activations(("fuse", in_dim, batch), batch * in_dim, bf16=(digits == 3))
    xo = gpu.from_numpy(x)
    want = orc.mlx_gemm(x, batch, w, s, b, out_dim, in_dim, 64, nthreads=8)
    got = []
    gpu.SetOption("mlx_digits", digits)
    try:
        for fuse in (1, 0):
            gpu.SetOption("mlx_fuse", fuse)
            out = out_with_canary(gpu, batch * out_dim)
            gpu.GemmMLX(out, xo, h, batch)
            gpu.Sync()
            got.append(read_and_check_canary(out, batch * out_dim))
            out.Free()
    finally:
        gpu.SetOption("mlx_fuse", 1)
        gpu.SetOption("mlx_digits", 4)
    assert pkg.synth.rel_err(got[0], want) <= TOL
    assert np.array_equal(got[0].view(np.uint32), got[1].view(np.uint32))
    h.Free(); xo.Free()
