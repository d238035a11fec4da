"""GPU parity of the small-batch tensor-core products (9 to 256 activation rows, MLX 4-bit and FP8
E4M3) against the CPU oracle, through the C ABI: small ragged shapes, and the Llama-3-70B
projection shapes 8192x8192, 28672x8192 and 8192x28672 at 16, 64 and 256 rows."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc

pytestmark = pytest.mark.gpu


def _bf16_buffer(gpu, x):
    """x (bf16-valued f32) as a device buffer of bf16 bit patterns."""
    return gpu.from_numpy(gpu.to_bf16_bits(x))


def _fp8_bytes(key, out_dim, in_dim, all_codes=False):
    """E4M3 bytes of clip(N(0,1), +-448) (torch's encoder: fast enough for 235M weights), or every
    code but the two NaNs uniformly (subnormals and the largest magnitudes included)."""
    import zlib

    import torch
    g = torch.Generator().manual_seed(zlib.crc32(repr(key).encode()))
    if all_codes:
        w = torch.randint(0, 256, (out_dim * in_dim,), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
        w[(w & 0x7F) == 0x7F] = 0x3A
        return w
    return torch.randn(out_dim * in_dim, generator=g).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()


# ---------------------------------------------------------------------------------- MLX 4-bit
@pytest.mark.parametrize("xkind", ["f32", "bf16"])
@pytest.mark.parametrize("batch", [9, 16, 17, 33, 64, 100])
@pytest.mark.parametrize("out_dim,in_dim", [(300, 1024), (1024, 512)])
def test_mlx_small_shapes(gpu, pkg, out_dim, in_dim, batch, xkind):
    # backends/mlx/gemm_test.go:29-66: every batch row is the batch-1 product of that row of x
    gpu.SetOption("mlx_layout", 2)
    try:
        w, s, b = pkg.synth.mlx_weight(("gemm", out_dim, in_dim), out_dim, in_dim, 64)
        h = gpu.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
    finally:
        gpu.SetOption("mlx_layout", 0)
    x = pkg.synth.activations(("gemm", batch, in_dim, xkind), batch * in_dim, bf16=(xkind == "bf16"))
    out = out_with_canary(gpu, batch * out_dim)
    if xkind == "bf16":
        xo = _bf16_buffer(gpu, x)
        gpu.GemmMLXBF16(out, xo, h, batch)
    else:
        xo = gpu.from_numpy(x)
        gpu.GemmMLX(out, xo, h, batch)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.mlx_gemm(x, batch, w, s, b, out_dim, in_dim, 64, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    assert gpu.KernelStatus() == 0
    for t in (h, xo, out):
        t.Free()


def test_mlx_bf16_entry_rejects_row_major(gpu, pkg):
    w, s, b = pkg.synth.mlx_weight("rm", 64, 256, 64)
    h = gpu.UploadMLXWeight(w, s, b, 256, 64, 64, True)  # small: row-major
    xo, out = gpu.MallocBytes(16 * 256 * 2), gpu.Malloc(16 * 64)
    with pytest.raises(gpu.GophError) as e:
        gpu.GemmMLXBF16(out, xo, h, 16)
    assert "tiled layout" in str(e.value)
    for t in (h, xo, out):
        t.Free()


def _row_sample(out_dim):
    """Rows of the first tile, a middle tile and the last (possibly partial) tile."""
    mid = (out_dim // 2) // 128 * 128
    rows = np.concatenate([np.arange(0, 128), np.arange(mid, mid + 128), np.arange(max(out_dim - 128, 0), out_dim)])
    return np.unique(rows)


@pytest.mark.parametrize("out_dim,in_dim", [(8192, 8192), (28672, 8192), (8192, 28672)])
def test_mlx_llama70b_shapes(gpu, pkg, out_dim, in_dim):
    w, s, b = pkg.synth.mlx_weight(("l70", out_dim, in_dim), out_dim, in_dim, 64)
    h = gpu.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
    rows = _row_sample(out_dim)
    wr = np.ascontiguousarray(w.reshape(out_dim, in_dim // 8)[rows]).reshape(-1)
    sr = np.ascontiguousarray(s.reshape(out_dim, in_dim // 64)[rows]).reshape(-1)
    br = np.ascontiguousarray(b.reshape(out_dim, in_dim // 64)[rows]).reshape(-1)
    xfull = pkg.synth.activations(("l70x", in_dim), 256 * in_dim, bf16=True)
    want_all = orc.mlx_gemm(xfull, 256, wr, sr, br, len(rows), in_dim, 64, nthreads=16).reshape(256, len(rows))
    x32, x16 = gpu.from_numpy(xfull), _bf16_buffer(gpu, xfull)
    gemv = None
    for batch in (16, 64, 256):
        want = want_all[:batch]
        for entry in ("bf16", "f32"):
            if entry == "f32" and batch == 256:
                continue  # sixteen passes of the same kernel the batch-64 case runs four times
            out = out_with_canary(gpu, batch * out_dim)
            if entry == "bf16":
                gpu.GemmMLXBF16(out, x16, h, batch)
            else:
                gpu.GemmMLX(out, x32, h, batch)
            gpu.Sync()
            got = read_and_check_canary(out, batch * out_dim).reshape(batch, out_dim)
            assert pkg.synth.rel_err(got[:, rows], want) <= TOL, (entry, batch)
            if gemv is None:
                # row 0 of the batch against the batch-1 product (the integer tensor-core kernel)
                o1 = out_with_canary(gpu, out_dim)
                gpu.GemvMLX(o1, x32, h)
                gpu.Sync()
                gemv = read_and_check_canary(o1, out_dim)
                o1.Free()
            assert pkg.synth.rel_err(got[0], gemv) <= TOL
            out.Free()
    assert gpu.KernelStatus() == 0
    for t in (h, x32, x16):
        t.Free()


# ---------------------------------------------------------------------------------- FP8 E4M3
def test_fp8_tiled_dequant_bit_exact_all_codes(gpu, pkg):
    out_dim, in_dim = 200, 512
    w = _fp8_bytes("deq", out_dim, in_dim, all_codes=True)
    scale = pkg.synth.fp8_linear("deq", out_dim, 16)[1]
    gpu.SetOption("fp8_layout", 2)
    try:
        lin = gpu.UploadFP8E4M3Linear(w, scale, None, out_dim, in_dim)
    finally:
        gpu.SetOption("fp8_layout", 0)
    out = out_with_canary(gpu, out_dim * in_dim)
    gpu.DequantFP8E4M3(out, lin)
    gpu.Sync()
    got = read_and_check_canary(out, out_dim * in_dim)
    want = orc.fp8_dequant(w, scale, out_dim, in_dim).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    lin.Free(); out.Free()


@pytest.mark.parametrize("xkind", ["f32", "bf16"])
@pytest.mark.parametrize("batch", [1, 3, 8, 16, 40, 64, 100])
@pytest.mark.parametrize("out_dim,in_dim,all_codes", [(300, 1024, True), (1024, 512, False)])
def test_fp8_small_shapes(gpu, pkg, out_dim, in_dim, all_codes, batch, xkind):
    # every E4M3 code (subnormals, +-448) goes to the tensor cores
    w = _fp8_bytes(("g", out_dim, in_dim), out_dim, in_dim, all_codes=all_codes)
    _, scale, bias = pkg.synth.fp8_linear(("g", out_dim), out_dim, 16, bias=True)
    gpu.SetOption("fp8_layout", 2)
    try:
        lin = gpu.UploadFP8E4M3Linear(w, scale, bias, out_dim, in_dim)
    finally:
        gpu.SetOption("fp8_layout", 0)
    x = pkg.synth.activations(("g", batch, in_dim, xkind), batch * in_dim, bf16=(xkind == "bf16"))
    out = out_with_canary(gpu, batch * out_dim)
    if xkind == "bf16":
        xo = _bf16_buffer(gpu, x)
        gpu.GemmFP8E4M3BF16Buffer(out, xo, batch, lin)
    else:
        xo = gpu.from_numpy(x)
        gpu.GemmFP8E4M3Buffer(out, xo, batch, lin)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.fp8_batch_gemv(x, batch, w, scale, bias, out_dim, in_dim, avx2=True, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    assert gpu.KernelStatus() == 0
    for t in (lin, xo, out):
        t.Free()


@pytest.mark.parametrize("xkind", ["f32", "bf16"])
@pytest.mark.parametrize("splits", [1, 2, 3, 7])
def test_fp8_k_splits(gpu, pkg, splits, xkind):
    # the K range of a tile shared by several CTAs (partial sums through device scratch, added in split order)
    out_dim, in_dim, batch = 700, 4096, 5
    w = _fp8_bytes(("ks", out_dim, in_dim), out_dim, in_dim)
    _, scale, bias = pkg.synth.fp8_linear(("ks", out_dim), out_dim, 16, bias=True)
    gpu.SetOption("fp8_layout", 2)
    gpu.SetOption("mlx_splits", splits)
    try:
        lin = gpu.UploadFP8E4M3Linear(w, scale, bias, out_dim, in_dim)
        x = pkg.synth.activations(("ks", xkind), batch * in_dim, bf16=(xkind == "bf16"))
        out = out_with_canary(gpu, batch * out_dim)
        if xkind == "bf16":
            xo = _bf16_buffer(gpu, x)
            gpu.GemmFP8E4M3BF16Buffer(out, xo, batch, lin)
        else:
            xo = gpu.from_numpy(x)
            gpu.GemmFP8E4M3Buffer(out, xo, batch, lin)
        gpu.Sync()
    finally:
        gpu.SetOption("fp8_layout", 0)
        gpu.SetOption("mlx_splits", 0)
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.fp8_batch_gemv(x, batch, w, scale, bias, out_dim, in_dim, avx2=True, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    assert gpu.KernelStatus() == 0
    for t in (lin, xo, out):
        t.Free()


def test_fp8_activations_of_wide_dynamic_range(gpu, pkg):
    # the activation pieces are e4m3 values under one power-of-two scale per row: elements 2^30 apart in
    # one row, an all-zero row and a row of tiny values must all come out at f32 level
    out_dim, in_dim, batch = 384, 2048, 4
    w = _fp8_bytes("dyn", out_dim, in_dim)
    _, scale, _ = pkg.synth.fp8_linear(("dyn", out_dim), out_dim, 16)
    g = pkg.synth.rng("dyn-x")
    x = g.standard_normal(batch * in_dim).astype(F).reshape(batch, in_dim)
    x[0] *= np.exp2(g.integers(-20, 11, in_dim)).astype(F)
    x[1] = 0
    x[2] *= F(1e-30)
    x[3, ::7] *= F(1e6)
    x = x.reshape(-1)
    gpu.SetOption("fp8_layout", 2)
    try:
        lin = gpu.UploadFP8E4M3Linear(w, scale, None, out_dim, in_dim)
    finally:
        gpu.SetOption("fp8_layout", 0)
    xo, out = gpu.from_numpy(x), out_with_canary(gpu, batch * out_dim)
    gpu.GemmFP8E4M3Buffer(out, xo, batch, lin)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim).reshape(batch, out_dim)
    want = orc.fp8_batch_gemv(x, batch, w, scale, None, out_dim, in_dim, avx2=True, nthreads=8).reshape(batch, out_dim)
    for m in range(batch):
        assert pkg.synth.rel_err(got[m], want[m]) <= TOL, m
    assert np.all(got[1] == 0)
    for t in (lin, xo, out):
        t.Free()


def test_fp8_nan_codes_keep_the_row_major_layout(gpu, pkg):
    # the two NaN codes must stay NaN (backends/simd/quant/fp8/fp8.go:85-106): such a matrix is not
    # tiled, its products run on the CUDA-core kernel and the bf16 entry refuses it
    out_dim, in_dim = 256, 512
    w = _fp8_bytes("nan", out_dim, in_dim)
    w[5 * in_dim + 17] = 0x7F
    scale = np.ones(out_dim, dtype=F)
    gpu.SetOption("fp8_layout", 2)
    try:
        lin = gpu.UploadFP8E4M3Linear(w, scale, None, out_dim, in_dim)
    finally:
        gpu.SetOption("fp8_layout", 0)
    x = pkg.synth.activations("nanx", in_dim)
    xo, out = gpu.from_numpy(x), out_with_canary(gpu, out_dim)
    gpu.GemvFP8E4M3Buffer(out, xo, lin)
    gpu.Sync()
    got = read_and_check_canary(out, out_dim)
    assert np.isnan(got[5]) and not np.isnan(np.delete(got, 5)).any()
    x16 = _bf16_buffer(gpu, x)
    with pytest.raises(gpu.GophError) as e:
        gpu.GemmFP8E4M3BF16Buffer(out, x16, 1, lin)
    assert "tensor-core layout" in str(e.value)
    for t in (lin, xo, x16, out):
        t.Free()


@pytest.mark.parametrize("out_dim,in_dim", [(8192, 8192), (28672, 8192), (8192, 28672)])
def test_fp8_llama70b_shapes(gpu, pkg, out_dim, in_dim):
    w = _fp8_bytes(("l70", out_dim, in_dim), out_dim, in_dim)
    _, scale, bias = pkg.synth.fp8_linear(("l70", out_dim), out_dim, 16, bias=True)
    scale = (scale * F(4.0 / np.sqrt(in_dim))).astype(F)
    lin = gpu.UploadFP8E4M3Linear(w, scale, bias, out_dim, in_dim)
    rows = _row_sample(out_dim)
    wr = np.ascontiguousarray(w.reshape(out_dim, in_dim)[rows]).reshape(-1)
    xfull = pkg.synth.activations(("l70x8", in_dim), 256 * in_dim, bf16=True)
    want_all = orc.fp8_batch_gemv(xfull, 256, wr, scale[rows], bias[rows], len(rows), in_dim, avx2=True,
                                  nthreads=16).reshape(256, len(rows))
    x32, x16 = gpu.from_numpy(xfull), _bf16_buffer(gpu, xfull)
    gemv = None
    for batch in (1, 4, 16, 64, 256):
        want = want_all[:batch]
        for entry in ("bf16", "f32"):
            if entry == "f32" and batch == 256:
                continue
            out = out_with_canary(gpu, batch * out_dim)
            if entry == "bf16":
                gpu.GemmFP8E4M3BF16Buffer(out, x16, batch, lin)
            else:
                gpu.GemmFP8E4M3Buffer(out, x32, batch, lin)
            gpu.Sync()
            got = read_and_check_canary(out, batch * out_dim).reshape(batch, out_dim)
            assert pkg.synth.rel_err(got[:, rows], want) <= TOL, (entry, batch)
            if gemv is None:
                gemv = got[0].copy()
            assert pkg.synth.rel_err(got[0], gemv) <= TOL
            out.Free()
    assert gpu.KernelStatus() == 0
    for t in (lin, x32, x16):
        t.Free()
