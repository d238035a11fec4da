"""GPU parity of the FP8 E4M3 path against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc

pytestmark = pytest.mark.gpu


def test_decode_table_bit_exact_including_nan_codes(gpu, pkg):
    # backends/simd/quant/fp8/dynamic_test.go:8-36: all 256 codes through the device decoder
    w = np.arange(256, dtype=np.uint8).reshape(16, 16)
    scale = np.ones(16, dtype=F)
    lin = gpu.UploadFP8E4M3Linear(w, scale, None, 16, 16)
    out = gpu.Malloc(256)
    gpu.DequantFP8E4M3(out, lin)
    gpu.Sync()
    got = out.Download()
    want = orc.e4m3_table()
    nan = np.isnan(want)
    assert list(np.nonzero(nan)[0]) == [0x7F, 0xFF]
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    lin.Free(); out.Free()


@pytest.mark.parametrize("out_dim,in_dim,per_tensor", [(64, 4096, False), (33, 80, False), (16, 48, True)])
def test_dequant_bit_exact(gpu, pkg, out_dim, in_dim, per_tensor):
    w, scale, _ = pkg.synth.fp8_linear("deq", out_dim, in_dim)
    if per_tensor:
        scale = scale[:1]
    lin = gpu.UploadFP8E4M3Linear(w, scale, None, out_dim, in_dim)
    out = out_with_canary(gpu, out_dim * in_dim)
    gpu.DequantFP8E4M3(out, lin)
    gpu.Sync()
    got = read_and_check_canary(out, out_dim * in_dim)
    want = orc.fp8_dequant(w, scale, out_dim, in_dim).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    lin.Free(); out.Free()


@pytest.mark.parametrize("rows", [0, 1, 2, 4])
@pytest.mark.parametrize("out_dim,in_dim,bias", [(1024, 4096, False), (8192, 1024, True), (77, 80, True), (5, 77, True)])
def test_gemv_parity(gpu, pkg, out_dim, in_dim, bias, rows):
    gpu.SetOption("fp8_rows", rows)
    try:
        w, scale, b = pkg.synth.fp8_linear(("gemv", out_dim, in_dim), out_dim, in_dim, bias=bias)
        lin = gpu.UploadFP8E4M3Linear(w, scale, b, out_dim, in_dim)
        x = pkg.synth.activations(("gemv", in_dim), in_dim)
        xo = gpu.from_numpy(x)
        out = out_with_canary(gpu, out_dim)
        gpu.GemvFP8E4M3Buffer(out, xo, lin)
        gpu.Sync()
        got = read_and_check_canary(out, out_dim)
        want = orc.fp8_gemv(x, w, scale, b, out_dim, in_dim, avx2=True, nthreads=8)
        assert pkg.synth.rel_err(got, want) <= TOL
        for t in (lin, xo, out):
            t.Free()
    finally:
        gpu.SetOption("fp8_rows", 0)


@pytest.mark.parametrize("batch", [2, 4, 5, 8, 9])
def test_batched_product(gpu, pkg, batch):
    # fp8.Linear.BatchGemvTo (backends/simd/quant/fp8/batch.go:56-87) folds the scale into the
    # dequantised row; the GPU applies it after the dot.  Both stay within the product tolerance.
    out_dim, in_dim = 2048, 1024
    w, scale, b = pkg.synth.fp8_linear("batch", out_dim, in_dim, bias=True)
    lin = gpu.UploadFP8E4M3Linear(w, scale, b, out_dim, in_dim)
    x = pkg.synth.activations(("batch", batch), batch * in_dim)
    xo = gpu.from_numpy(x)
    out = out_with_canary(gpu, batch * out_dim)
    gpu.GemmFP8E4M3Buffer(out, xo, batch, lin)
    gpu.Sync()
    got = read_and_check_canary(out, batch * out_dim)
    want = orc.fp8_batch_gemv(x, batch, w, scale, b, out_dim, in_dim, avx2=True, nthreads=8)
    assert pkg.synth.rel_err(got, want) <= TOL
    host = gpu.GemmFP8E4M3(x, batch, lin)
    assert np.array_equal(host, got)
    for t in (lin, xo, out):
        t.Free()


def test_nan_code_poisons_only_its_row(gpu, pkg):
    out_dim, in_dim = 8, 64
    w, scale, _ = pkg.synth.fp8_linear("nan", out_dim, in_dim)
    w = w.copy(); w[3 * in_dim + 5] = 0x7F
    lin = gpu.UploadFP8E4M3Linear(w, scale, None, out_dim, in_dim)
    x = pkg.synth.activations("nan", in_dim)
    got = gpu.GemvFP8E4M3(x, lin)
    want = orc.fp8_gemv(x, w, scale, None, out_dim, in_dim)
    assert np.isnan(got[3]) and np.isnan(want[3])
    ok = np.arange(out_dim) != 3
    assert pkg.synth.rel_err(got[ok], want[ok]) <= TOL
    lin.Free()


def test_malformed_calls_raise(gpu, pkg):
    w, scale, _ = pkg.synth.fp8_linear("bad", 4, 32)
    with pytest.raises(gpu.GophError):
        gpu.UploadFP8E4M3Linear(w[:-1], scale, None, 4, 32)
    with pytest.raises(gpu.GophError):
        gpu.UploadFP8E4M3Linear(w, scale[:3], None, 4, 32)
    with pytest.raises(gpu.GophError):
        gpu.UploadFP8E4M3Linear(w, scale, np.zeros(3, F), 4, 32)
    lin = gpu.UploadFP8E4M3Linear(w, scale, None, 4, 32)
    x = gpu.Malloc(32); out = out_with_canary(gpu, 4)
    with pytest.raises(gpu.GophError):
        gpu.GemmFP8E4M3Buffer(out, x, 2, lin)
    with pytest.raises(gpu.GophError):
        gpu.GemmFP8E4M3Buffer(out, x, 1, None)
    gpu.Sync()
    assert np.all(out.Download() == F(123.0))
    lin.Free(); lin.Free()
    x.Free(); out.Free()


@pytest.mark.parametrize("out_dim,in_dim", [(8192, 8192), (28672, 8192), (8192, 28672)])
def test_full_size_against_device_dequant(gpu, pkg, out_dim, in_dim):
    """Llama-3-70B shapes: fused product vs bit-exact device dequantisation and an f64 product."""
    import torch
    g = torch.Generator().manual_seed(out_dim + in_dim)
    w = torch.randn(out_dim, in_dim, generator=g).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    scale = (pkg.synth.rng("full", out_dim).uniform(0.5, 2.0, out_dim) / np.sqrt(in_dim)).astype(F)
    lin = gpu.UploadFP8E4M3Linear(w.reshape(-1), scale, None, out_dim, in_dim)
    x = pkg.synth.activations(("full", in_dim), in_dim)
    xt = torch.from_numpy(x).cuda()
    deq = torch.empty(out_dim * in_dim, dtype=torch.float32, device="cuda")
    gpu.DequantFP8E4M3(gpu.wrap(deq.data_ptr(), deq.numel() * 4), lin)
    out = torch.empty(out_dim, dtype=torch.float32, device="cuda")
    gpu.GemvFP8E4M3Buffer(gpu.wrap(out.data_ptr(), out_dim * 4), gpu.wrap(xt.data_ptr(), in_dim * 4), lin)
    gpu.Sync()
    ref = deq.view(out_dim, in_dim).double() @ xt.double()
    assert pkg.synth.rel_err(out.cpu().numpy(), ref.cpu().numpy()) <= TOL
    want = orc.fp8_dequant(w.reshape(-1)[:8 * in_dim], scale[:8], 8, in_dim).reshape(-1)
    assert np.array_equal(deq[:8 * in_dim].cpu().numpy().view(np.uint32), want.view(np.uint32))
    lin.Free()
