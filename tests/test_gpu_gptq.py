"""GPU parity of the GPTQ symmetric INT4 path against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc
from test_oracle_pins import gptq_test_case_irregular, gptq_test_case_known

pytestmark = pytest.mark.gpu


def run(gpu, w, x, batch):
    xo = gpu.from_numpy(x)
    out = out_with_canary(gpu, batch * w.OutDim)
    gpu.GemmQ4(out, xo, w, batch)
    gpu.Sync()
    got = read_and_check_canary(out, batch * w.OutDim)
    xo.Free(); out.Free()
    return got


def test_reference_known_values(gpu, pkg):
    # backends/simd/quant/q4/known_values_test.go:62-132: exact answers (small dyadic numbers)
    for case in (gptq_test_case_known, gptq_test_case_irregular):
        qw, gidx, scales, x, in_dim, out_dim = case()
        w = gpu.UploadQuantWeight(qw, gidx, scales, in_dim, out_dim)
        want = orc.gptq_gemm_sym(x, 1, qw, gidx, scales, in_dim, out_dim)
        assert np.array_equal(run(gpu, w, x, 1), want)
        out = out_with_canary(gpu, out_dim * in_dim)
        w.Dequant(out)
        gpu.Sync()
        deq = orc.gptq_dequant_sym(qw, gidx, scales, in_dim, out_dim).reshape(-1)
        assert np.array_equal(read_and_check_canary(out, out_dim * in_dim).view(np.uint32), deq.view(np.uint32))
        w.Free(); out.Free()


@pytest.mark.parametrize("f16_scales", [True, False])
@pytest.mark.parametrize("act_order", [False, True])
@pytest.mark.parametrize("out_dim,in_dim,gs", [(128, 256, 128), (1536, 2048, 128), (2050, 1536, 128), (259, 2816, 64),
                                               (4096, 4096, 32), (64, 512, 8)])
def test_dequant_bit_exact_and_gemv_parity(gpu, pkg, out_dim, in_dim, gs, act_order, f16_scales):
    qw, gidx, sc = pkg.synth.gptq_weight("t", out_dim, in_dim, gs, act_order, f16_scales)
    w = gpu.UploadQuantWeight(qw, gidx, sc, in_dim, out_dim)
    assert w.UsesMLXKernels() == (not act_order)
    out = out_with_canary(gpu, out_dim * in_dim)
    w.Dequant(out)
    gpu.Sync()
    deq = orc.gptq_dequant_sym(qw, gidx, sc, in_dim, out_dim).reshape(-1)
    assert np.array_equal(read_and_check_canary(out, out_dim * in_dim).view(np.uint32), deq.view(np.uint32))
    x = pkg.synth.activations(("gptq", in_dim), in_dim, bf16=False)
    want = orc.gptq_gemm_sym(x, 1, qw, gidx, sc, in_dim, out_dim)
    assert pkg.synth.rel_err(run(gpu, w, x, 1), want) <= TOL
    w.Free(); out.Free()


@pytest.mark.parametrize("act_order", [False, True])
@pytest.mark.parametrize("batch", [2, 3, 4, 5, 8, 11])
def test_batched_product(gpu, pkg, batch, act_order):
    # runtime/gemm_q4_test.go:9-170: GemmQ4 over B rows vs the dequantised product, and vs GemvQ4 per row
    out_dim, in_dim = 1024, 2048
    qw, gidx, sc = pkg.synth.gptq_weight("b", out_dim, in_dim, 128, act_order)
    w = gpu.UploadQuantWeight(qw, gidx, sc, in_dim, out_dim)
    x = pkg.synth.activations(("gptq-b", batch), batch * in_dim, bf16=False)
    got = run(gpu, w, x, batch)
    want = orc.gptq_gemm_sym(x, batch, qw, gidx, sc, in_dim, out_dim)
    assert pkg.synth.rel_err(got, want) <= TOL
    for b in (0, batch - 1):
        one = run(gpu, w, x[b * in_dim:(b + 1) * in_dim], 1)
        assert pkg.synth.rel_err(got[b * out_dim:(b + 1) * out_dim], one) <= TOL
    w.Free()


def test_full_size_regular_goes_through_the_tensor_core_layout(gpu, pkg):
    # Llama-3-8B gate projection: regular g_idx, 58.7 Mi weights -> the tiled MLX layout
    import torch
    out_dim, in_dim = 14336, 4096
    qw, gidx, sc = pkg.synth.gptq_weight("full", out_dim, in_dim, 128)
    w = gpu.UploadQuantWeight(qw, gidx, sc, in_dim, out_dim)
    assert w.UsesMLXKernels()
    x = pkg.synth.activations(("gptq-full", in_dim), in_dim, bf16=False)
    deq = torch.empty(out_dim * in_dim, dtype=torch.float32, device="cuda")
    w.Dequant(gpu.wrap(deq.data_ptr(), deq.numel() * 4))
    got = run(gpu, w, x, 1)
    ref = (deq.view(out_dim, in_dim).double() @ torch.from_numpy(x).cuda().double()).cpu().numpy()
    assert pkg.synth.rel_err(got, ref) <= TOL
    want = orc.gptq_dequant_sym(qw, gidx, sc, in_dim, out_dim)
    assert np.array_equal(deq.cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32))
    w.Free()


def test_malformed_calls_raise(gpu, pkg):
    # runtime/gemm_q4_test.go:172-201 (UploadQuantWeight validation) and :203-240 (dispatch on bad buffers)
    qw, gidx, sc = pkg.synth.gptq_weight("bad", 16, 256, 128)
    for args in [(qw, gidx, sc, 255, 16), (qw, gidx, sc, 0, 16), (qw, gidx, sc, 256, 0), (qw[:-1], gidx, sc, 256, 16),
                 (qw, gidx[:-1], sc, 256, 16), (qw, gidx, sc[:-1], 256, 16), (qw, gidx, sc[:0], 256, 16)]:
        with pytest.raises(gpu.GophError):
            gpu.UploadQuantWeight(*args)
    bad = gidx.copy(); bad[7] = 2
    with pytest.raises(gpu.GophError):
        gpu.UploadQuantWeight(qw, bad, sc, 256, 16)
    bad[7] = -1
    with pytest.raises(gpu.GophError):
        gpu.UploadQuantWeight(qw, bad, sc, 256, 16)
    w = gpu.UploadQuantWeight(qw, gidx, sc, 256, 16)
    x = gpu.Malloc(256); out = out_with_canary(gpu, 16)
    with pytest.raises(gpu.GophError):
        gpu.GemmQ4(out, x, w, 2)
    with pytest.raises(gpu.GophError):
        gpu.GemmQ4(out, x, w, 0)
    gpu.Sync()
    assert np.all(out.Download() == F(123.0))
    w.Free(); w.Free()
    with pytest.raises(gpu.GophError):
        gpu.GemvQ4(out, x, w)
    x.Free(); out.Free()
