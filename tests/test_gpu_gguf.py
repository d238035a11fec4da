"""GPU parity of the GGUF Q8_0 / Q4_K path against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary
from oracle import binding as orc
from test_oracle_pins import q4k_test_rows, q8_0_test_rows

pytestmark = pytest.mark.gpu

Q8_0, Q4_K = orc.Q8_0, orc.Q4_K


def make(pkg, qtype, key, out_dim, in_dim):
    gen = pkg.synth.q8_0_matrix if qtype == Q8_0 else pkg.synth.q4k_matrix
    return gen(key, out_dim, in_dim)


@pytest.mark.parametrize("qtype,out_dim,in_dim", [(Q8_0, 64, 4096), (Q8_0, 3, 32), (Q8_0, 17, 96),
                                                   (Q4_K, 64, 4096), (Q4_K, 2, 256), (Q4_K, 9, 2816)])
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


@pytest.mark.parametrize("rows", [0, 1, 2, 4])
@pytest.mark.parametrize("qtype", [Q8_0, Q4_K])
@pytest.mark.parametrize("out_dim,in_dim", [(1024, 4096), (4096, 4096), (259, 2816), (2048, 768)])
def test_gemv_parity(gpu, pkg, qtype, out_dim, in_dim, rows):
    gpu.SetOption("gguf_rows", rows)
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


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K])
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
        gpu.UploadGGUFMatrix(14, raw, 256, 4)  # Q6_K is not on this path
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


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K])
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
