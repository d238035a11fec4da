"""The allocation-free GEMV entry point against the regular one, through the C ABI.

goph_mlx_gemv_noalloc exists for callers that cannot allocate device memory where they need a
product (a serving loop with a fully committed memory budget, a thread that must not take the
allocator's synchronisation mid-step, code already capturing its stream).  Its scratch is a
fixed array inside the library, shared by every call, so the test runs it twice in a row and
demands the regular entry point's answer both times.  This file is collected last on purpose:
a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

from gpu_util import F, TOL, out_with_canary, read_and_check_canary

pytestmark = pytest.mark.gpu


def tiled_weight(gpu, pkg, key, out_dim, in_dim):
    w, s, b = pkg.synth.mlx_weight(key, out_dim, in_dim, 64)
    gpu.SetOption("mlx_layout", 2)
    try:
        return gpu.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
    finally:
        gpu.SetOption("mlx_layout", 0)


@pytest.mark.parametrize("out_dim,in_dim", [(4096, 4096), (1000, 1024), (18944, 2048)])
def test_noalloc_matches_regular_entry_point_twice(gpu, pkg, out_dim, in_dim):
    import torch
    from oracle import binding as orc
    w, s, b = pkg.synth.mlx_weight(("na", out_dim, in_dim), out_dim, in_dim, 64)
    h = tiled_weight(gpu, pkg, ("na", out_dim, in_dim), out_dim, in_dim)
    x1 = pkg.synth.activations(("na", in_dim, 1), in_dim, bf16=False)
    x2 = pkg.synth.activations(("na", in_dim, 2), in_dim, bf16=False)
    for x in (x1, x2):  # two calls in a row share the built-in scratch
        xo = gpu.from_numpy(x)
        ref = out_with_canary(gpu, out_dim)
        gpu.GemvMLX(ref, xo, h)
        gpu.Sync()
        want = read_and_check_canary(ref, out_dim)
        out = out_with_canary(gpu, out_dim)
        gpu.GemvMLXNoAlloc(out, xo, h)   # the first call on the device resolves the scratch address and loads the kernels
        gpu.Sync()
        # the entry point's one promise: the device's free memory is the same before and after a call
        free_before = torch.cuda.mem_get_info()[0]
        gpu.GemvMLXNoAlloc(out, xo, h)
        gpu.Sync()
        assert torch.cuda.mem_get_info()[0] == free_before
        got = read_and_check_canary(out, out_dim)
        # the same kernel on the same digits: the regular entry point's bits, and the oracle's answer
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert pkg.synth.rel_err(got, orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64, nthreads=8)) <= TOL
        assert gpu.GemvMLXNoAllocStatus() == 0
        for t in (xo, ref, out):
            t.Free()
    h.Free()


def test_noalloc_rejects_what_its_scratch_cannot_hold(gpu, pkg):
    # above the in_dim limit of the built-in scratch
    big = tiled_weight(gpu, pkg, "na-big", 128, 16384 + 256)
    x = gpu.Malloc(16384 + 256); out = out_with_canary(gpu, 128)
    with pytest.raises(gpu.GophError) as e:
        gpu.GemvMLXNoAlloc(out, x, big)
    assert e.value.code == 4 and "16384" in str(e.value)
    # a row-major weight (group size 32) has no tiled layout
    w, s, b = pkg.synth.mlx_weight("na-rm", 64, 256, 32)
    rm = gpu.UploadMLXWeight(w, s, b, 256, 64, 32, True)
    with pytest.raises(gpu.GophError) as e:
        gpu.GemvMLXNoAlloc(out, x, rm)
    assert e.value.code == 4 and "tiled" in str(e.value)
    # short buffers
    ok = tiled_weight(gpu, pkg, "na-ok", 256, 512)
    with pytest.raises(gpu.GophError):
        gpu.GemvMLXNoAlloc(gpu.wrap(out.Ptr, 255 * 4), x, ok)
    gpu.Sync()
    assert np.all(out.Download() == F(123.0))
    for t in (big, rm, ok, x, out):
        t.Free()
