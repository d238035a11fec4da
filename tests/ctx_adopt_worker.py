"""Child process of tests/test_gpu_context.py: the library bound to a driver context the CALLER
created (as the reference does, backends/nvidia/runtime/runtime.go:226-274), with x and out
allocated by the caller's cuMemAlloc in that context.  Prints "ok" and exits 0 on success."""
import ctypes as C
import os
import sys
import threading

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from conftest import load_package  # noqa: E402
from oracle import binding as orc  # noqa: E402


def check(rc, what):
    if rc != 0:
        raise SystemExit("%s failed with CUresult %d" % (what, rc))


def main():
    cu = C.CDLL("libcuda.so.1")
    check(cu.cuInit(0), "cuInit")
    dev = C.c_int(0)
    check(cu.cuDeviceGet(C.byref(dev), 0), "cuDeviceGet")
    ctx = C.c_void_p(0)
    check(cu.cuCtxCreate_v2(C.byref(ctx), 0, dev), "cuCtxCreate")   # current on this thread from here on
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    assert rt.InitCurrentContext() == 0
    try:
        rt.init(0)
    except rt.GophError as e:  # one context per device and process
        assert "adopted context" in str(e)
    else:
        raise SystemExit("goph_init accepted a device that is bound to an adopted context")
    for out_dim, in_dim, layout in ((4096, 4096, 0), (1000, 1024, 2), (640, 512, 1)):   # tensor-core and CUDA-core kernels
        w, s, b = syn.mlx_weight(("ctx", out_dim, in_dim), out_dim, in_dim, 64)
        rt.SetOption("mlx_layout", layout)
        h = rt.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
        rt.SetOption("mlx_layout", 0)
        x = syn.activations(("ctx", in_dim), in_dim, bf16=False)
        xd, od = C.c_uint64(0), C.c_uint64(0)
        check(cu.cuMemAlloc_v2(C.byref(xd), C.c_size_t(in_dim * 4)), "cuMemAlloc")
        check(cu.cuMemAlloc_v2(C.byref(od), C.c_size_t((out_dim + 64) * 4)), "cuMemAlloc")
        canary = np.full(out_dim + 64, 123.0, dtype=np.float32)
        check(cu.cuMemcpyHtoD_v2(xd, x.ctypes.data_as(C.c_void_p), C.c_size_t(x.nbytes)), "cuMemcpyHtoD")
        check(cu.cuMemcpyHtoD_v2(od, canary.ctypes.data_as(C.c_void_p), C.c_size_t(canary.nbytes)), "cuMemcpyHtoD")
        # the product is issued from a thread that has never had a context current (goroutines
        # migrate between OS threads, runtime/runtime.go:258-274): the library binds its own
        failure = []

        def product():
            try:
                rt.GemvMLX(rt.wrap(od.value, out_dim * 4), rt.wrap(xd.value, in_dim * 4), h)
                rt.Sync()
            except Exception as e:  # noqa: BLE001 - reported to the parent thread
                failure.append(e)

        t = threading.Thread(target=product)
        t.start()
        t.join()
        assert not failure, failure
        cur = C.c_void_p(0)
        check(cu.cuCtxGetCurrent(C.byref(cur)), "cuCtxGetCurrent")
        assert cur.value == ctx.value, "the library left another context current"
        got = np.empty(out_dim + 64, dtype=np.float32)
        check(cu.cuMemcpyDtoH_v2(got.ctypes.data_as(C.c_void_p), od, C.c_size_t(got.nbytes)), "cuMemcpyDtoH")
        assert np.all(got[out_dim:] == 123.0), "kernel wrote past the end of out"
        want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64, nthreads=8)
        err = syn.rel_err(got[:out_dim], want)
        assert err <= 2e-3, (out_dim, in_dim, err)
        assert rt.KernelStatus() == 0
        h.Free()
        check(cu.cuMemFree_v2(xd), "cuMemFree")
        check(cu.cuMemFree_v2(od), "cuMemFree")
    check(cu.cuCtxDestroy_v2(ctx), "cuCtxDestroy")
    print("ok")


if __name__ == "__main__":
    main()
