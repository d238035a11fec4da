"""CPU-side checks of the drop-in boundary: the built library loads and exports every
symbol include/goph_b200.h declares, and argument validation rejects malformed input before
any device work (no compute call is made here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "goph_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(goph_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_python_binds(pkg):
    assert header_symbols() == sorted(pkg.runtime.EXPORTS)


def test_library_exports_every_declared_symbol(pkg):
    if not os.path.exists(pkg.runtime.LIB_PATH):
        pkg.build.build()
    lib = C.CDLL(pkg.runtime.LIB_PATH)
    missing = [s for s in header_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_calls_before_init_fail_cleanly(pkg):
    rt = pkg.runtime
    if not os.path.exists(rt.LIB_PATH):
        pkg.build.build()
    L = rt.lib()
    p = C.c_void_p(0)
    # device 7 is never initialised in the CPU test run
    assert L.goph_malloc(7, C.c_uint64(16), C.byref(p)) == 3  # GOPH_E_NOINIT
    assert b"goph_init" in L.goph_last_error()
    assert L.goph_sm_count(7) == 0
    assert L.goph_set_option(b"no_such_option", 1) == 1
    assert L.goph_set_option(b"mlx_unpack", 9) == 1
    assert L.goph_set_option(b"mlx_unpack", 1) == 0
    # nil / freed handles are rejected, freeing nil is fine (Buffer.Free is nil-safe)
    assert L.goph_mlx_free(None) == 0 and L.goph_gguf_free(None) == 0 and L.goph_fp8_free(None) == 0
    assert L.goph_mlx_gemv(None, C.c_uint64(0), None, C.c_uint64(0), None, None) == 1
    assert L.goph_gguf_project(None, C.c_uint64(0), None, C.c_uint64(0), 1, None, None) == 1
    assert L.goph_fp8_gemm(None, C.c_uint64(0), None, C.c_uint64(0), 1, None, None) == 1


def test_upload_validation_happens_before_device_use(pkg):
    """validateMLXUploadInputs (backends/nvidia/runtime/mlx.go:34-55) and fp8.Linear.Validate
    (backends/simd/quant/fp8/fp8.go:140-158) reject bad shapes without touching a GPU."""
    import numpy as np
    rt = pkg.runtime
    L = rt.lib()
    h = C.c_void_p(0)
    w = np.zeros(8, dtype=np.uint32)
    s = np.zeros(8, dtype=np.float32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    bad = [(0, 4, 64), (64, 0, 64), (64, 4, 0), (60, 4, 64), (64, 4, 48), (12, 4, 4)]
    for in_dim, out_dim, gs in bad:
        rc = L.goph_mlx_upload(7, vp(w), C.c_uint64(8), vp(s), vp(s), C.c_uint64(8), in_dim, out_dim, gs, C.byref(h))
        assert rc == 1, (in_dim, out_dim, gs)
    # short weight / short scales
    assert L.goph_mlx_upload(7, vp(w), C.c_uint64(8), vp(s), vp(s), C.c_uint64(8), 64, 4, 64, C.byref(h)) == 1
    assert L.goph_mlx_upload(7, vp(w), C.c_uint64(8), vp(s), vp(s), C.c_uint64(0), 64, 1, 64, C.byref(h)) == 1
    # well-formed but device 7 not initialised
    assert L.goph_mlx_upload(7, vp(w), C.c_uint64(8), vp(s), vp(s), C.c_uint64(8), 64, 1, 64, C.byref(h)) == 3
    raw = np.zeros(144, dtype=np.uint8)
    assert L.goph_gguf_upload(7, 12, vp(raw), C.c_uint64(144), 255, 1, C.byref(h)) == 1   # not a multiple of 256
    assert L.goph_gguf_upload(7, 8, vp(raw), C.c_uint64(33), 32, 1, C.byref(h)) == 1      # short raw
    assert L.goph_gguf_upload(7, 10, vp(raw), C.c_uint64(144), 256, 1, C.byref(h)) == 4   # Q2_K unsupported
    assert L.goph_gguf_upload(7, 13, vp(raw), C.c_uint64(144), 256, 1, C.byref(h)) == 1   # Q5_K wants 176 bytes
    assert L.goph_gguf_upload(7, 14, vp(raw), C.c_uint64(144), 256, 1, C.byref(h)) == 1   # Q6_K wants 210 bytes
    assert L.goph_gguf_upload(7, 14, vp(raw), C.c_uint64(105), 128, 1, C.byref(h)) == 1   # not a multiple of 256
    # UploadQuantWeight validation (backends/nvidia/runtime/q4.go:30-56)
    qw, gi = np.zeros(32, dtype=np.int32), np.zeros(64, dtype=np.int32)
    sc = np.ones(4, dtype=np.float32)
    gptq = lambda nq, ng, ns, i, o: L.goph_gptq_upload(7, vp(qw), C.c_uint64(nq), vp(gi), C.c_uint64(ng), vp(sc),
                                                        C.c_uint64(ns), i, o, C.byref(h))
    assert gptq(32, 64, 4, 60, 4) == 1 and gptq(31, 64, 4, 64, 4) == 1 and gptq(32, 63, 4, 64, 4) == 1
    assert gptq(32, 64, 3, 64, 4) == 1 and gptq(32, 64, 0, 64, 4) == 1
    gi[5] = 1
    assert gptq(32, 64, 4, 64, 4) == 1      # g_idx names group 1 of 1
    gi[5] = 0
    assert gptq(32, 64, 4, 64, 4) == 3      # well-formed, device 7 not initialised
    assert L.goph_fp8_upload(7, vp(raw), C.c_uint64(6), vp(s), 3, None, 0, 2, 3, C.byref(h)) == 1  # scale len 3
    assert L.goph_fp8_upload(7, vp(raw), C.c_uint64(5), vp(s), 1, None, 0, 2, 3, C.byref(h)) == 1  # weight bytes
