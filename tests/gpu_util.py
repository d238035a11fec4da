"""Helpers shared by the GPU parity tests."""
import numpy as np

F = np.float32
TOL = 2e-3  # max relative error of a product against the f32-accumulating oracle
CANARY = F(123.0)  # the reference's tail sentinel (backends/mlx/gemm_test.go:55)


def out_with_canary(rt, n):
    """Device buffer of n floats followed by 64 sentinel floats."""
    buf = rt.Malloc(n + 64)
    buf.Upload(np.full(n + 64, CANARY, dtype=F))
    return buf


def read_and_check_canary(buf, n):
    host = buf.Download()
    assert np.all(host[n:] == CANARY), "kernel wrote past the end of out"
    return host[:n]
