"""Multi-rank tests: world_size-2 gloo ranks on CPU for the partitioning logic, and — where the
box has two or more GPUs — one rank per GPU through the C ABI and the peer-memory exchange."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(mode, world, timeout):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "multi_worker.py"), "--mode", mode]
    env = dict(os.environ, OMP_NUM_THREADS="2", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    for rank in range(world):
        assert "rank %d of %d ok" % (rank, world) in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 3])
def test_partitioning_with_gloo_ranks(world):
    launch("cpu", world, 600)


@pytest.mark.gpu
def test_sharded_products_and_exchange_one_rank_per_gpu():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two or more GPUs on the box")
    launch("gpu", min(n, 4) if n != 8 else 8, 900)


@pytest.mark.gpu
def test_exchange_single_rank(gpu, pkg):
    """world = 1: the exchange degenerates to a copy into the own result buffer."""
    import numpy as np
    from oracle import binding as orc
    rt, syn = gpu, pkg.synth
    g = rt.Gather(0, 1, 1 << 16)
    out_dim, in_dim = 1024, 512
    w, s, b = syn.mlx_weight("solo", out_dim, in_dim, 64)
    h = rt.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True)
    for i in range(5):
        x = syn.activations(("solo", i), 2 * in_dim)
        xb = rt.from_numpy(x)
        res = g.GemmMLX(xb, h, 2, 0, out_dim)
        rt.Sync()
        want = orc.mlx_gemm(x, 2, w, s, b, out_dim, in_dim, 64)
        assert syn.rel_err(res.Download(2 * out_dim), want) <= 2e-3
        xb.Free()
    assert g.Status() == 0
    with pytest.raises(rt.GophError):
        g.GemmMLX(rt.Malloc(in_dim), h, 1, 8, out_dim)        # rows past the full output
    with pytest.raises(rt.GophError):
        g.All(rt.Malloc(16), 2, 1 << 16, 1 << 16, 1 << 16)    # past the capacity
    with pytest.raises(rt.GophError):
        rt.Gather(0, 9, 1024)                                 # more ranks than the exchange supports
    h.Free(); g.Free()


def test_shard_rows_partition(pkg):
    sh = pkg.sharding
    for out_dim in (0, 1, 7, 8, 20, 1000, 1024, 151936, 128256):
        for world in (1, 2, 3, 4, 8):
            parts = [sh.shard_rows(out_dim, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == out_dim
            for (a, b), (c, d) in zip(parts, parts[1:]):
                assert b == c and a <= b and c <= d
            assert all(lo % 8 == 0 or lo == out_dim for lo, _ in parts)
            per = parts[0][1] - parts[0][0]
            assert all(lo == min(out_dim, r * per) for r, (lo, _) in enumerate(parts))
            assert parts == [pkg.runtime.ShardRows(out_dim, r, world) for r in range(world)]
