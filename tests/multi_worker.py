"""One rank of the multi-GPU tests; started by tests/test_multi_rank.py as
    python -m torch.distributed.run --nproc-per-node N ... tests/multi_worker.py --mode cpu|gpu

cpu: the host-side partitioning only.  Every rank runs the CPU oracle on ITS rows / experts, the
     blocks travel through a gloo all-gather, and the assembled result must equal the oracle on the
     whole matrix bit for bit (row sharding does not change any row's arithmetic).
gpu: the same partitioning through the C ABI on one GPU per rank: sharded upload, product, the
     peer-memory exchange; results against the oracle within 2e-3.  torch.distributed (gloo) is
     only used to pass the 64-byte area tokens around and to agree on pass/fail."""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from conftest import load_package  # noqa: E402
from oracle import binding as orc  # noqa: E402

F = np.float32
TOL = 2e-3
MLX_SHAPES = [(3072, 1024, 1), (1000, 512, 5), (20, 256, 2), (8192, 2048, 1)]   # (out, in, batch)


def gloo_gather_rows(block, out_dim, per, batch, rank, world):
    """all-gather of [batch, per] blocks (padded) -> [batch, out_dim]."""
    pad = np.zeros((batch, per), dtype=F)
    pad[:, :block.shape[1]] = block
    parts = [torch.zeros(batch, per) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(pad))
    return np.concatenate([p.numpy() for p in parts], axis=1)[:, :out_dim]


def moe_layer_arrays(syn, experts, hidden, inter, gs):
    g = syn.rng("moe-multi", experts, hidden, inter)

    def stack(o, i):
        w = g.integers(0, 2**32, size=(experts, o * (i // 8)), dtype=np.uint32)
        s = syn.bf16_round(np.abs(g.standard_normal((experts, o * (i // gs)), dtype=F)) * F(0.02) + F(1e-3))
        return w, s, syn.bf16_round(F(-8) * s)
    return stack(inter, hidden), stack(inter, hidden), stack(hidden, inter), syn.mlx_weight("moe-router", experts, hidden, gs)


def run_cpu(rank, world, pkg):
    syn, sh = pkg.synth, pkg.sharding
    rt = pkg.runtime
    for out_dim, in_dim, batch in MLX_SHAPES:
        lo, hi = sh.shard_rows(out_dim, rank, world)
        assert (lo, hi) == rt.ShardRows(out_dim, rank, world), "python and C partition rules differ"
        per = sh.shard_rows(out_dim, 0, world)[1]
        w, s, b = syn.mlx_weight(("multi", out_dim), out_dim, in_dim, 64)
        x = syn.activations(("multi", out_dim), batch * in_dim)
        full = orc.mlx_gemm(x, batch, w, s, b, out_dim, in_dim, 64).reshape(batch, out_dim)
        if hi > lo:
            ws, ss, bs = sh.slice_mlx(w, s, b, in_dim, 64, lo, hi)
            mine = orc.mlx_gemm(x, batch, ws, ss, bs, hi - lo, in_dim, 64).reshape(batch, hi - lo)
        else:
            mine = np.zeros((batch, 0), dtype=F)
        got = gloo_gather_rows(mine, out_dim, per, batch, rank, world)
        assert np.array_equal(got.view(np.uint32), full.view(np.uint32)), ("mlx", out_dim, in_dim)
    for qtype, block, gen in ((rt.GGUF_Q8_0, sh.Q8_0_BLOCK, syn.q8_0_matrix), (rt.GGUF_Q4_K, sh.Q4_K_BLOCK, syn.q4k_matrix)):
        out_dim, in_dim = 520, 512
        raw = gen("multi", out_dim, in_dim)
        x = syn.activations("multi-gguf", in_dim, bf16=False)
        lo, hi = sh.shard_rows(out_dim, rank, world)
        per = sh.shard_rows(out_dim, 0, world)[1]
        mine = orc.gguf_gemv(x, sh.slice_gguf(raw, block, in_dim, lo, hi), qtype, in_dim, hi - lo).reshape(1, hi - lo)
        got = gloo_gather_rows(mine, out_dim, per, 1, rank, world)
        assert np.array_equal(got[0].view(np.uint32), orc.gguf_gemv(x, raw, qtype, in_dim, out_dim).view(np.uint32)), qtype
    out_dim, in_dim = 264, 128
    w, scale, bias = syn.fp8_linear("multi", out_dim, in_dim, bias=True)
    x = syn.activations("multi-fp8", in_dim)
    lo, hi = sh.shard_rows(out_dim, rank, world)
    per = sh.shard_rows(out_dim, 0, world)[1]
    ws, ss, bs = sh.slice_fp8(w, scale, bias, in_dim, lo, hi)
    mine = orc.fp8_gemv(x, ws, ss, bs, hi - lo, in_dim).reshape(1, hi - lo)
    got = gloo_gather_rows(mine, out_dim, per, 1, rank, world)
    assert np.array_equal(got[0].view(np.uint32), orc.fp8_gemv(x, w, scale, bias, out_dim, in_dim).view(np.uint32))
    # MoE: experts placed per rank; partial sums gathered and added in rank order
    experts, hidden, inter, top_k = 16, 256, 128, 4
    gate, up, down, router = moe_layer_arrays(syn, experts, hidden, inter, 64)
    x = syn.activations("multi-moe", hidden)
    ids, wts = orc.moe_route(orc.mlx_gemv(x, *router, experts, hidden, 64), top_k, True)
    mine_e = sh.place_experts(experts, rank, world)
    keep = [k for k, e in enumerate(ids) if e in mine_e]
    part = orc.moe_experts(x, hidden, inter, 64, gate, up, down, ids[keep], wts[keep])
    parts = [torch.zeros(hidden) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(part))
    total = np.zeros(hidden, dtype=F)
    for p in parts:
        total = total + p.numpy()
    full = orc.moe_experts(x, hidden, inter, 64, gate, up, down, ids, wts)
    assert syn.rel_err(total, full) <= 1e-5
    assert sorted(e for r in range(world) for e in sh.place_experts(experts, r, world)) == list(range(experts))


def run_gpu(rank, world, pkg):
    syn, sh, rt = pkg.synth, pkg.sharding, pkg.runtime
    rt.init(int(os.environ.get("LOCAL_RANK", rank)))
    g = rt.Gather(rank, world, 1 << 20)
    g.Connect(dist)
    checks = []
    # ---- MLX shards, both layouts, several exchanges in a row (exercises both result buffers)
    for rep in range(3):
        for out_dim, in_dim, batch in MLX_SHAPES + [(151936, 1024, 1)]:
            lo, hi = rt.ShardRows(out_dim, rank, world)
            w, s, b = syn.mlx_weight(("multi", out_dim), out_dim, in_dim, 64)
            x = syn.activations(("multi", out_dim, rep), batch * in_dim)
            xb = rt.from_numpy(x)
            if hi > lo:
                h = rt.UploadMLXWeight(*sh.slice_mlx(w, s, b, in_dim, 64, lo, hi), in_dim, hi - lo, 64, True)
                res = g.GemmMLX(xb, h, batch, lo, out_dim)
            else:
                h = None
                res = g.GemmMLX(xb, None, batch, lo, out_dim)
            rt.Sync()
            got = res.Download(batch * out_dim)
            want = orc.mlx_gemm(x, batch, w, s, b, out_dim, in_dim, 64, nthreads=8)
            checks.append(("mlx", out_dim, in_dim, batch, syn.rel_err(got, want)))
            if h is not None:
                h.Free()
            xb.Free()
    # ---- back-to-back exchanges without a host sync in between, read afterwards
    out_dim, in_dim = 2048, 1024
    lo, hi = rt.ShardRows(out_dim, rank, world)
    w, s, b = syn.mlx_weight(("multi", "b2b"), out_dim, in_dim, 64)
    h = rt.UploadMLXWeight(*sh.slice_mlx(w, s, b, in_dim, 64, lo, hi), in_dim, hi - lo, 64, True)
    xs = [syn.activations(("b2b", i), in_dim) for i in range(40)]
    xbs = [rt.from_numpy(x) for x in xs]
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    stream = torch.cuda.Stream()
    keep = torch.zeros(40, out_dim, device="cuda")
    with torch.cuda.stream(stream):
        for i in range(40):
            res = g.GemmMLX(xbs[i], h, 1, lo, out_dim, stream)
            # copy the result aside on the same stream before the buffer is reused two exchanges later
            keep[i].copy_(as_tensor(res, out_dim))
    stream.synchronize()
    allv = keep.cpu().numpy()
    for i in range(40):
        want = orc.mlx_gemv(xs[i], w, s, b, out_dim, in_dim, 64, nthreads=8)
        checks.append(("b2b", i, in_dim, 1, syn.rel_err(allv[i], want)))
    # ---- a pair of exchanges captured in a CUDA graph and replayed
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        cs = torch.cuda.current_stream()
        for i in range(2):
            res = g.GemmMLX(xbs[i], h, 1, lo, out_dim, cs)
            keep[i].copy_(as_tensor(res, out_dim))
    for _ in range(5):
        keep.zero_()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        allv = keep.cpu().numpy()
        for i in range(2):
            want = orc.mlx_gemv(xs[i], w, s, b, out_dim, in_dim, 64, nthreads=8)
            checks.append(("graph", i, in_dim, 1, syn.rel_err(allv[i], want)))
    h.Free()
    # ---- GGUF and FP8 shards
    for qtype, block, gen in ((rt.GGUF_Q8_0, sh.Q8_0_BLOCK, syn.q8_0_matrix), (rt.GGUF_Q4_K, sh.Q4_K_BLOCK, syn.q4k_matrix)):
        out_dim, in_dim, batch = 4096, 2048, 3
        raw = gen("multi", out_dim, in_dim)
        x = syn.activations("multi-gguf", batch * in_dim, bf16=False)
        lo, hi = rt.ShardRows(out_dim, rank, world)
        m = rt.UploadGGUFMatrix(qtype, sh.slice_gguf(raw, block, in_dim, lo, hi), in_dim, hi - lo)
        xb = rt.from_numpy(x)
        res = g.ProjectGGUF(xb, m, batch, lo, out_dim)
        rt.Sync()
        want = orc.gguf_gemv(x, raw, qtype, in_dim, out_dim, batch, nthreads=8)
        checks.append(("gguf", qtype, in_dim, batch, syn.rel_err(res.Download(batch * out_dim), want)))
        m.Free(); xb.Free()
    out_dim, in_dim, batch = 4096, 2048, 2
    w8, scale, bias = syn.fp8_linear("multi", out_dim, in_dim, bias=True)
    x = syn.activations("multi-fp8", batch * in_dim)
    lo, hi = rt.ShardRows(out_dim, rank, world)
    lin = rt.UploadFP8E4M3Linear(*sh.slice_fp8(w8, scale, bias, in_dim, lo, hi), hi - lo, in_dim)
    xb = rt.from_numpy(x)
    res = g.GemmFP8E4M3(xb, lin, batch, lo, out_dim)
    rt.Sync()
    want = orc.fp8_batch_gemv(x, batch, w8, scale, bias, out_dim, in_dim, nthreads=8)
    checks.append(("fp8", out_dim, in_dim, batch, syn.rel_err(res.Download(batch * out_dim), want)))
    lin.Free(); xb.Free()
    # ---- MoE with experts placed per GPU
    experts, hidden, inter, top_k, tokens = 32, 512, 256, 8, 5
    gate, up, down, router = moe_layer_arrays(syn, experts, hidden, inter, 64)
    rt.SetOption("mlx_layout", 1)
    layer = rt.GPUMoELayer(experts, hidden, inter, 64, top_k, True, 8)
    rw = rt.UploadMLXWeight(*router, hidden, experts, 64, True)
    layer.SetRouter(rw)
    for e in sh.place_experts(experts, rank, world):
        layer.SetExpert(e, *[rt.UploadMLXWeight(t[0][e], t[1][e], t[2][e], i, o, 64, True)
                             for t, o, i in ((gate, inter, hidden), (up, inter, hidden), (down, hidden, inter))])
    rt.SetOption("mlx_layout", 0)
    x = syn.activations("multi-moe", tokens * hidden).reshape(tokens, hidden)
    xb, ob = rt.from_numpy(x), rt.Malloc(tokens * hidden)
    g.MoEForward(layer, ob, xb, tokens)
    rt.Sync()
    got = ob.Download().reshape(tokens, hidden)
    ids, wts = layer.LastRouting(tokens)
    for t in range(tokens):
        want = orc.moe_experts(x[t], hidden, inter, 64, gate, up, down, ids[t], wts[t])
        checks.append(("moe", t, hidden, tokens, syn.rel_err(got[t], want)))
    assert g.Status() == 0, "an exchange wait gave up: status %d" % g.Status()
    assert rt.KernelStatus() == 0
    bad = [c for c in checks if not c[4] <= TOL]
    assert not bad, bad
    dist.barrier()
    g.Free()
    return len(checks)


class _Raw:
    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def as_tensor(buf, n):
    """A torch view of a library buffer (torch is only the plumbing for the copy-aside)."""
    return torch.as_tensor(_Raw(buf.Ptr, n), device="cuda")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["cpu", "gpu"], required=True)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    pkg = load_package()
    n = run_cpu(rank, world, pkg) if args.mode == "cpu" else run_gpu(rank, world, pkg)
    dist.barrier()
    print("rank %d of %d ok (%s)" % (rank, world, n), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
