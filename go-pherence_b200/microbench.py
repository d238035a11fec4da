"""Per-shape kernel throughput of the quantized products, measured with CUDA events.

    python go-pherence_b200/microbench.py --format mlx4 --out 4096 --in 4096 [--batch 1]
           [--opt mlx_unpack=0] [--launches 200] [--copies N]

The launches are captured once into a CUDA graph and replayed, so the figure is device time
per launch, not the host's launch rate.  The weight is uploaded `copies` times (default: enough copies to exceed 512 MB, four times
the L2) and consecutive launches walk through the copies, so every launch streams its weights
from HBM.  Prints one JSON line: microseconds per launch, GB/s of algorithmic bytes and the
fraction of the measured HBM copy bandwidth.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from __graft_entry__ import load_package  # noqa: E402


def algorithmic_bytes(fmt, out_dim, in_dim, batch):
    per_weight = {"mlx4": 0.5625, "q4k": 0.5625, "q5k": 0.6875, "q6k": 0.8203125, "q8_0": 1.0625, "fp8": 1.0}[fmt]
    extra = 4 * out_dim if fmt == "fp8" else 0
    return out_dim * in_dim * per_weight + extra + batch * in_dim * 4 + batch * out_dim * 4


def run(fmt, out_dim, in_dim, batch=1, launches=200, copies=0, opts=(), warmup=10, chain=False, xbf16=False):
    import torch
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(0)
    tune = dict((k, v) for k, v in opts if k.startswith("tune_"))
    opts = [(k, v) for k, v in opts if not k.startswith("tune_")]
    if tune:  # tuning build only: parts of the kernels left out / chunk rotation off
        rt.lib().goph_tuning_set(int(tune.get("tune_dbg", 0)), int(tune.get("tune_rotate", 1)))
        rt.lib().goph_tuning_set_gemv(int(tune.get("tune_gemv", 0)))
    for k, v in opts:
        rt.SetOption(k, v)
    nbytes = algorithmic_bytes(fmt, out_dim, in_dim, batch)
    if copies <= 0:
        copies = max(2, int(512e6 // nbytes) + 1)
    copies = min(copies, 256)
    handles = []
    if fmt == "mlx4":
        w, s, b = syn.mlx_weight("mb", out_dim, in_dim, 64)
        handles = [rt.UploadMLXWeight(w, s, b, in_dim, out_dim, 64, True) for _ in range(copies)]
    elif fmt in ("q4k", "q5k", "q6k", "q8_0"):
        qt = {"q4k": rt.GGUF_Q4_K, "q5k": rt.GGUF_Q5_K, "q6k": rt.GGUF_Q6_K, "q8_0": rt.GGUF_Q8_0}[fmt]
        raw = {"q4k": syn.q4k_matrix, "q5k": syn.q5k_matrix, "q6k": syn.q6k_matrix, "q8_0": syn.q8_0_matrix}[fmt]("mb", out_dim, in_dim)
        handles = [rt.UploadGGUFMatrix(qt, raw, in_dim, out_dim) for _ in range(copies)]
    else:
        w = torch.randn(out_dim, in_dim).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy().reshape(-1)
        sc = syn.fp8_linear("mb", 8, 16)[1][:1].repeat(out_dim)
        handles = [rt.UploadFP8E4M3Linear(w, sc, None, out_dim, in_dim) for _ in range(copies)]
    x = torch.from_numpy(syn.activations("mb", batch * in_dim)).cuda()
    out = torch.empty(batch * out_dim, dtype=torch.float32, device="cuda")
    xb, ob = rt.wrap(x.data_ptr(), x.numel() * 4), rt.wrap(out.data_ptr(), out.numel() * 4)
    if xbf16:  # the activations as bf16 in device memory (the bf16 entry points, tensor-core layouts only)
        x16 = x.to(torch.bfloat16)
        xb = rt.wrap(x16.data_ptr(), x16.numel() * 2)
    stream = torch.cuda.current_stream()
    if chain:
        # every launch consumes the output of the one before it (square matrices only), as the
        # projections of a decode step do: nothing of a launch's activations exists before its
        # predecessor has finished.  The values overflow after a few dozen launches; the time does not care.
        if out_dim != in_dim:
            raise SystemExit("--chain needs out == in")
        flip = [0]

    def launch(h):
        if chain:
            i = flip[0]
            flip[0] ^= 1
            _launch(h, (xb, ob)[i], (xb, ob)[1 - i])
        else:
            _launch(h, xb, ob)

    def _launch(h, xb, ob):
        if fmt == "mlx4" and xbf16:
            rt.GemmMLXBF16(ob, xb, h, batch, stream)
        elif fmt == "fp8" and xbf16:
            rt.GemmFP8E4M3BF16Buffer(ob, xb, batch, h, stream)
        elif fmt == "mlx4":
            rt.GemmMLX(ob, xb, h, batch, stream)
        elif fmt == "fp8":
            rt.GemmFP8E4M3Buffer(ob, xb, batch, h, stream)
        else:
            h.ProjectBatchToBuffer(ob, xb, batch, stream)

    for i in range(warmup):
        launch(handles[i % copies])
    torch.cuda.synchronize()
    # the launches are replayed from a CUDA graph so the host's launch rate is not what is timed
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        stream = torch.cuda.current_stream()
        for i in range(launches):
            launch(handles[i % copies])
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (launches * reps)
    peak = 6650.0
    pk = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["hbm_gbs"])
    gbs = nbytes / us / 1e3
    tflops = 2.0 * out_dim * in_dim * batch / us / 1e6
    res = {"format": fmt, "out": out_dim, "in": in_dim, "batch": batch, "x": "bf16" if xbf16 else "f32", "tflops": round(tflops, 1), "opts": dict(opts), "copies": copies, "chain": bool(chain),
           "us_per_launch": round(us, 3), "GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
           "bytes": nbytes}
    if hasattr(rt.lib(), "goph_tuning_probe"):  # tuning build: clock64 timeline of one CTA's last launch
        import ctypes
        buf = (ctypes.c_longlong * 512)()
        (rt.lib().goph_tuning_probe if batch > 8 or fmt == "fp8" else rt.lib().goph_tuning_probe_gemv)(buf)
        t0 = buf[7 * 64]
        names = ["loads_issued", "mma_sees_stage", "mma_issued", "conv_starts", "conv_done", "epi_sees_unit0", "epi_done"]
        res["trace"] = {"end": buf[7 * 64 + 1] - t0, "pdl_wait_done": buf[7 * 64 + 2] - t0}
        res["trace"]["item_end"] = [buf[7 * 64 + k] - t0 for k in range(8, 16) if buf[7 * 64 + k]]
        for e, n in enumerate(names):
            res["trace"][n] = [buf[e * 64 + i] - t0 for i in range(40) if buf[e * 64 + i]]
    for h in handles:
        h.Free()
    return res


def run_moe(tokens, experts=128, hidden=2048, inter=768, top_k=8, layers=4, launches=40, opts=(), keep_alive=None,
            expert_layout=1, eager=False):
    """Selected-expert projection at the Qwen3-30B-A3B layer shape: `layers` distinct layers are walked
    so consecutive calls do not find their experts in L2.  Bytes counted: the router plus three matrices
    of every distinct expert the call's tokens selected.  expert_layout: 1 = row-major experts (CUDA-core
    expert kernels), 2 = tiled experts (grouped launches of the tensor-core kernel)."""
    import numpy as np
    import torch
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(0)
    tune = dict((k, v) for k, v in opts if k.startswith("tune_"))
    opts = [(k, v) for k, v in opts if not k.startswith("tune_")]
    if tune:  # tuning build only
        rt.lib().goph_tuning_set_gemv(int(tune.get("tune_gemv", 0)))
    for k, v in opts:
        rt.SetOption(k, v)
    rt.SetOption("mlx_layout", 1)
    g = syn.rng("moe-bench")
    mods, keep = [], []
    for l in range(layers):
        m = rt.GPUMoELayer(experts, hidden, inter, 64, top_k, True, max(tokens, 1))
        r = rt.UploadMLXWeight(*syn.mlx_weight(("r", l), experts, hidden, 64), hidden, experts, 64, True)
        m.SetRouter(r)
        keep.append(r)
        rt.SetOption("mlx_layout", expert_layout)
        for e in range(experts):
            hs = []
            for o, i in ((inter, hidden), (inter, hidden), (hidden, inter)):
                w = g.integers(0, 2**32, size=o * i // 8, dtype=np.uint32)
                sc = syn.bf16_round(np.abs(g.standard_normal(o * i // 64, dtype=np.float32)) * np.float32(0.02) + np.float32(1e-3))
                hs.append(rt.UploadMLXWeight(w, sc, syn.bf16_round(np.float32(-8) * sc), i, o, 64, True))
            m.SetExpert(e, *hs)
            keep += hs
        rt.SetOption("mlx_layout", 1)
        mods.append(m)
    rt.SetOption("mlx_layout", 0)
    x = torch.from_numpy(syn.activations("moe-bench", tokens * hidden)).cuda()
    out = torch.empty(tokens * hidden, dtype=torch.float32, device="cuda")
    xb, ob = rt.wrap(x.data_ptr(), x.numel() * 4), rt.wrap(out.data_ptr(), out.numel() * 4)
    stream = torch.cuda.current_stream()
    distinct = []
    for m in mods:
        m.Forward(ob, xb, tokens, stream)
        torch.cuda.synchronize()
        distinct.append(len(set(m.LastRouting(tokens)[0].reshape(-1).tolist())))
    class Eager:  # plain launches instead of a graph replay (for a profiler's launch list)
        def replay(self):
            for i in range(launches):
                mods[i % layers].Forward(ob, xb, tokens, torch.cuda.current_stream())
    if eager:
        graph = Eager()
    else:
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(launches):
                mods[i % layers].Forward(ob, xb, tokens, torch.cuda.current_stream())
    graph.replay()
    torch.cuda.synchronize()
    trace = None
    if hasattr(rt.lib(), "goph_tuning_probe_gemv"):  # tuning build: timeline of one CTA of the last tensor-core launch
        import ctypes
        buf = (ctypes.c_longlong * 512)()
        rt.lib().goph_tuning_probe_gemv(buf)
        t0 = buf[7 * 64]
        names = ["loads_issued", "mma_sees_stage", "mma_issued", "conv_starts", "conv_done", "epi_sees_unit0", "epi_done"]
        trace = {"entry": buf[7 * 64 + 3] - t0, "end": buf[7 * 64 + 1] - t0}
        for e, n in enumerate(names):
            trace[n] = [buf[e * 64 + i] - t0 for i in range(40) if buf[e * 64 + i]]
    if hasattr(rt.lib(), "goph_tuning_probe_moe") and tokens == 1 and expert_layout == 1:
        import ctypes
        buf = (ctypes.c_longlong * 24)()
        rt.lib().goph_tuning_probe_moe(buf)
        trace = {"one_launch_phase_ends": [buf[i] - buf[0] for i in range(1, 9)],
                 "routing_points": [buf[i] - buf[0] for i in range(16, 21)]}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 1 if eager else 5
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (launches * reps)
    per_expert = (2 * inter * hidden + hidden * inter) * 0.5625
    nbytes = sum(distinct) / layers * per_expert + experts * hidden * 0.5625 + tokens * hidden * 8
    peak = 6650.0
    pk = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["hbm_gbs"])
    gbs = nbytes / us / 1e3
    return {"format": "moe-mlx4", "tokens": tokens, "experts": experts, "top_k": top_k, "hidden": hidden, "inter": inter,
            "distinct_experts_per_call": sum(distinct) / layers, "us_per_call": round(us, 2), "GBps": round(gbs, 1),
            "frac_of_hbm_peak": round(gbs / peak, 4), "bytes": nbytes, "trace": trace}


_WORK_MATRICES = {}


def run_gguf_work(tokens, experts=128, hidden=2048, inter=768, top_k=8, launches=20, layout=1):
    """The work-list GGUF products of an MoE layer whose experts are stacked in one matrix: fused gate|up
    (Q4_K) with tanh-GELU by work list, then the weighted scatter-add of the down projection (Q8_0) by
    work list, `tokens * top_k` items with experts drawn like a routing (distinct per token).  Two work
    lists alternate, so a call does not find its experts in L2.  Bytes counted: gate|up and down rows of
    every distinct expert of a call."""
    import numpy as np
    import torch
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(0)
    key = (experts, hidden, inter, layout)
    if key not in _WORK_MATRICES:  # kept for the life of the process: several list lengths share the uploads
        rt.SetOption("gguf_layout", layout)
        try:
            _WORK_MATRICES[key] = (
                rt.UploadGGUFMatrix(rt.GGUF_Q4_K, syn.q4k_matrix("work-gu", experts * 2 * inter, hidden), hidden, experts * 2 * inter),
                rt.UploadGGUFMatrix(rt.GGUF_Q8_0, syn.q8_0_matrix("work-dn", experts * hidden, inter), inter, experts * hidden))
        finally:
            rt.SetOption("gguf_layout", 0)
    gu, dn = _WORK_MATRICES[key]
    g = syn.rng("work-lists", tokens)
    n = tokens * top_k
    lists, distinct = [], []
    for _ in range(2):
        ex = np.concatenate([g.choice(experts, size=top_k, replace=False) for _ in range(tokens)]).astype(np.uint32)
        pos = np.repeat(np.arange(tokens, dtype=np.uint32), top_k)
        wt = g.uniform(0.05, 0.2, n).astype(np.float32)
        lists.append(tuple(rt.from_numpy(a) for a in (ex, pos, wt)))
        distinct.append(len(set(ex.tolist())))
    x = np.repeat(syn.activations("work-x", tokens * hidden).reshape(tokens, hidden), top_k, axis=0).reshape(-1)  # one row per item
    xb = rt.from_numpy(x)
    act = rt.Malloc(n * inter)
    out = rt.Malloc(tokens * hidden)
    stream = torch.cuda.current_stream()

    def call(i):
        ex, pos, wt = lists[i % 2]
        rt.GateUpGELUQ4KByWorkToBuffer(act, xb, ex, n, inter, experts, gu, stream)
        rt.GemvQ8_0ScatterByWork(out, act, ex, pos, wt, n, experts, dn, stream)

    call(0)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        stream = torch.cuda.current_stream()
        for i in range(launches):
            call(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (launches * reps)
    per_expert = 2 * inter * hidden * 144 / 256 + hidden * inter * 34 / 32
    nbytes = sum(distinct) / 2 * per_expert
    peak = 6650.0
    pk = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["hbm_gbs"])
    status = rt.KernelStatus()
    for t in (xb, act, out):
        t.Free()
    return {"format": "gguf-work q4_k gate|up + q8_0 down", "tokens": tokens, "items": n, "layout": layout,
            "distinct_experts_per_call": sum(distinct) / 2, "us_per_call": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
            "frac_of_hbm_peak": round(nbytes / us / 1e3 / peak, 4), "bytes": nbytes, "kernel_status": status}


def run_layer_chain(fmt, hidden=4096, ffn=14336, kv=1024, layers=8, reps=5, opts=(), qdim=0, as_list=False):
    """The projections of decoder layers (Llama-3-8B shapes by default) as one dependent chain, batch 1:
    q|k|v (qdim+2kv x hidden) -> o (hidden x qdim, fed by the first `qdim` outputs) ->
    gate|up (2 ffn x hidden) -> down (hidden x ffn, fed by the first `ffn` outputs) -> next layer.
    Every launch reads what the launch before it wrote, as in a decode step; `layers` layers have
    their own device copies of the weights (more than the L2 holds), replayed as a CUDA graph."""
    import numpy as np
    import torch
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(0)
    for k, v in opts:
        rt.SetOption(k, v)
    qdim = qdim or hidden
    shapes = [(qdim + 2 * kv, hidden), (hidden, qdim), (2 * ffn, hidden), (hidden, ffn)]
    host = []
    for o, i in shapes:
        if fmt == "mlx4":
            host.append(syn.mlx_weight(("chain", o, i), o, i, 64))
        elif fmt == "q4k":
            host.append(syn.q4k_matrix(("chain", o, i), o, i))
        elif fmt == "q8_0":
            host.append(syn.q8_0_matrix(("chain", o, i), o, i))
        else:
            w = torch.randn(o, i).clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy().reshape(-1)
            host.append((w, np.full(o, 1.0 / np.sqrt(i), dtype=np.float32)))
    handles, nbytes = [], 0.0
    for _ in range(layers):
        hs = []
        for (o, i), hw in zip(shapes, host):
            if fmt == "mlx4":
                hs.append(rt.UploadMLXWeight(*hw, i, o, 64, True))
            elif fmt in ("q4k", "q8_0"):
                hs.append(rt.UploadGGUFMatrix(rt.GGUF_Q4_K if fmt == "q4k" else rt.GGUF_Q8_0, hw, i, o))
            else:
                hs.append(rt.UploadFP8E4M3Linear(hw[0], hw[1], None, o, i))
            nbytes += algorithmic_bytes(fmt, o, i, 1)
        handles.append(hs)
    bufs = [torch.zeros(max(2 * ffn, qdim + 2 * kv), dtype=torch.float32, device="cuda") for _ in range(2)]
    bufs[0][:hidden] = torch.from_numpy(syn.activations("chain", hidden)).cuda()
    wrap = lambda t: rt.wrap(t.data_ptr(), t.numel() * 4)

    def launch(h, x, out, stream):
        if fmt == "mlx4":
            rt.GemvMLX(out, x, h, stream)
        elif fmt == "fp8":
            rt.GemvFP8E4M3Buffer(out, x, h, stream)
        else:
            h.ProjectBatchToBuffer(out, x, 1, stream)

    program = None
    if as_list:   # the same chain as one product list (one cooperative launch)
        if fmt != "mlx4":
            raise SystemExit("--list needs --format mlx4")
        ops, cur = [], 0
        for hs in handles:
            for h in hs:
                ops.append((wrap(bufs[cur]), [h], [wrap(bufs[1 - cur])]))
                cur ^= 1
        program = rt.MLXProgram(ops)

    def step(stream):
        if program is not None:
            program.Run(stream)
            return
        cur = 0
        for hs in handles:
            for h in hs:
                launch(h, wrap(bufs[cur]), wrap(bufs[1 - cur]), stream)
                cur ^= 1

    step(torch.cuda.current_stream())
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step(torch.cuda.current_stream())
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / reps
    peak = 6650.0
    pk = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = float(json.load(open(pk))["hbm_gbs"])
    gbs = nbytes / us / 1e3
    for hs in handles:
        for h in hs:
            h.Free()
    if program is not None:
        program.Free()
    return {"format": fmt, "workload": "%d decoder layers of projections (hidden %d, q %d, kv %d, ffn %d), dependent chain, batch 1"
                                       % (layers, hidden, qdim, kv, ffn),
            "launches": 1 if as_list else 4 * layers, "us_per_product": round(us / (4 * layers), 3), "us_per_layer": round(us / layers, 2), "GBps": round(gbs, 1),
            "frac_of_hbm_peak": round(gbs / peak, 4), "bytes": nbytes}


def run_decode_tokens(steps=3, position=150, opts=()):
    """A few greedy steps of the Qwen3-0.6B-shaped MLX 4-bit decoder at a given position, as plain
    launches (for a profiler's launch list; the timing figure is bench.py's `decode`)."""
    import types
    import numpy as np
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(0)
    for k, v in opts:
        rt.SetOption(k, v)
    F = np.float32
    cfg = types.SimpleNamespace(hidden=1024, layers=28, heads=16, kv_heads=8, head_dim=128, inter=3072, vocab=151936,
                                eps=1e-6, theta=1e6, qk_norm=True, max_seq=192)
    shapes = {"q": (2048, 1024), "k": (1024, 1024), "v": (1024, 1024), "o": (1024, 2048), "gate": (3072, 1024),
              "up": (3072, 1024), "down": (1024, 3072)}
    base = [{n: syn.mlx_weight(("dec", n, k), o, i, 64) for n, (o, i) in shapes.items()} for k in range(4)]
    layers = []
    for l in range(cfg.layers):
        d = dict(base[l % 4])
        for n, sz in (("input_norm", 1024), ("post_norm", 1024), ("q_norm", 128), ("k_norm", 128)):
            d[n] = np.ones(sz, dtype=F)
        layers.append(d)
    lm = syn.mlx_weight(("dec", "lm"), cfg.vocab, cfg.hidden, 64)
    table = np.zeros((cfg.max_seq, cfg.head_dim // 2, 2), dtype=F)
    table[:, :, 0] = 1
    dec = pkg.decode.MLXDecoder(rt, cfg, layers, lm, np.ones(1024, dtype=F), table)
    ints = np.full(2 + 2 * cfg.max_seq, -1, dtype=np.int32)
    ints[0], ints[1] = 5, position   # current token and position: the cache rows before it are zeros
    dec.ints.UploadBytes(ints.view(np.uint8))
    for _ in range(steps):
        dec.step(None)
    rt.Sync()
    return {"workload": "qwen3-0.6b mlx4 decode, %d eager steps from position %d" % (steps, position),
            "launches_per_token": dec.launches_per_step}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--eager", action="store_true", help="--format moe: plain launches instead of a CUDA graph")
    ap.add_argument("--expert-layout", type=int, default=1, choices=[1, 2], help="--format moe: 1 row-major experts, 2 tiled")
    ap.add_argument("--layer-chain", action="store_true", help="decoder-layer projections at Llama-3-8B shapes as a dependent chain")
    ap.add_argument("--format", default="mlx4", choices=["mlx4", "q4k", "q5k", "q6k", "q8_0", "fp8", "moe", "gguf-work"])
    ap.add_argument("--out", type=int, default=4096)
    ap.add_argument("--in", dest="in_dim", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--launches", type=int, default=200)
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--opt", action="append", default=[], help="name=value for goph_set_option")
    ap.add_argument("--xbf16", action="store_true", help="activations held as bf16 (the bf16 entry points)")
    ap.add_argument("--chain", action="store_true", help="each launch reads the previous launch's output (out == in)")
    ap.add_argument("--list", action="store_true", help="--layer-chain as one product list (one cooperative launch)")
    ap.add_argument("--decode-tokens", type=int, default=0, help="run this many eager decoder steps (for a launch list)")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--qdim", type=int, default=0)
    ap.add_argument("--kv", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--layers", type=int, default=8)
    args = ap.parse_args()
    opts = [(o.split("=")[0], int(o.split("=")[1])) for o in args.opt]
    if args.decode_tokens:
        print(json.dumps(run_decode_tokens(args.decode_tokens, opts=opts)))
        return
    if args.layer_chain:
        print(json.dumps(run_layer_chain(args.format, args.hidden, args.ffn, args.kv, args.layers, opts=opts, qdim=args.qdim,
                                         as_list=args.list)))
        return
    if args.format == "gguf-work":
        print(json.dumps(run_gguf_work(args.tokens, launches=min(args.launches, 20), layout=args.expert_layout)))
        return
    if args.format == "moe":
        print(json.dumps(run_moe(args.tokens, opts=opts, expert_layout=args.expert_layout, eager=args.eager,
                                 launches=min(args.launches, 40), layers=2 if args.eager else 4)))
        return
    print(json.dumps(run(args.format, args.out, args.in_dim, args.batch, args.launches, args.copies, opts, chain=args.chain, xbf16=args.xbf16)))


if __name__ == "__main__":
    main()
