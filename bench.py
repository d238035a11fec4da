#!/usr/bin/env python
"""Headline benchmark: quantized-GEMV weight bandwidth on the Qwen3-0.6B MLX 4-bit decode step.

One step = every linear projection one decode token needs, on random-init weights of the
Qwen3-0.6B architecture in MLX 4-bit g64 form: per layer q|k|v (one launch, shared x), o,
gate|up (one launch, shared x), down — 28 layers — then the tied 151936x1024 LM head.
113 launches, 197 matrices, 335 MB of packed weights per step (larger than L2, so every
step streams them from HBM again).  Data is synthetic and seeded.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is GB/s of algorithmic bytes
with inputs resident in HBM; `e2e` is the same step with the activations copied from pinned
host memory and the logits copied back inside the timed region.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

HIDDEN, LAYERS, VOCAB, FFN, QDIM, KVDIM, GS = 1024, 28, 151936, 3072, 2048, 1024, 64
# (name, [(out_dim, in_dim) of the weights that share one x])
LAYER_OPS = [("qkv", [(QDIM, HIDDEN), (KVDIM, HIDDEN), (KVDIM, HIDDEN)]),
             ("o", [(HIDDEN, QDIM)]),
             ("gate_up", [(FFN, HIDDEN), (FFN, HIDDEN)]),
             ("down", [(HIDDEN, FFN)])]
# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, from the ncu captures
# summarised under profiles/ (mlx_gemv_kernel on 3072x1024: 1.787 MB against 1.786 MB;
# mlx_program_kernel on the 112-product chain: 252.3 MB against 249.9 MB;
# mlx_mma_kernel on 65536x4096: 151.08 + 4.8 MB against 151.27 MB).  Traffic grows with the bytes
# streamed, so a launch's traffic is its algorithmic bytes times this ratio.
TRAFFIC_RATIO = {"mlx_gemv_kernel": 1.001, "mlx_program_kernel": 1.010, "mlx_mma_kernel": 1.031}
WORKLOAD = "qwen3-0.6b mlx4-g64 decode-step projections (28 layers x q|k|v,o,gate|up,down + LM head 151936x1024)"


def algorithmic_bytes(out_dim, in_dim, batch=1):
    """0.5625 B per weight (4-bit nibble + bf16 scale and bias per 64) + bf16-valued x + f32 out."""
    return out_dim * in_dim * 0.5625 + batch * in_dim * 2 + batch * out_dim * 4


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.p is not None:
            self.p.terminate()
            try:
                self.p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            c = [t.strip() for t in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.f.close()
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class _Raw:
    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


class DecodeStepProjections:
    """Weights, activations and the launch list of one decode step.

    One GPU: the weights that share an x (q|k|v, gate|up) are separate handles driven by one
    multi-weight launch.  Several GPUs: the same weights are concatenated by rows, every rank
    uploads its row shard, and each launch is followed by the peer-memory exchange that leaves the
    whole output on every rank (`gather="p2p"`), or by an NCCL all-gather (`gather="nccl"`, kept
    as the library baseline)."""

    def __init__(self, rt, syn, sharding, rank=0, world=1, layers=LAYERS, gather="p2p", shard_min_mb=16.0, product_list=True):
        import torch
        self.rt, self.torch, self.rank, self.world, self.gather_kind = rt, torch, rank, world, gather
        self.ops = []  # (name, [handles], x_tensor, [out_tensors], [(out_dim_shard, in_dim)], (lo, out_full))
        self.weight_bytes = 0
        self.bytes_per_step = 0.0
        ops = [(l, n, shapes) for l in range(layers) for n, shapes in LAYER_OPS] + [(layers, "lm_head", [(VOCAB, HIDDEN)])]
        # Data flow of a decode step: every product reads what the product before it wrote (q of
        # q|k|v feeds o, o feeds gate|up, gate feeds down, down feeds the next layer's q|k|v and at the
        # end the LM head); only the first product's x comes from outside.  The operations between
        # the projections (attention, norms, SiLU) are not part of this workload, so the values are
        # not a model's; scales and biases are quartered (exactly, they are bf16) to keep them finite.
        self.x_arena = torch.from_numpy(syn.activations(("x", 0, ops[0][1]), ops[0][2][0][1])).cuda()
        prev_out = None
        for l, name, shapes in ops:
            in_dim = shapes[0][1]
            if prev_out is None:
                x = self.x_arena
            elif prev_out.numel() >= in_dim:
                x = prev_out[:in_dim]
            else:   # the product in front is row-sharded here: its whole output lives in the exchange's buffer
                x = torch.from_numpy(syn.activations(("x", l, name), in_dim)).cuda()
            # every layer of a random-init model has its own weights; generation is the slow
            # part on the host, so layers draw from 4 distinct seeds (contents never repeat in L2:
            # the copies are separate device buffers)
            parts = [syn.mlx_weight((name, i, l % 4), o, in_dim, GS) for i, (o, _) in enumerate(shapes)]
            parts = [(w, s * np.float32(0.25), b * np.float32(0.25)) for w, s, b in parts]
            hs, outs, dims = [], [], []
            packed_mb = sum(o for o, _ in shapes) * in_dim * 0.5625 / 1e6
            if world == 1 or packed_mb < shard_min_mb:
                # small projections are not worth an exchange: every rank computes them whole
                for (o, _), (w, s, b) in zip(shapes, parts):
                    hs.append(rt.UploadMLXWeight(w, s, b, in_dim, o, GS, True))
                    outs.append(torch.empty(o, dtype=torch.float32, device="cuda"))
                    dims.append((o, in_dim))
                span = None
            else:
                w, s, b = (np.concatenate([p[k] for p in parts]) for k in range(3))
                out_full = sum(o for o, _ in shapes)
                lo, hi = sharding.shard_rows(out_full, rank, world)
                hs.append(rt.UploadMLXWeight(*sharding.slice_mlx(w, s, b, in_dim, GS, lo, hi), in_dim, hi - lo, GS, True))
                outs.append(torch.empty(hi - lo, dtype=torch.float32, device="cuda"))
                dims.append((hi - lo, in_dim))
                span = (lo, out_full)
            for h, (o, i) in zip(hs, dims):
                self.weight_bytes += h.ResidentBytes()
                # replicated work counts once for the job: rank 0's copy
                if span is not None or rank == 0:
                    self.bytes_per_step += algorithmic_bytes(o, i)
            self.ops.append((name, hs, x, outs, dims, span))
            prev_out = outs[0]
        self.sharded_ops = sum(1 for op in self.ops if op[5] is not None)
        # the leading run of whole, row-major products (under 8 Mi weights each: the layer projections)
        # goes into one product list: a single cooperative launch, products ordered by their data
        self.program, self.listed = None, 0
        if product_list:
            while (self.listed < len(self.ops) and self.ops[self.listed][5] is None
                   and all(o * i < (8 << 20) for o, i in self.ops[self.listed][4])):
                self.listed += 1
            if self.listed >= 2:
                self.program = rt.MLXProgram([(rt.wrap(x.data_ptr(), x.numel() * 4), hs,
                                               [rt.wrap(o.data_ptr(), o.numel() * 4) for o in outs])
                                              for _, hs, x, outs, _, _ in self.ops[:self.listed]])
            else:
                self.listed = 0
        # launches of this library per step: the list, one per remaining product, one more for every
        # product on the tensor-core path (its activation digits are a launch of their own), the exchanges
        tensor_core = sum(1 for op in self.ops[self.listed:] if any(o * i >= (8 << 20) for o, i in op[4]))
        self.launches_per_step = (len(self.ops) - self.listed + (1 if self.program else 0) + tensor_core
                                  + (self.sharded_ops if gather == "p2p" else 0))
        self.exchange = None
        if world > 1:
            import torch.distributed as dist
            if gather == "p2p":
                self.exchange = rt.Gather(rank, world, VOCAB + 64)
                handles = [torch.zeros(64, dtype=torch.uint8, device="cuda") for _ in range(world)]
                mine = torch.tensor(list(self.exchange.Export()), dtype=torch.uint8, device="cuda")
                dist.all_gather(handles, mine)
                for r, h in enumerate(handles):
                    if r != rank:
                        self.exchange.OpenPeer(r, bytes(h.cpu().tolist()))
                dist.barrier()
            else:
                self.gathered = [torch.empty(world * op[3][0].numel(), dtype=torch.float32, device="cuda") if op[5] else None
                                 for op in self.ops]
        self.logits_n = VOCAB

    def _launch(self, k, op, stream):
        """Returns the device address of the op's complete output on this rank."""
        rt = self.rt
        _, hs, x, outs, _, span = op
        xb = rt.wrap(x.data_ptr(), x.numel() * 4)
        if span is not None and self.gather_kind == "p2p":
            return self.exchange.GemmMLX(xb, hs[0], 1, span[0], span[1], stream).Ptr
        obs = [rt.wrap(o.data_ptr(), o.numel() * 4) for o in outs]
        if len(hs) == 1:
            rt.GemvMLX(obs[0], xb, hs[0], stream)
        else:
            rt.GemmMLXMulti(obs, xb, hs, 1, stream)
        if span is not None:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.gathered[k], outs[0])
            return self.gathered[k].data_ptr()
        return outs[-1].data_ptr()

    def step(self, stream):
        """One decode step's projections; returns the device address of the logits."""
        ptr = 0
        if self.program is not None:
            self.program.Run(stream)
            ptr = self.ops[self.listed - 1][3][-1].data_ptr()
        for k in range(self.listed, len(self.ops)):
            ptr = self._launch(k, self.ops[k], stream)
        return ptr

    def logits_tensor(self, ptr):
        return self.torch.as_tensor(_Raw(ptr, self.logits_n), device="cuda")

    def timed_launches(self, stream):
        """One eager pass with events around every launch: [(name, bytes, ms)]."""
        torch = self.torch
        evs = []
        for k, op in enumerate(self.ops):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            self._launch(k, op, stream)
            b.record(stream)
            evs.append((op[0], sum(algorithmic_bytes(o, i) for o, i in op[4]), a, b))
        torch.cuda.synchronize()
        return [(n, by, a.elapsed_time(b)) for n, by, a, b in evs]


def cpu_step(orc, syn, nthreads, layers):
    """The same projections through the CPU oracle (mlx.GemvParallel order); returns bytes done."""
    done = 0.0
    ops = [(n, shapes) for _ in range(layers) for n, shapes in LAYER_OPS]
    for name, shapes in ops:
        in_dim = shapes[0][1]
        if name not in cpu_step.cache:
            cpu_step.cache[name] = syn.activations(("x", 0, name), in_dim)
        x = cpu_step.cache[name]
        for i, (out_dim, _) in enumerate(shapes):
            if (name, i) not in cpu_step.cache:
                cpu_step.cache[(name, i)] = syn.mlx_weight((name, i, 0), out_dim, in_dim, GS)
            w, s, b = cpu_step.cache[(name, i)]
            orc.mlx_gemv(x, w, s, b, out_dim, in_dim, GS, nthreads=nthreads)
            done += algorithmic_bytes(out_dim, in_dim)
    return done


cpu_step.cache = {}


def time_cpu(orc, syn, steps, warmup, layers):
    """Times the oracle on all host cores over `layers` layers of the step per repetition."""
    n = os.cpu_count() or 1
    for _ in range(max(1, warmup)):
        cpu_step(orc, syn, n, layers)
    t0 = time.perf_counter()
    total = 0.0
    for _ in range(steps):
        total += cpu_step(orc, syn, n, layers)
    dt = time.perf_counter() - t0
    return total / dt / 1e9, dt / steps * 1e3, n


def run_reference(args):
    """The reference's CPU path for this workload (its Go code cannot be built here: no Go
    toolchain), restated in oracle/ and run on all host cores.  Each step is a bounded sample:
    4 of the 28 layers (the layers are identical in shape), without the LM head."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    syn = load_package().synth
    from oracle import binding as orc
    layers = 4
    gbs, ms, cores = time_cpu(orc, syn, args.steps, args.warmup, layers)
    sample = "%d of 28 layers x 7 projections per step (%.1f MB of packed weights), mlx.GemvParallel order" % (
        layers, layers * 8.85)
    print(json.dumps({
        "impl": "reference", "metric": "quant_gemv_weight_bandwidth", "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "timing": "wall clock, host cores"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def decode_rate(rt, syn, pkg, cpu=False):
    """Greedy decode of the random-init Qwen3-0.6B MLX-4bit model (BASELINE config 1): every operation
    of a token step on the GPU, the step captured once as a CUDA graph; 128 prompt tokens are fed
    one by one, then 64 tokens are generated and those 64 steps are timed with CUDA events."""
    import math
    import types
    import torch
    F = np.float32
    cfg = types.SimpleNamespace(hidden=HIDDEN, layers=LAYERS, heads=16, kv_heads=8, head_dim=128, inter=FFN, vocab=VOCAB,
                                eps=1e-6, theta=1e6, qk_norm=True, max_seq=192)
    shapes = {"q": (QDIM, HIDDEN), "k": (KVDIM, HIDDEN), "v": (KVDIM, HIDDEN), "o": (HIDDEN, QDIM),
              "gate": (FFN, HIDDEN), "up": (FFN, HIDDEN), "down": (HIDDEN, FFN)}
    g = syn.rng("bench-decode")
    base = [{n: syn.mlx_weight(("dec", n, k), o, i, GS) for n, (o, i) in shapes.items()} for k in range(4)]
    layers = []
    for l in range(LAYERS):
        d = dict(base[l % 4])
        for n, sz in (("input_norm", HIDDEN), ("post_norm", HIDDEN), ("q_norm", 128), ("k_norm", 128)):
            d[n] = (F(1) + F(0.1) * g.standard_normal(sz, dtype=F)).astype(F)
        layers.append(d)
    lm = syn.mlx_weight(("dec", "lm"), VOCAB, HIDDEN, GS)
    half = 64
    table = np.empty((cfg.max_seq, half, 2), dtype=F)
    for i in range(half):
        ang = np.arange(cfg.max_seq, dtype=np.float64) * (1.0 / math.pow(cfg.theta, 2.0 * i / 128.0))
        table[:, i, 0], table[:, i, 1] = np.cos(ang).astype(F), np.sin(ang).astype(F)
    dec = pkg.decode.MLXDecoder(rt, cfg, layers, lm, (F(1) + F(0.1) * g.standard_normal(HIDDEN, dtype=F)).astype(F), table)
    prompt = [int(t) for t in g.integers(0, VOCAB, 128)]
    dec.reset(prompt)
    dec.capture()
    dec.reset(prompt)
    for _ in range(127):
        dec.graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(64):
        dec.graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 64
    weight_bytes = 335241216
    cpu_tok_s = None
    if cpu:
        # the same model through the CPU restatement of the reference's loop, a few tokens on all cores
        from oracle import binding as orc
        from oracle import decode as od
        ocfg = od.DecodeConfig(hidden=HIDDEN, layers=LAYERS, heads=16, kv_heads=8, head_dim=128, inter=FFN, vocab=VOCAB,
                               eps=1e-6, theta=1e6, qk_norm=True, max_seq=192)
        lo = [{**{n: (d[n], *shapes[n]) for n in shapes}, **{n: d[n] for n in ("input_norm", "post_norm", "q_norm", "k_norm")}}
              for d in layers]
        oracle = od.OracleDecoder(ocfg, od.MLXWeights(orc, ocfg, lo, lm, np.ones(HIDDEN, dtype=F), nthreads=os.cpu_count() or 1))
        oracle.step(prompt[0], 0)
        t0 = time.perf_counter()
        for p in range(1, 5):
            oracle.step(prompt[p], p)
        cpu_tok_s = round(4 / (time.perf_counter() - t0), 2)
    return {"tok_s": round(1e3 / ms, 1), "cpu_restatement_tok_s": cpu_tok_s, "cpu_cores": (os.cpu_count() or 1) if cpu else None, "ms_per_token": round(ms, 4), "launches_per_token": dec.launches_per_step,
            "positions": "128..191 after a 128-token prompt fed token by token", "batch": 1,
            "weight_GBps": round(weight_bytes / ms / 1e6, 1),
            "gate": "64 greedy tokens identical to the CPU restatement (tests/test_gpu_decode.py::test_greedy_tokens_qwen3_0_6b)"}


def extras(wl):
    """Figures for the other BASELINE configs, measured in the same run with the same harness as
    go-pherence_b200/microbench.py (device time per launch, CUDA-graph replay, weights rotated
    through copies larger than the L2).  Reported beside the headline, not part of it."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("goph_microbench", os.path.join(ROOT, "go-pherence_b200", "microbench.py"))
    mb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mb)
    # free the headline workload's weights first
    for op in wl.ops:
        for h in op[1]:
            h.Free()
    out = {}
    keep = ("us_per_launch", "GBps", "frac_of_hbm_peak")
    out["llama3_8b_gemv_batch1"] = {
        fmt: {"%dx%d" % (o, i): {k: mb.run(fmt, o, i, launches=60)[k] for k in keep}
              for o, i in ((14336, 4096), (128256, 4096))}
        for fmt in ("mlx4", "q4k", "q8_0", "fp8")}
    out["llama3_8b_layer_chain_batch1"] = {
        fmt: {k: v for k, v in mb.run_layer_chain(fmt, layers=6, reps=3).items() if k in ("us_per_layer", "GBps", "frac_of_hbm_peak")}
        for fmt in ("mlx4", "q4k", "q8_0")}
    out["llama3_70b_small_m"] = {
        fmt: {"8192x8192 M=%d" % m: {k: mb.run(fmt, 8192, 8192, batch=m, launches=20)[k] for k in ("us_per_launch",)}
              for m in (1, 4, 16, 64)}
        for fmt in ("mlx4", "fp8")}
    out["qwen3_30b_a3b_moe_layer"] = {
        "T=%d" % t: {k: v for k, v in mb.run_moe(t, layers=2, launches=20).items()
                     if k in ("us_per_call", "GBps", "frac_of_hbm_peak", "distinct_experts_per_call")}
        for t in (1, 8, 32)}
    return out


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(local)
    for o in args.opt:   # tuning: library options (goph_set_option) for this run
        rt.SetOption(o.split("=")[0], int(o.split("=")[1]))
    wl = DecodeStepProjections(rt, syn, pkg.sharding, rank, world, gather=args.gather, shard_min_mb=args.shard_min_mb,
                               product_list=bool(args.list))
    stream = torch.cuda.Stream()
    hbm_peak, peak_kind = peaks()
    p2p = world > 1 and args.gather == "p2p"
    use_graph = bool(args.graph) and (world == 1 or p2p)
    steps_per_graph = 1

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput: the step replayed as a CUDA graph -------------------
    with torch.cuda.stream(stream):
        for _ in range(2 * max(3, args.warmup)):
            wl.step(stream)
    torch.cuda.synchronize()
    graph, graph_logits = None, 0
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(steps_per_graph):
                graph_logits = wl.step(torch.cuda.current_stream())
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    timed_steps = (args.steps + steps_per_graph - 1) // steps_per_graph * steps_per_graph if graph is not None else args.steps

    def run_steps(k):
        if graph is not None:
            for _ in range(k // steps_per_graph):
                graph.replay()
        else:
            with torch.cuda.stream(stream):
                for _ in range(k):
                    wl.step(stream)

    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rec_stream = torch.cuda.current_stream() if graph is not None else stream
    ev0.record(rec_stream)
    run_steps(timed_steps)
    ev1.record(rec_stream)
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    # keep the GPU busy a little longer so the clock sampler sees the loaded state
    t_end = time.time() + 1.0
    while time.time() < t_end:
        run_steps(20)
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None

    # ---- eager launches (no graph), for comparison --------------------------------------
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    with torch.cuda.stream(stream):
        for _ in range(timed_steps):
            wl.step(stream)
    e1.record(stream)
    barrier()
    ms_eager = e0.elapsed_time(e1)

    # ---- end to end: activations from pinned host memory, logits back -------------------
    x_host = wl.x_arena.cpu().pin_memory()
    logits_host = torch.empty(wl.logits_n, dtype=torch.float32).pin_memory()
    h2d = x_host.numel() * 4
    d2h = logits_host.numel() * 4

    def e2e_step():
        wl.x_arena.copy_(x_host, non_blocking=True)   # the step's only outside input: the first product's x
        if graph is not None and steps_per_graph == 1:
            graph.replay()
            ptr = graph_logits
        else:
            ptr = wl.step(torch.cuda.current_stream())
        logits_host.copy_(wl.logits_tensor(ptr), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(4):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(timed_steps):
        e2e_step()
    barrier()
    ms_e2e = (time.perf_counter() - t0) * 1e3

    # ---- roofline of the two kernels: graph replays of their launches alone, CUDA events around -------
    # (events around single eager launches would time the host's launch rate, not the kernels)
    def replay_time(ops_subset, reps):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            cs = torch.cuda.current_stream()
            if ops_subset == "list":
                wl.program.Run(cs)
            else:
                for k, op in ops_subset:
                    wl._launch(k, op, cs)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    indexed = list(enumerate(wl.ops))
    small_ops = [(k, op) for k, op in indexed if op[0] != "lm_head"]
    lm_ops = [(k, op) for k, op in indexed if op[0] == "lm_head"]
    small_bytes = sum(sum(algorithmic_bytes(o, i) for o, i in op[4]) for _, op in small_ops)
    lm_bytes = sum(sum(algorithmic_bytes(o, i) for o, i in op[4]) for _, op in lm_ops)
    listed = wl.program is not None and wl.listed == len(small_ops)
    if use_graph:
        small_ms = replay_time("list" if listed else small_ops, 50)
        # the LM head by difference: replayed alone its 88 MB would stay in the 126 MB L2
        lm_ms = max(ms_total / timed_steps - small_ms, 1e-6)
    else:
        with torch.cuda.stream(stream):
            per = []
            for _ in range(4):
                per = wl.timed_launches(stream)
        small_ms = sum(t for n, _, t in per if n != "lm_head")
        lm_ms = sum(t for n, _, t in per if n == "lm_head")
    lm = ("lm_head", lm_bytes, lm_ms)
    small = small_ops
    k_bytes, k_ms = small_bytes + lm_bytes, small_ms + lm_ms
    status = rt.KernelStatus() + (wl.exchange.Status() if wl.exchange is not None else 0)

    # max over ranks
    times = torch.tensor([ms_total, ms_eager, ms_e2e, float(status)], dtype=torch.float64, device="cuda")
    total_bytes = torch.tensor([wl.bytes_per_step], dtype=torch.float64, device="cuda")
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    ms_total, ms_eager, ms_e2e, status = [float(t) for t in times.cpu()]
    job_bytes = float(total_bytes.cpu()[0])
    if status != 0:
        raise SystemExit("a bounded device-side wait gave up (status %d): the numbers are void" % int(status))

    if rank == 0:
        gbs = job_bytes * timed_steps / (ms_total * 1e-3) / 1e9
        achieved = k_bytes / (k_ms * 1e-3) / 1e9
        lm_gbs = lm[1] / (lm[2] * 1e-3) / 1e9
        small_gbs = small_bytes / (small_ms * 1e-3) / 1e9
        line = {
            "metric": "quant_gemv_weight_bandwidth", "value": round(gbs, 2), "unit": "GB/s", "n_gpus": world,
            "steps": timed_steps, "warmup": 2 * max(3, args.warmup), "ms_per_step": round(ms_total / timed_steps, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch": 1, "launch": "cuda graph replay" if graph is not None else "eager",
                       "product_list": wl.listed,
                       "l2": "inputs larger than L2 (335 MB of weights per step vs 126 MB L2)",
                       "parallelism": ("%d of %d projections (those of %g MB or more packed: the LM head) row-sharded x%d, "
                                       "outputs exchanged through %s; the smaller ones computed whole on every rank and "
                                       "counted once" % (wl.sharded_ops, len(wl.ops), args.shard_min_mb, world,
                                                         "peer memory (one launch per exchange)" if p2p else "NCCL all-gather"))
                       if world > 1 else "single GPU"},
            "decode_tok_s_projections_only": round(timed_steps / (ms_total * 1e-3), 1),
            "eager": {"value": round(job_bytes * timed_steps / (ms_eager * 1e-3) / 1e9, 2), "unit": "GB/s",
                      "ms_per_step": round(ms_eager / timed_steps, 4)},
            "e2e": {"value": round(job_bytes * timed_steps / (ms_e2e * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(ms_e2e / timed_steps, 4)},
            "gpu_launches": wl.launches_per_step * timed_steps,
            # dominant kernel by time (95 % of the step's kernel time in the ncu launch list): the
            # CUDA-core GEMV behind the layer projections; the LM head's tensor-core launch beside it
            "roofline": {"bound": "hbm",
                         "kernel": ("mlx_program_kernel (the %d layer-projection products of a step as one cooperative launch, "
                                    "replayed alone as a CUDA graph, CUDA events around the replays)" % len(small)) if listed else
                                   ("mlx_gemv_kernel (the %d layer-projection launches of a step replayed as a CUDA graph, CUDA "
                                    "events around the replays)" % len(small)),
                         "achieved": round(small_gbs, 1), "peak": hbm_peak, "unit": "GB/s",
                         "frac": round(small_gbs / hbm_peak, 4), "peak_kind": peak_kind,
                         "bytes_per_launch": round(small_bytes if listed else small_bytes / len(small)),
                         "us_per_launch": round((small_ms if listed else small_ms / len(small)) * 1e3, 3),
                         "us_per_product": round(small_ms / len(small) * 1e3, 3),
                         "traffic": round((small_bytes if listed else small_bytes / len(small))
                                          * TRAFFIC_RATIO["mlx_program_kernel" if listed else "mlx_gemv_kernel"]),
                         "lm_head_launch": {"kernel": "mlx_mma_kernel (tcgen05) on %dx%d" % (wl.ops[-1][4][0][0], HIDDEN),
                                            "bytes": lm[1], "ms": round(lm[2], 5), "achieved": round(lm_gbs, 1),
                                            "frac": round(lm_gbs / hbm_peak, 4),
                                            "traffic": round(lm[1] * TRAFFIC_RATIO["mlx_mma_kernel"])},
                         "whole_step": {"achieved": round(achieved, 1), "frac": round(achieved / hbm_peak, 4)}},
            "clocks": clocks,
        }
        if not args.no_extra and world == 1:
            line["extra"] = extras(wl)
            line["decode"] = decode_rate(rt, syn, pkg, cpu=not args.no_cpu)
        if not args.no_cpu and world == 1:
            from oracle import binding as orc
            gbs_cpu, ms_cpu, cores = time_cpu(orc, syn, 3, 1, 4)
            line["cpu_baseline"] = {"value": round(gbs_cpu, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": "3 repetitions of 4 of the 28 layers x 7 projections (35 MB of packed "
                                              "weights each), oracle restatement of mlx.GemvParallel"}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--graph", type=int, default=1)
    ap.add_argument("--shard-min-mb", type=float, default=16.0,
                    help="N>1: projections below this many MB of packed weights are computed whole on every rank")
    ap.add_argument("--gather", default="p2p", choices=["p2p", "nccl"],
                    help="N>1: how the row shards' outputs reach every rank")
    ap.add_argument("--opt", action="append", default=[], help="name=value for goph_set_option (tuning)")
    ap.add_argument("--list", type=int, default=1,
                    help="1: the layer projections run as one product list (a cooperative launch); 0: one launch each")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-format / MoE / small-M figures beside the headline")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
