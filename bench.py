#!/usr/bin/env python
"""Headline benchmark: quantized-GEMV weight bandwidth over the projections of one Llama-3-8B
decode token in MLX 4-bit g64 form.

One step = every linear projection one decode token needs, as the dependent chain a decode step
forms: per layer q|k|v (6144x4096, the three weights stacked by rows), o (4096x4096), gate|up
(28672x4096, stacked), down (4096x14336) -- 32 layers -- then the 128256x4096 LM head.  129
products, 4.2 GB of packed weights per step (33 times the L2, so every step streams them from
HBM).  Every product reads what the product before it wrote; only the first x comes from outside.
Data is synthetic and seeded.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is GB/s of algorithmic bytes with everything resident in HBM;
`e2e` is the same step with the first activations copied from pinned host memory and the logits
copied back inside the timed region.  With N > 1 (one rank per GPU) every projection is
row-sharded over the ranks and each product is followed by the exchange that leaves the whole
output on every rank; before anything is timed each kind of sharded product is compared with the
same product computed whole on the rank, and a mismatch ends the run with a non-zero exit code.
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

HIDDEN, LAYERS, VOCAB, FFN, QKV, GS = 4096, 32, 128256, 14336, 6144, 64
# (name, out_dim, in_dim): the weights that share an x are stacked by rows into one matrix
LAYER_OPS = [("qkv", QKV, HIDDEN), ("o", HIDDEN, HIDDEN), ("gate_up", 2 * FFN, HIDDEN), ("down", HIDDEN, FFN)]
WORKLOAD = ("llama-3-8b mlx4-g64 decode-step projections as a dependent chain (32 layers x q|k|v 6144x4096, o 4096x4096, "
            "gate|up 28672x4096, down 4096x14336 + LM head 128256x4096), batch 1")
# Share of the step's kernel time spent in mlx_mma_kernel (the rest is mlx_prep_x_kernel, the
# activation-digit launch in front of 97 of the 129 products), from the ncu launch list of this
# program, and DRAM bytes over algorithmic bytes of that kernel, from its ncu captures at
# 14336x4096 (1.000) and 128256x4096 (1.012); both summarised under profiles/.
MMA_SHARE = 0.856
MMA_TRAFFIC_RATIO = 1.003


def algorithmic_bytes(out_dim, in_dim, batch=1):
    """0.5625 B per weight (4-bit nibble + bf16 scale and bias per 64) + f32 x + f32 out."""
    return out_dim * in_dim * 0.5625 + batch * in_dim * 4 + batch * out_dim * 4


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


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


def chain_ops(layers):
    return [(l, n, o, i) for l in range(layers) for n, o, i in LAYER_OPS] + [(layers, "lm_head", VOCAB, HIDDEN)]


# Exact (power-of-two) factors on the scales that keep the chain's values in range: the gain of a
# product is sqrt(in_dim * E[(n - 7.5)^2] * E[scale^2]) = 0.77 (in 4096) or 1.44 (in 14336) at
# 0.125 and twice that at 0.25; a layer's four products then multiply to 1.3, 32 layers to ~5e3.
CHAIN_GAIN = {"qkv": 0.125, "o": 0.25, "gate_up": 0.125, "down": 0.125, "lm_head": 0.125}


def chain_weight(syn, name, l, out_dim, in_dim):
    """Every layer of a random-init model has its own weights; generation is the slow part on the
    host, so layers draw from 4 distinct seeds per projection (contents never repeat in L2: the
    copies are separate device buffers).  The biases are -7.5 x scale (rounded to bf16), so a weight
    has mean zero and a product does not amplify the mean of its input — with the generator's -8 x
    scale the mean grew fourfold per product and the chain overflowed after a few layers."""
    key = (name, l % 4)
    if key not in chain_weight.cache:
        w, s, _ = syn.mlx_weight(("chain",) + key, out_dim, in_dim, GS)
        s = s * np.float32(CHAIN_GAIN[name])
        chain_weight.cache[key] = (w, s, syn.bf16_round(np.float32(-7.5) * s))
    return chain_weight.cache[key]


chain_weight.cache = {}


class DecodeStepProjections:
    """Weights, activation buffers and the launch list of one decode step's projections.

    One GPU: one handle per projection.  Several GPUs: every rank uploads its row shard of every
    projection, and each product is followed by the peer-memory exchange that leaves the whole
    output on every rank (`gather="p2p"`), or by an NCCL all-gather (`gather="nccl"`, kept as the
    library baseline)."""

    def __init__(self, rt, syn, sharding, rank=0, world=1, layers=LAYERS, gather="p2p"):
        import torch
        self.rt, self.torch, self.rank, self.world, self.gather_kind, self.syn, self.sharding = rt, torch, rank, world, gather, syn, sharding
        self.ops = []  # (name, handle, x_tensor or None (x is the exchange's result), out_tensor, (out_shard, in_dim), (lo, out_full))
        self.weight_bytes = 0
        self.bytes_per_step = 0.0
        self.x_arena = torch.from_numpy(syn.activations(("x", 0), HIDDEN)).cuda()
        prev_out = None
        self.op_layer = [l for l, _, _, _ in chain_ops(layers)]
        for l, name, out_dim, in_dim in chain_ops(layers):
            w, s, b = chain_weight(syn, name, l, out_dim, in_dim)
            lo, hi = sharding.shard_rows(out_dim, rank, world) if world > 1 else (0, out_dim)
            if world > 1:
                w, s, b = sharding.slice_mlx(w, s, b, in_dim, GS, lo, hi)
            h = rt.UploadMLXWeight(w, s, b, in_dim, hi - lo, GS, True)
            out = torch.empty(hi - lo, dtype=torch.float32, device="cuda")
            x = self.x_arena if prev_out is None else (prev_out[:in_dim] if world == 1 else None)
            self.weight_bytes += h.ResidentBytes()
            self.bytes_per_step += algorithmic_bytes(hi - lo, in_dim)
            self.ops.append((name, h, x, out, (hi - lo, in_dim), (lo, out_dim)))
            prev_out = out
        self.launches_per_step = 0  # set from the library's launch counter over one step
        self.exchange = None
        if world > 1:
            import torch.distributed as dist
            if gather == "p2p":
                self.exchange = rt.Gather(rank, world, max(VOCAB + 64, world * 32 * 2048))  # logits, or the MoE partial sums of 32 tokens
                handles = [torch.zeros(64, dtype=torch.uint8, device="cuda") for _ in range(world)]
                mine = torch.tensor(list(self.exchange.Export()), dtype=torch.uint8, device="cuda")
                dist.all_gather(handles, mine)
                for r, h in enumerate(handles):
                    if r != rank:
                        self.exchange.OpenPeer(r, bytes(h.cpu().tolist()))
                dist.barrier()
            else:
                self.gathered = [torch.empty(world * op[3].numel(), dtype=torch.float32, device="cuda") for op in self.ops]
        self.logits_n = VOCAB

    def _launch(self, k, op, x_ptr, stream):
        """Runs product k on x at device address x_ptr; returns the address of its complete output."""
        rt = self.rt
        _, h, _, out, (_, in_dim), (lo, out_full) = op
        xb = rt.wrap(x_ptr, in_dim * 4)
        if self.world > 1 and self.gather_kind == "p2p":
            return self.exchange.GemmMLX(xb, h, 1, lo, out_full, stream).Ptr
        rt.GemvMLX(rt.wrap(out.data_ptr(), out.numel() * 4), xb, h, stream)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.gathered[k], out)
            return self.gathered[k].data_ptr()
        return out.data_ptr()

    def step(self, stream):
        """One decode step's projections; returns the device address of the logits."""
        ptr = self.x_arena.data_ptr()
        for k, op in enumerate(self.ops):
            ptr = self._launch(k, op, ptr, stream)
        return ptr

    def logits_tensor(self, ptr):
        return self.torch.as_tensor(_Raw(ptr, self.logits_n), device="cuda")

    def verify_sharding(self, stream):
        """Each kind of sharded product against the same product computed whole on this rank (layer
        0's projections and the LM head, each on the x the chain gives it).  Returns the largest
        relative difference; the caller ends the run when it is not at rounding level."""
        rt, torch, syn = self.rt, self.torch, self.syn
        worst = 0.0
        ptr = self.x_arena.data_ptr()
        kinds = {0: "qkv", 1: "o", 2: "gate_up", 3: "down", len(self.ops) - 1: "lm_head"}
        for k, op in enumerate(self.ops):
            name, _, _, _, (_, in_dim), (_, out_full) = op
            if k in kinds:
                x_host = torch.as_tensor(_Raw(ptr, in_dim), device="cuda").cpu().numpy().copy()
            nxt = self._launch(k, op, ptr, stream)
            if k in kinds:
                torch.cuda.synchronize()
                got = torch.as_tensor(_Raw(nxt, out_full), device="cuda").cpu().numpy().copy()
                w, s, b = chain_weight(syn, name, self.op_layer[k], out_full, in_dim)
                full = rt.UploadMLXWeight(w, s, b, in_dim, out_full, GS, True)
                xo, oo = rt.from_numpy(x_host), rt.Malloc(out_full)
                rt.GemvMLX(oo, xo, full)
                rt.Sync()
                want = oo.Download()
                if not (np.isfinite(got).all() and np.isfinite(want).all()):
                    return float("inf")  # a chain that overflowed proves nothing
                worst = max(worst, syn.rel_err(got, want))
                for t in (full, xo, oo):
                    t.Free()
            ptr = nxt
        torch.cuda.synchronize()
        return worst


def cpu_step(orc, syn, nthreads, layers):
    """The same projections through the CPU oracle (mlx.GemvParallel order); returns bytes done."""
    done = 0.0
    for l in range(layers):
        for name, out_dim, in_dim in LAYER_OPS:
            if name not in cpu_step.cache:
                cpu_step.cache[name] = syn.activations(("x", 0, name), in_dim)
            w, s, b = chain_weight(syn, name, l, out_dim, in_dim)
            orc.mlx_gemv(cpu_step.cache[name], w, s, b, out_dim, in_dim, GS, nthreads=nthreads)
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


CPU_SAMPLE = "%d of 32 layers x 4 projections per step (%.0f MB of packed weights), oracle restatement of mlx.GemvParallel"


def run_reference(args):
    """The reference's CPU path for this workload (its Go code cannot be built here: no Go
    toolchain), restated in oracle/ and run on all host cores.  Each step is a bounded sample:
    2 of the 32 layers (the layers are identical in shape), without the LM head."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    syn = load_package().synth
    from oracle import binding as orc
    layers = 2
    gbs, ms, cores = time_cpu(orc, syn, args.steps, min(args.warmup, 2), layers)
    sample = CPU_SAMPLE % (layers, layers * 122.7)
    print(json.dumps({
        "impl": "reference", "metric": "quant_gemv_weight_bandwidth", "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": 1, "layers": LAYERS, "products_per_step": len(chain_ops(LAYERS)),
                   "packed_weight_bytes_per_step": int(sum(0.5625 * o * i for _, _, o, i in chain_ops(LAYERS))),
                   "launch": "host threads, wall clock; every step is the bounded sample named in cpu_baseline",
                   "l2": "inputs larger than L2 (4.2 GB of weights per step vs 126 MB L2)",
                   "parallelism": "host cores"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def decode_rate(rt, syn, pkg, cpu=False):
    """Greedy decode of a random-init Qwen3-0.6B-architecture model in MLX 4-bit g64 (28 layers,
    hidden 1024, 16/8 heads of 128, FFN 3072, tied 151936x1024 LM head): every operation of a token
    step on the GPU, the step captured once as a CUDA graph; 128 prompt tokens are fed one by one,
    then 64 tokens are generated and those 64 steps are timed with CUDA events."""
    import math
    import types
    import torch
    F = np.float32
    hidden, nlayers, vocab, ffn, qdim, kvdim = 1024, 28, 151936, 3072, 2048, 1024
    cfg = types.SimpleNamespace(hidden=hidden, layers=nlayers, heads=16, kv_heads=8, head_dim=128, inter=ffn, vocab=vocab,
                                eps=1e-6, theta=1e6, qk_norm=True, max_seq=192)
    shapes = {"q": (qdim, hidden), "k": (kvdim, hidden), "v": (kvdim, hidden), "o": (hidden, qdim),
              "gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
    g = syn.rng("bench-decode")
    base = [{n: syn.mlx_weight(("dec", n, k), o, i, GS) for n, (o, i) in shapes.items()} for k in range(4)]
    layers = []
    for l in range(nlayers):
        d = dict(base[l % 4])
        for n, sz in (("input_norm", hidden), ("post_norm", hidden), ("q_norm", 128), ("k_norm", 128)):
            d[n] = (F(1) + F(0.1) * g.standard_normal(sz, dtype=F)).astype(F)
        layers.append(d)
    lm = syn.mlx_weight(("dec", "lm"), vocab, hidden, GS)
    final_norm = (F(1) + F(0.1) * g.standard_normal(hidden, dtype=F)).astype(F)
    half = 64
    table = np.empty((cfg.max_seq, half, 2), dtype=F)
    for i in range(half):
        ang = np.arange(cfg.max_seq, dtype=np.float64) * (1.0 / math.pow(cfg.theta, 2.0 * i / 128.0))
        table[:, i, 0], table[:, i, 1] = np.cos(ang).astype(F), np.sin(ang).astype(F)
    dec = pkg.decode.MLXDecoder(rt, cfg, layers, lm, final_norm, table)
    prompt = [int(t) for t in g.integers(0, vocab, 128)]
    dec.reset(prompt)
    dec.capture()
    dec.reset(prompt)
    first_logits = []
    for p in range(127):
        dec.graph.replay()
        if cpu and p < 4:
            torch.cuda.synchronize()
            first_logits.append(dec.logits.Download(vocab).copy())
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(64):
        dec.graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 64
    weight_bytes = 335241216
    res = {"model": "random-init qwen3-0.6b architecture, mlx4-g64", "tok_s": round(1e3 / ms, 1), "ms_per_token": round(ms, 4),
           "launches_per_token": dec.launches_per_step, "positions": "128..191 after a 128-token prompt fed token by token",
           "batch": 1, "weight_GBps": round(weight_bytes / ms / 1e6, 1)}
    if cpu:
        # the same model through the CPU restatement of the reference's loop: a few tokens on all
        # cores for its rate, and the logits of those positions against the GPU's
        from oracle import binding as orc
        from oracle import decode as od
        ocfg = od.DecodeConfig(hidden=hidden, layers=nlayers, heads=16, kv_heads=8, head_dim=128, inter=ffn, vocab=vocab,
                               eps=1e-6, theta=1e6, qk_norm=True, max_seq=192)
        lo = [{**{n: (d[n], *shapes[n]) for n in shapes}, **{n: d[n] for n in ("input_norm", "post_norm", "q_norm", "k_norm")}}
              for d in layers]
        oracle = od.OracleDecoder(ocfg, od.MLXWeights(orc, ocfg, lo, lm, final_norm, nthreads=os.cpu_count() or 1))
        worst = 0.0
        t0 = time.perf_counter()
        for p in range(4):
            ref = oracle.step(prompt[p], p)
            worst = max(worst, float(np.max(np.abs(first_logits[p] - ref)) / np.max(np.abs(ref))))
        res["cpu_restatement_tok_s"] = round(4 / (time.perf_counter() - t0), 2)
        res["cpu_cores"] = os.cpu_count() or 1
        res["max_logit_diff_vs_cpu_restatement"] = {"positions": "0..3", "value": float("%.3g" % worst),
                                                    "unit": "max|dlogit| / max|logit|"}
    return res


def extras(tensor_peak):
    """Figures for the other workloads of the path, measured in the same run with the harness of
    go-pherence_b200/microbench.py (device time per launch, CUDA-graph replay, weights rotated
    through copies larger than the L2).  Reported beside the headline, not part of it."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("goph_microbench", os.path.join(ROOT, "go-pherence_b200", "microbench.py"))
    mb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mb)
    out = {}
    keep = ("us_per_launch", "GBps", "frac_of_hbm_peak")
    def one(fmt, o, i):
        r = mb.run(fmt, o, i, launches=60)
        return {k: r[k] for k in keep}

    # (Q5_K / Q6_K fractions are on the FILE's bytes per weight; on the device their tensor-core layout is a byte per weight)
    out["llama3_8b_gemv_batch1"] = {
        fmt: {"%dx%d" % (o, i): one(fmt, o, i) for o, i in ((14336, 4096), (4096, 14336), (128256, 4096))}
        for fmt in ("mlx4", "q4k", "q5k", "q6k", "q8_0", "fp8")}
    out["llama3_8b_layer_chain_batch1"] = {
        fmt: {k: v for k, v in mb.run_layer_chain(fmt, layers=6, reps=3).items() if k in ("us_per_layer", "GBps", "frac_of_hbm_peak")}
        for fmt in ("q4k", "q8_0")}
    small = {}
    for fmt in ("mlx4", "fp8"):
        small[fmt] = {}
        for o, i in ((8192, 8192), (28672, 8192), (8192, 28672)):
            for m in (1, 4, 16, 64, 256):
                r = mb.run(fmt, o, i, batch=m, launches=12, xbf16=m >= 16)
                small[fmt]["%dx%d M=%d" % (o, i, m)] = {
                    "x": r["x"], "us_per_launch": r["us_per_launch"], "frac_of_hbm_peak": r["frac_of_hbm_peak"],
                    "tflops": r["tflops"], "frac_of_bf16_tensor_peak": round(r["tflops"] / tensor_peak, 4)}
    out["llama3_70b_small_m"] = small
    # the work-list GGUF products over stacked experts (Q4_K gate|up with GELU, Q8_0 down with scatter-add)
    out["gguf_work_list_stacked_experts"] = {
        "T=%d" % t: {k: v for k, v in mb.run_gguf_work(t, launches=10).items()
                     if k in ("items", "us_per_call", "GBps", "frac_of_hbm_peak", "distinct_experts_per_call")}
        for t in (1, 8, 32)}
    # experts row-major (CUDA-core expert kernels) and tiled (grouped launches of the tensor-core kernel)
    for name, layout in (("qwen3_30b_a3b_moe_layer", 1), ("qwen3_30b_a3b_moe_layer_tiled_experts", 2)):
        out[name] = {
            "T=%d" % t: {k: v for k, v in mb.run_moe(t, layers=2, launches=20, expert_layout=layout).items()
                         if k in ("us_per_call", "GBps", "frac_of_hbm_peak", "distinct_experts_per_call")}
            for t in (1, 8, 32)}
    return out


def moe_sharded(rt, syn, sharding, exchange, rank, world, dist):
    """Selected-expert projection at the Qwen3-30B-A3B layer shape with the 128 experts placed
    128/N per GPU: every rank routes the same tokens, computes the partial sums of the experts it
    holds, and the partials are exchanged and added in rank order.  Device time per call (CUDA
    events around a graph replay of 20 calls over 2 distinct layers), max over ranks."""
    import torch
    experts, hidden, inter, top_k = 128, 2048, 768, 8
    g = syn.rng("moe-sharded")

    def build(expert_layout):
        mods = []
        for l in range(2):
            m = rt.GPUMoELayer(experts, hidden, inter, 64, top_k, True, 32)
            rt.SetOption("mlx_layout", 1)
            r = rt.UploadMLXWeight(*syn.mlx_weight(("r", l), experts, hidden, 64), hidden, experts, 64, True)
            m.SetRouter(r)
            keep.append(r)
            gen = syn.rng("moe-sharded", l)
            rt.SetOption("mlx_layout", expert_layout)
            for e in range(experts):
                arrs = []
                for o, i in ((inter, hidden), (inter, hidden), (hidden, inter)):
                    w = gen.integers(0, 2**32, size=o * i // 8, dtype=np.uint32)
                    sc = syn.bf16_round(np.abs(gen.standard_normal(o * i // 64, dtype=np.float32)) * np.float32(0.02) + np.float32(1e-3))
                    arrs.append((w, sc, syn.bf16_round(np.float32(-8) * sc), i, o))
                if e in sharding.place_experts(experts, rank, world):
                    hs = [rt.UploadMLXWeight(w, sc, bi, i, o, 64, True) for w, sc, bi, i, o in arrs]
                    m.SetExpert(e, *hs)
                    keep.extend(hs)
            mods.append(m)
        rt.SetOption("mlx_layout", 0)
        return mods

    keep = []
    # experts row-major (CUDA-core kernels; one launch at one token) and tiled (grouped tensor-core launches)
    forms = {"row_major_experts": build(1), "tiled_experts": build(2)}
    res = {}
    for tokens in (1, 8, 32):
        x = torch.from_numpy(syn.activations(("moe-sharded", tokens), tokens * hidden)).cuda()
        out = torch.empty(tokens * hidden, dtype=torch.float32, device="cuda")
        xb, ob = rt.wrap(x.data_ptr(), x.numel() * 4), rt.wrap(out.data_ptr(), out.numel() * 4)
        entry = {"experts_per_gpu": experts // world}
        for name, mods in forms.items():
            for m in mods:
                exchange.MoEForward(m, ob, xb, tokens, torch.cuda.current_stream())
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(20):
                    exchange.MoEForward(mods[i % 2], ob, xb, tokens, torch.cuda.current_stream())
            graph.replay()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                graph.replay()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / 60 * 1e3], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            entry["us_per_call_" + name] = round(float(t.cpu()[0]), 2)
        entry["us_per_call"] = min(entry["us_per_call_row_major_experts"], entry["us_per_call_tiled_experts"])
        res["T=%d" % tokens] = entry
    return res


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    rt, syn = pkg.runtime, pkg.synth
    rt.init(local)
    for o in args.opt:   # tuning: library options (goph_set_option) for this run
        rt.SetOption(o.split("=")[0], int(o.split("=")[1]))
    wl = DecodeStepProjections(rt, syn, pkg.sharding, rank, world, layers=args.layers, gather=args.gather)
    stream = torch.cuda.Stream()
    hbm_peak, tensor_peak, peak_kind = peaks()
    p2p = world > 1 and args.gather == "p2p"
    use_graph = bool(args.graph) and (world == 1 or p2p)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- N > 1: the sharded products against the whole products, before anything is timed ----
    shard_check = None
    if world > 1:
        with torch.cuda.stream(stream):
            worst = wl.verify_sharding(stream)
        t = torch.tensor([worst], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = float(t.cpu()[0])
        # (the measure divides by max(|whole|, 1e-3 max|whole|): f32 sums taken in another split order differ
        # by ~1e-6 of the largest output, i.e. up to ~1e-3 here; the bound is the products' tolerance against the oracle)
        if not worst <= 2e-3:
            raise SystemExit("row-sharded products differ from the whole products: relative difference %.3g" % worst)
        shard_check = {"max_rel_diff_vs_whole_product": float("%.3g" % worst), "products": "layer 0's four and the LM head, on every rank"}

    # ---- device-resident throughput: the step replayed as a CUDA graph -------------------
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            n0 = rt.LaunchCount()
            logits_ptr = wl.step(stream)
            wl.launches_per_step = rt.LaunchCount() - n0  # kernels of one step, counted by the library
    torch.cuda.synchronize()
    lg = wl.logits_tensor(logits_ptr)
    if not bool(torch.isfinite(lg).all()) or float(lg.abs().max()) == 0.0:
        raise SystemExit("the chained activations overflowed or vanished: the step's logits are not finite, non-zero values")
    logit_absmax = float(lg.abs().max())
    graph, graph_logits = None, 0
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            graph_logits = wl.step(torch.cuda.current_stream())
        graph.replay()
        torch.cuda.synchronize()
    timed_steps = args.steps

    def run_steps(k):
        if graph is not None:
            for _ in range(k):
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
        run_steps(5)
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
        if graph is not None:
            graph.replay()
            ptr = graph_logits
        else:
            ptr = wl.step(torch.cuda.current_stream())
        logits_host.copy_(wl.logits_tensor(ptr), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(timed_steps):
        e2e_step()
    barrier()
    ms_e2e = (time.perf_counter() - t0) * 1e3

    status = rt.KernelStatus() + (wl.exchange.Status() if wl.exchange is not None else 0)

    # max over ranks
    times = torch.tensor([ms_total, ms_eager, ms_e2e, float(status)], dtype=torch.float64, device="cuda")
    total_bytes = torch.tensor([wl.bytes_per_step], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    ms_total, ms_eager, ms_e2e, status = [float(t) for t in times.cpu()]
    job_bytes = float(total_bytes.cpu()[0])
    if status != 0:
        raise SystemExit("a bounded device-side wait gave up (status %d): the numbers are void" % int(status))

    moe = None
    if world > 1 and p2p and not args.no_extra:
        for op in wl.ops:  # make room: the chain's weights are not needed any more
            op[1].Free()
        try:
            moe = moe_sharded(rt, syn, pkg.sharding, wl.exchange, rank, world, dist)
        except Exception as e:  # the headline stands without it
            moe = {"error": str(e)[:200]}

    if rank == 0:
        gbs = job_bytes * timed_steps / (ms_total * 1e-3) / 1e9
        n_products = len(wl.ops)
        ms_step = ms_total / timed_steps
        # the tensor-core GEMV kernel of this rank: its share of the step's device time
        rank_bytes = wl.bytes_per_step
        mma_ms = ms_step * MMA_SHARE
        achieved = rank_bytes / (mma_ms * 1e-3) / 1e9
        line = {
            "metric": "quant_gemv_weight_bandwidth", "value": round(gbs, 2), "unit": "GB/s", "n_gpus": world,
            "steps": timed_steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch": 1, "layers": args.layers, "products_per_step": n_products,
                       "packed_weight_bytes_per_step": int(sum(0.5625 * o * i for _, _, o, i in chain_ops(args.layers))),
                       "launch": "cuda graph replay" if graph is not None else "eager",
                       "l2": "inputs larger than L2 (4.2 GB of weights per step vs 126 MB L2)",
                       "parallelism": ("every projection row-sharded x%d, outputs exchanged through %s" % (
                           world, "peer memory (one launch per exchange)" if p2p else "NCCL all-gather"))
                       if world > 1 else "single GPU"},
            "frac_of_hbm_peak": round(gbs / (hbm_peak * world), 4),
            "logits_absmax": float("%.3g" % logit_absmax),  # the chained values stayed finite and non-zero
            "decode_tok_s_projections_only": round(timed_steps / (ms_total * 1e-3), 1),
            "eager": {"value": round(job_bytes * timed_steps / (ms_eager * 1e-3) / 1e9, 2), "unit": "GB/s",
                      "ms_per_step": round(ms_eager / timed_steps, 4)},
            "e2e": {"value": round(job_bytes * timed_steps / (ms_e2e * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(ms_e2e / timed_steps, 4)},
            "gpu_launches": wl.launches_per_step * timed_steps,
            "roofline": {"bound": "hbm",
                         "kernel": ("mlx_mma_kernel (tcgen05 GEMV): %d launches per step; its duration is the step's CUDA-event "
                                    "time times its share of the step's serialised kernel time in the ncu launch list (%.3f; "
                                    "the other launches are mlx_prep_x_kernel, which live runs inside the product kernels' "
                                    "prologues: the whole step is frac_of_hbm_peak)" % (n_products, MMA_SHARE)),
                         "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                         "frac": round(achieved / hbm_peak, 4), "peak_kind": peak_kind,
                         "bytes_per_launch": round(rank_bytes / n_products),
                         "us_per_launch": round(mma_ms / n_products * 1e3, 3),
                         "traffic": round(rank_bytes / n_products * MMA_TRAFFIC_RATIO)},
            "clocks": clocks,
        }
        if shard_check is not None:
            line["shard_check"] = shard_check
        if moe is not None:
            line["moe_sharded_qwen3_30b_a3b_layer"] = moe
        if not args.no_extra and world == 1:
            for op in wl.ops:  # free the headline workload's weights first
                op[1].Free()
            chain_weight.cache.clear()
            line["extra"] = extras(tensor_peak)
            line["decode"] = decode_rate(rt, syn, pkg, cpu=not args.no_cpu)
        if not args.no_cpu and world == 1:
            from oracle import binding as orc
            gbs_cpu, ms_cpu, cores = time_cpu(orc, syn, 10, 1, 2)
            line["cpu_baseline"] = {"value": round(gbs_cpu, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": "10 repetitions of " + CPU_SAMPLE % (2, 2 * 122.7)}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--graph", type=int, default=1)
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of the chain (tuning; the headline uses all 32)")
    ap.add_argument("--gather", default="p2p", choices=["p2p", "nccl"],
                    help="N>1: how the row shards' outputs reach every rank")
    ap.add_argument("--opt", action="append", default=[], help="name=value for goph_set_option (tuning)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-format / MoE / small-M figures beside the headline")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
