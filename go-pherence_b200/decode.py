"""Greedy decode of a llama/qwen3-family model with MLX 4-bit projections on one GPU.

Host-side mirror of GPUModel.Generate (model/gpu_forward.go:993-1357) over the C ABI: the seven
projections of a layer run as four fused products (q|k|v, o, gate|up, down) through goph_mlx_gemv,
everything between them through the decode-step operations (goph_add_rmsnorm,
goph_qk_norm_rope_append, goph_attn_decode, goph_silu_mul, goph_argmax_advance, goph_mlx_embed) or
their fused forms (goph_mlx_gemv_pre, goph_attn_decode_fused: five launches per layer), or — with
product lists (goph_mlx_program_create_pre) — everything between two attentions (o, add + norm,
gate|up, SiLU * up, down, add + norm, the next layer's q|k|v) as one cooperative launch: two launches
per layer.
The position, the current token, the prompt and the produced tokens live in device memory, so the
whole step is captured once as a CUDA graph and replayed per token — prompt tokens included (they
are fed one by one, as the reference's sequential loop does).  torch is used for stream capture only.
"""
import math

import numpy as np


class MLXDecoder:
    def __init__(self, rt, cfg, layers, lm_head, final_norm, rope_table, group_size=64, fuse=True, lists=False):
        """cfg: an object with hidden, layers, heads, kv_heads, head_dim, inter, vocab, eps, qk_norm, max_seq.
        layers[l]: dict with "q","k","v","o","gate","up","down" -> (words, scales, biases) in the MLX
        layout, and "input_norm","post_norm" (+ "q_norm","k_norm") f32 vectors.  lm_head: the tied
        [vocab x hidden] MLX weight, also the embedding table.  rope_table: [max_seq][head_dim/2][2] f32."""
        self.rt, self.cfg = rt, cfg
        c = cfg
        qd, kvd = c.heads * c.head_dim, c.kv_heads * c.head_dim
        self.qd, self.kvd = qd, kvd

        def cat(parts):
            return tuple(np.concatenate([p[i] for p in parts]) for i in range(3))

        self.L = []
        for d in layers:
            e = {}
            e["qkv"] = rt.UploadMLXWeight(*cat([d["q"], d["k"], d["v"]]), c.hidden, qd + 2 * kvd, group_size, True)
            e["o"] = rt.UploadMLXWeight(*d["o"], qd, c.hidden, group_size, True)
            e["gate_up"] = rt.UploadMLXWeight(*cat([d["gate"], d["up"]]), c.hidden, 2 * c.inter, group_size, True)
            e["down"] = rt.UploadMLXWeight(*d["down"], c.inter, c.hidden, group_size, True)
            for n in ("input_norm", "post_norm", "q_norm", "k_norm"):
                e[n] = rt.from_numpy(np.asarray(d[n], dtype=np.float32)) if n in d and d[n] is not None else None
            e["kc"], e["vc"] = rt.Malloc(c.max_seq * kvd), rt.Malloc(c.max_seq * kvd)
            self.L.append(e)
        self.lm = rt.UploadMLXWeight(*lm_head, c.hidden, c.vocab, group_size, True)
        self.final_norm = rt.from_numpy(np.asarray(final_norm, dtype=np.float32))
        self.table = rt.from_numpy(np.ascontiguousarray(rope_table, dtype=np.float32).reshape(-1))
        self.hidden, self.hidden2, self.normed = rt.Malloc(c.hidden), rt.Malloc(c.hidden), rt.Malloc(c.hidden)
        self.proj2 = rt.Malloc(c.hidden)
        # the fused launches need the row-major layout (the library keeps projections under 8 Mi weights in it)
        big = 8 << 20
        self.fused = fuse and group_size >= 32 and c.hidden % 32 == 0 and c.inter % 32 == 0 and max(
            (qd + 2 * kvd) * c.hidden, 2 * c.inter * c.hidden, c.inter * c.hidden) < big
        self.qkv, self.attn = rt.Malloc(qd + 2 * kvd), rt.Malloc(qd)
        self.proj, self.gu, self.act = rt.Malloc(c.hidden), rt.Malloc(2 * c.inter), rt.Malloc(c.inter)
        self.logits = rt.Malloc(c.vocab)
        self.ints = rt.MallocBytes(8 + 8 * c.max_seq)   # tok, pos, history[max_seq], forced[max_seq]
        self.tok = rt.wrap(self.ints.Ptr, 4)
        self.pos = rt.wrap(self.ints.Ptr + 4, 4)
        self.history = rt.wrap(self.ints.Ptr + 8, 4 * c.max_seq)
        self.forced = rt.wrap(self.ints.Ptr + 8 + 4 * c.max_seq, 4 * c.max_seq)
        self.scale = 1.0 / math.sqrt(c.head_dim)
        self.graph = None
        self.launches_per_step = 0
        self.lists = self._build_lists() if (self.fused and lists) else None

    def _build_lists(self):
        """The fused step's products grouped between the attentions: [q|k|v of layer 0], then per layer
        [o, gate|up, down, q|k|v of the next layer] (the last without a next).  The buffers rotate exactly
        as in step(); they are the same every token, so the lists are built once."""
        rt, c = self.rt, self.cfg
        cur, other = self.hidden, self.hidden2
        gate, up = self._sub(self.gu, 0, c.inter), self._sub(self.gu, c.inter, c.inter)
        lists, ops, pre, prev = [], [], [], None
        for e in self.L:
            ops.append((cur, [e["qkv"]], [self.qkv]))
            pre.append(dict(op=1, b=prev, w=e["input_norm"], hidden=other if prev is not None else None, eps=c.eps))
            if prev is not None:
                cur, other = other, cur
            lists.append(rt.MLXProgram(ops, pre))
            ops = [(self.attn, [e["o"]], [self.proj]), (cur, [e["gate_up"]], [self.gu]), (gate, [e["down"]], [self.proj2])]
            pre = [None, dict(op=1, b=self.proj, w=e["post_norm"], hidden=other, eps=c.eps), dict(op=2, b=up)]
            cur, other = other, cur
            prev = self.proj2
        lists.append(rt.MLXProgram(ops, pre))
        self._final = (cur, prev)
        return lists

    def _sub(self, buf, off, n):
        return self.rt.wrap(buf.Ptr + 4 * off, 4 * n)

    def step(self, stream=None, dump=None):
        """dump: optional list (plain launches only, not inside a graph capture) that receives
        ("layer<l>.hidden", f32 array) after every layer -- the labelled-tensor hook the reference's
        loop has for layer-by-layer comparison (debugLayerHook, model/gpu_forward.go:883-1542).

        One token: embed the current token, the layer stack, logits, pick and advance.  Where the
        weights allow it (row-major layout: projections under 8 Mi weights) the residual add + RMSNorm
        in front of q|k|v and gate|up and the SiLU*up in front of down run inside the product's launch
        (goph_mlx_gemv_pre); otherwise as separate launches."""
        rt, c = self.rt, self.cfg
        n = 0
        cur, other = self.hidden, self.hidden2
        rt.EmbedMLX(cur, self.lm, self.tok, stream); n += 1
        if self.lists is not None:
            q, k, v = self._sub(self.qkv, 0, self.qd), self._sub(self.qkv, self.qd, self.kvd), self._sub(self.qkv, self.qd + self.kvd, self.kvd)
            for li, e in enumerate(self.L):
                self.lists[li].Run(stream)
                rt.AttnDecodeFused(self.attn, q, k, v, e["q_norm"], e["k_norm"], self.table, self.pos, e["kc"], e["vc"], c.max_seq,
                                   c.heads, c.kv_heads, c.head_dim, self.scale, c.eps, stream)
                n += 2
            self.lists[-1].Run(stream)
            cur, prev = self._final
            rt.AddRMSNorm(None, self.normed, cur, prev, self.final_norm, c.hidden, 1, c.eps, stream)
            rt.GemvMLX(self.logits, self.normed, self.lm, stream)
            rt.ArgmaxAdvance(self.logits, c.vocab, self.tok, self.pos, self.history, self.forced, c.max_seq, stream)
            self.launches_per_step = n + 4 + (1 if self.lm.OutDim * self.lm.InDim >= (8 << 20) else 0)
            return
        prev = None   # the projection output still to be added to the residual stream
        for e in self.L:
            if self.fused:
                # v = cur (+ prev) -> other; q|k|v = W . RMSNorm(v)
                rt.GemvMLXPre(self.qkv, e["qkv"], 1, cur, prev, e["input_norm"], other if prev is not None else None, c.eps, stream)
                if prev is not None:
                    cur, other = other, cur
                n += 1
            else:
                rt.AddRMSNorm(cur if prev is not None else None, self.normed, cur, prev, e["input_norm"], c.hidden, 1, c.eps, stream)
                rt.GemvMLX(self.qkv, self.normed, e["qkv"], stream)
                n += 2
            q, k, v = self._sub(self.qkv, 0, self.qd), self._sub(self.qkv, self.qd, self.kvd), self._sub(self.qkv, self.qd + self.kvd, self.kvd)
            if self.fused:
                rt.AttnDecodeFused(self.attn, q, k, v, e["q_norm"], e["k_norm"], self.table, self.pos, e["kc"], e["vc"], c.max_seq,
                                   c.heads, c.kv_heads, c.head_dim, self.scale, c.eps, stream)
                n += 1
            else:
                rt.QKNormRoPEAppend(q, k, v, e["q_norm"], e["k_norm"], self.table, self.pos, e["kc"], e["vc"], c.max_seq, c.heads, c.kv_heads,
                                    c.head_dim, c.eps, stream)
                rt.AttnDecode(self.attn, q, e["kc"], e["vc"], self.pos, c.max_seq, c.heads, c.kv_heads, c.head_dim, self.scale, stream)
                n += 2
            rt.GemvMLX(self.proj, self.attn, e["o"], stream)
            n += 1
            gate, up = self._sub(self.gu, 0, c.inter), self._sub(self.gu, c.inter, c.inter)
            if self.fused:
                rt.GemvMLXPre(self.gu, e["gate_up"], 1, cur, self.proj, e["post_norm"], other, c.eps, stream)
                cur, other = other, cur
                rt.GemvMLXPre(self.proj2, e["down"], 2, gate, up, None, None, c.eps, stream)
                n += 2
            else:
                rt.AddRMSNorm(cur, self.normed, cur, self.proj, e["post_norm"], c.hidden, 1, c.eps, stream)
                rt.GemvMLX(self.gu, self.normed, e["gate_up"], stream)
                rt.SiLUMul(self.act, gate, up, c.inter, stream)
                rt.GemvMLX(self.proj2, self.act, e["down"], stream)
                n += 4
            prev = self.proj2
            if dump is not None:
                # the residual stream after this layer is cur + prev (the add itself runs inside the
                # next layer's first launch); an f32 add on the host gives the same bits
                rt.Sync()
                dump.append(("layer%d.hidden" % len(dump), cur.Download(c.hidden) + prev.Download(c.hidden)))
        rt.AddRMSNorm(None, self.normed, cur, prev, self.final_norm, c.hidden, 1, c.eps, stream)
        rt.GemvMLX(self.logits, self.normed, self.lm, stream)
        rt.ArgmaxAdvance(self.logits, c.vocab, self.tok, self.pos, self.history, self.forced, c.max_seq, stream)
        self.launches_per_step = n + 3 + (1 if self.lm.OutDim * self.lm.InDim >= (8 << 20) else 0)

    def reset(self, prompt):
        c = self.cfg
        ints = np.full(2 + 2 * c.max_seq, -1, dtype=np.int32)
        ints[0], ints[1] = prompt[0], 0
        ints[2:2 + len(prompt)] = prompt                       # history
        ints[2 + c.max_seq:2 + c.max_seq + len(prompt)] = prompt   # forced
        self.ints.UploadBytes(ints.view(np.uint8))

    def capture(self):
        import torch
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            self.step(s)      # warm-up outside capture: lazy allocations happen here
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=s):
            self.step(torch.cuda.current_stream())
        return self.graph

    def generate(self, prompt, max_new, use_graph=True, logits_at=None, logits_all=None):
        """Returns prompt + max_new greedy tokens.  logits_at: optional list that receives the logits
        (numpy) that chose each generated token; logits_all: the logits of every position, prompt
        positions included."""
        c = self.cfg
        total = len(prompt) + max_new
        if total > c.max_seq:
            raise ValueError("sequence %d exceeds max_seq %d" % (total, c.max_seq))
        if use_graph and self.graph is None:
            self.reset(prompt)
            self.capture()
        self.reset(prompt)
        for i in range(total - 1):
            if use_graph:
                self.graph.replay()
            else:
                self.step(None)
            if logits_at is not None and i >= len(prompt) - 1:
                self.rt.Sync()
                logits_at.append(self.logits.Download())
            if logits_all is not None:
                self.rt.Sync()
                logits_all.append(self.logits.Download())
        self.rt.Sync()
        hist = self.history.Download(c.max_seq, dtype=np.int32)
        return [int(t) for t in hist[:total]]
