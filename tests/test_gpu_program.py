"""Product lists (goph_mlx_program_*): many dependent batch-1 products in one cooperative launch."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def chain(gpu, pkg, dims, gs=64):
    """dims: [(in, [outs])]; the first output of a product is the next product's x."""
    syn = pkg.synth
    x0 = gpu.from_numpy(syn.activations("prog", dims[0][0], bf16=False))
    ops, x = [], x0
    for k, (in_dim, outs) in enumerate(dims):
        hs = [gpu.UploadMLXWeight(*syn.mlx_weight(("prog", k, i), o, in_dim, gs), in_dim, o, gs, True) for i, o in enumerate(outs)]
        os_ = [gpu.Malloc(o) for o in outs]
        ops.append((x, hs, os_))
        x = os_[0]
    return x0, ops


def run_separately(gpu, ops):
    for x, hs, os_ in ops:
        if len(hs) == 1:
            gpu.GemvMLX(os_[0], x, hs[0])
        else:
            gpu.GemmMLXMulti(os_, x, hs, 1)
    gpu.Sync()
    return [o.Download() for _, _, os_ in ops for o in os_]


DIMS = [(1024, [2048]), (2048, [1024, 512, 96]), (1024, [3072]), (3072, [1024]), (1024, [40])]


def test_list_equals_separate_launches_bit_for_bit(gpu, pkg):
    x0, ops = chain(gpu, pkg, DIMS)
    want = run_separately(gpu, ops)
    for _, _, os_ in ops:
        for o in os_:
            o.Upload(np.full(o.n, 7.0, dtype=np.float32))
    prog = gpu.MLXProgram(ops)
    for rep in range(3):   # the barrier counter carries over from launch to launch
        prog.Run()
        gpu.Sync()
        got = [o.Download() for _, _, os_ in ops for o in os_]
        for g, w in zip(got, want):
            assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), rep
        assert prog.Status() == 0
    prog.Free(); prog.Free()
    with pytest.raises(gpu.GophError):
        prog.Run()


def test_list_replays_in_a_cuda_graph_with_new_inputs(gpu, pkg):
    import torch
    x0, ops = chain(gpu, pkg, DIMS)
    prog = gpu.MLXProgram(ops)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        prog.Run(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        prog.Run(torch.cuda.current_stream())
    for k in range(4):
        x0.Upload(pkg.synth.activations(("prog-x", k), DIMS[0][0], bf16=False))
        g.replay()
        torch.cuda.synchronize()
        got = [o.Download() for _, _, os_ in ops for o in os_]
        want = run_separately(gpu, ops)
        for a, b in zip(got, want):
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), k
    assert prog.Status() == 0
    prog.Free()


def test_ping_pong_buffers_and_independent_products(gpu, pkg):
    """Two buffers used alternately (every product overwrites the x of the product before it), then
    products that do not depend on each other but share memory: the list must order them as
    separate launches on one stream would."""
    syn = pkg.synth
    n = 1024
    bufs = [gpu.Malloc(n), gpu.Malloc(n)]
    bufs[0].Upload(syn.activations("pp", n, bf16=False))
    ws = [gpu.UploadMLXWeight(*syn.mlx_weight(("pp", k), n, n, 64), n, n, 64, True) for k in range(6)]
    ops = [(bufs[k & 1], [ws[k]], [bufs[1 - (k & 1)]]) for k in range(6)]
    # an unrelated product that overwrites the very first x while the chain may still be reading it,
    # and one more reading that result through a sub-range that straddles nothing (whole buffer)
    ext, side = gpu.from_numpy(syn.activations("pp-ext", n, bf16=False)), gpu.Malloc(n)
    ops.append((ext, [ws[0]], [bufs[0]]))
    ops.append((bufs[0], [ws[1]], [side]))
    x0 = bufs[0].Download()
    want = run_separately(gpu, ops)
    final = [b.Download() for b in bufs] + [side.Download()]
    prog = gpu.MLXProgram(ops)
    for rep in range(3):
        bufs[0].Upload(x0)
        prog.Run()
        gpu.Sync()
        got = [b.Download() for b in bufs] + [side.Download()]
        for g, w in zip(got, final):
            assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), rep
        assert prog.Status() == 0
    prog.Free()
    with pytest.raises(gpu.GophError):      # a product may not overwrite its own x
        gpu.MLXProgram([(bufs[0], [ws[0]], [bufs[0]])])


def test_x_straddling_two_outputs_waits_for_both(gpu, pkg):
    syn = pkg.synth
    both = gpu.Malloc(1024)
    lo, hi = gpu.wrap(both.Ptr, 4 * 512), gpu.wrap(both.Ptr + 4 * 512, 4 * 512)
    x = gpu.from_numpy(syn.activations("st", 256, bf16=False))
    wa = gpu.UploadMLXWeight(*syn.mlx_weight("st-a", 512, 256, 64), 256, 512, 64, True)
    wb = gpu.UploadMLXWeight(*syn.mlx_weight("st-b", 512, 256, 64), 256, 512, 64, True)
    wc = gpu.UploadMLXWeight(*syn.mlx_weight("st-c", 300, 1024, 64), 1024, 300, 64, True)
    out = gpu.Malloc(300)
    ops = [(x, [wa], [lo]), (x, [wb], [hi]), (both, [wc], [out])]
    want = run_separately(gpu, ops)[-1]
    out.Upload(np.zeros(300, dtype=np.float32))
    prog = gpu.MLXProgram(ops)
    for _ in range(2):
        prog.Run()
    gpu.Sync()
    assert np.array_equal(out.Download().view(np.uint32), want.view(np.uint32))
    assert prog.Status() == 0
    prog.Free()


def test_single_product_and_group_size_128(gpu, pkg):
    x0, ops = chain(gpu, pkg, [(2048, [300, 7])], gs=128)
    want = run_separately(gpu, ops)
    for o in ops[0][2]:
        o.Upload(np.zeros(o.n, dtype=np.float32))
    prog = gpu.MLXProgram(ops)
    prog.Run(); prog.Run()
    gpu.Sync()
    for o, w in zip(ops[0][2], want):
        assert np.array_equal(o.Download().view(np.uint32), w.view(np.uint32))
    prog.Free()


def test_malformed_lists_raise(gpu, pkg):
    syn = pkg.synth
    x0, ops = chain(gpu, pkg, [(1024, [64]), (64, [32])])
    with pytest.raises(gpu.GophError):
        gpu.MLXProgram([])
    with pytest.raises(gpu.GophError):
        gpu.MLXProgram([(x0, ops[0][1], [])])
    with pytest.raises(gpu.GophError):      # weights of one product must share x
        gpu.MLXProgram([(x0, [ops[0][1][0], ops[1][1][0]], [ops[0][2][0], ops[1][2][0]])])
    with pytest.raises(gpu.GophError):      # more than eight weights in one product
        gpu.MLXProgram([(x0, ops[0][1] * 9, ops[0][2] * 9)])
    gpu.SetOption("mlx_layout", 2)
    try:
        tiled = gpu.UploadMLXWeight(*syn.mlx_weight("prog-t", 256, 1024, 64), 1024, 256, 64, True)
    finally:
        gpu.SetOption("mlx_layout", 0)
    with pytest.raises(gpu.GophError):      # tensor-core layout
        gpu.MLXProgram([(x0, [tiled], [gpu.Malloc(256)])])
    odd = gpu.wrap(x0.Ptr + 4, 4 * 1020)
    with pytest.raises(gpu.GophError):      # x not 16-byte aligned
        gpu.MLXProgram([(odd, ops[0][1], ops[0][2])])
    ops[0][1][0].Free()
    with pytest.raises(gpu.GophError):
        gpu.MLXProgram(ops)


def test_list_with_operations_in_front_equals_single_launches(gpu, pkg):
    """o -> (add, norm) gate|up -> (SiLU, mul) down -> (add, norm) q|k|v as one list against
    goph_mlx_gemv / goph_mlx_gemv_pre launches, bit for bit (hidden vectors included)."""
    syn = pkg.synth
    hid, inter, qd = 512, 1024, 768
    g = syn.rng("list-pre")
    f = lambda n: gpu.from_numpy(g.standard_normal(n, dtype=np.float32))
    mk = lambda key, o, i: gpu.UploadMLXWeight(*syn.mlx_weight(("list-pre", key), o, i, 64), i, o, 64, True)
    w_o, w_gu, w_down, w_qkv = mk("o", hid, qd), mk("gu", 2 * inter, hid), mk("down", hid, inter), mk("qkv", qd, hid)
    attn, resid, n1, n2 = f(qd), f(hid), f(hid), f(hid)

    def buffers():
        gu = gpu.Malloc(2 * inter)
        return dict(proj=gpu.Malloc(hid), gu=gu, gate=gpu.wrap(gu.Ptr, 4 * inter), up=gpu.wrap(gu.Ptr + 4 * inter, 4 * inter),
                    proj2=gpu.Malloc(hid), h1=gpu.Malloc(hid), h2=gpu.Malloc(hid), qkv=gpu.Malloc(qd))

    A, B = buffers(), buffers()
    gpu.GemvMLX(A["proj"], attn, w_o)
    gpu.GemvMLXPre(A["gu"], w_gu, 1, resid, A["proj"], n1, A["h1"], 1e-6)
    gpu.GemvMLXPre(A["proj2"], w_down, 2, A["gate"], A["up"], None, None)
    gpu.GemvMLXPre(A["qkv"], w_qkv, 1, A["h1"], A["proj2"], n2, A["h2"], 1e-6)
    prog = gpu.MLXProgram([(attn, [w_o], [B["proj"]]), (resid, [w_gu], [B["gu"]]), (B["gate"], [w_down], [B["proj2"]]),
                           (B["h1"], [w_qkv], [B["qkv"]])],
                          [None, dict(op=1, b=B["proj"], w=n1, hidden=B["h1"], eps=1e-6), dict(op=2, b=B["up"]),
                           dict(op=1, b=B["proj2"], w=n2, hidden=B["h2"], eps=1e-6)])
    prog.Run(); prog.Run()
    gpu.Sync()
    for k in ("proj", "gu", "proj2", "h1", "h2", "qkv"):
        assert np.array_equal(A[k].Download().view(np.uint32), B[k].Download().view(np.uint32)), k
    assert prog.Status() == 0
    prog.Free()
    with pytest.raises(gpu.GophError):      # the hidden vector of operation 1 must not be one of its inputs
        gpu.MLXProgram([(resid, [w_gu], [B["gu"]])], [dict(op=1, b=B["proj"], w=n1, hidden=resid, eps=1e-6)])
    with pytest.raises(gpu.GophError):      # operation 2 needs its second operand
        gpu.MLXProgram([(B["gate"], [w_down], [B["proj2"]])], [dict(op=2)])
