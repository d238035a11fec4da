"""Checkpoint files through the loaders onto the GPU: the product of the loaded weight equals the oracle's on the same bytes."""
import numpy as np
import pytest

from gpu_util import TOL
from helpers_checkpoint import write_gguf, write_safetensors
from oracle import binding as orc

pytestmark = pytest.mark.gpu


def product(gpu, project, x, out_dim):
    xo, out = gpu.from_numpy(x), gpu.Malloc(out_dim)
    project(out, xo)
    gpu.Sync()
    got = out.Download()
    xo.Free(); out.Free()
    return got


def test_safetensors_mlx_gptq_fp8(gpu, pkg, tmp_path):
    ck, syn = pkg.checkpoint, pkg.synth
    out_dim, in_dim = 512, 1024
    w, s, b = syn.mlx_weight("ck", out_dim, in_dim, 64)
    qw, gidx, sc = syn.gptq_weight("ck", out_dim, in_dim, 128, act_order=True)
    fw, fs, fb = syn.fp8_linear("ck", out_dim, in_dim, bias=True)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {
        "m.q_proj.weight": ("U32", [out_dim, in_dim // 8], w.tobytes()),
        "m.q_proj.scales": ("BF16", [out_dim, in_dim // 64], (s.view(np.uint32) >> 16).astype(np.uint16).tobytes()),
        "m.q_proj.biases": ("BF16", [out_dim, in_dim // 64], (b.view(np.uint32) >> 16).astype(np.uint16).tobytes()),
        "g.q_proj.qweight": ("I32", [in_dim // 8, out_dim], qw.tobytes()),
        "g.q_proj.g_idx": ("I32", [in_dim], gidx.tobytes()),
        "g.q_proj.scales": ("F16", [in_dim // 128, out_dim], sc.astype(np.float16).tobytes()),
        "f.q_proj.weight": ("F8_E4M3", [out_dim, in_dim], fw.tobytes()),
        "f.q_proj.weight_scale": ("F32", [out_dim], fs.tobytes()),
        "f.q_proj.bias": ("F32", [out_dim], fb.tobytes()),
    })
    f = ck.SafetensorsFile(path)
    x = syn.activations("ck-x", in_dim, bf16=False)
    m = ck.UploadMLXFromSafetensors(gpu, f, "m.q_proj")
    assert (m.OutDim, m.InDim) == (out_dim, in_dim)
    want = orc.mlx_gemv(x, w, s, b, out_dim, in_dim, 64)
    assert syn.rel_err(product(gpu, lambda o, xo: gpu.GemvMLX(o, xo, m), x, out_dim), want) <= TOL
    g = ck.UploadGPTQFromSafetensors(gpu, f, "g.q_proj")
    want = orc.gptq_gemm_sym(x, 1, qw, gidx, sc, in_dim, out_dim)
    assert syn.rel_err(product(gpu, lambda o, xo: gpu.GemvQ4(o, xo, g), x, out_dim), want) <= TOL
    l = ck.UploadFP8FromSafetensors(gpu, f, "f.q_proj")
    want = orc.fp8_gemv(x, fw, fs, fb, out_dim, in_dim)
    assert syn.rel_err(product(gpu, lambda o, xo: gpu.GemvFP8E4M3Buffer(o, xo, l), x, out_dim), want) <= TOL
    with pytest.raises(ck.CheckpointError):
        ck.UploadMLXFromSafetensors(gpu, f, "g.q_proj")
    for h in (m, g, l):
        h.Free()
    f.Close()


def test_gguf_tensors(gpu, pkg, tmp_path):
    ck, syn = pkg.checkpoint, pkg.synth
    out_dim, in_dim = 384, 1024
    gens = {8: syn.q8_0_matrix, 12: syn.q4k_matrix, 13: syn.q5k_matrix, 14: syn.q6k_matrix}
    raws = {qt: gen("ck", out_dim, in_dim) for qt, gen in gens.items()}
    path = str(tmp_path / "model.gguf")
    write_gguf(path, {"general.architecture": "llama"},
               [("blk.0.t%d.weight" % qt, [in_dim, out_dim], qt, raw.tobytes()) for qt, raw in raws.items()])
    g = ck.GGUFFile(path)
    x = syn.activations("ck-x", in_dim, bf16=False)
    for qt, raw in raws.items():
        m = ck.UploadGGUFTensor(gpu, g, "blk.0.t%d.weight" % qt)
        assert (m.QType, m.InDim, m.OutDim, m.ResidentBytes()) == (qt, in_dim, out_dim, raw.size)
        want = orc.gguf_gemv(x, raw, qt, in_dim, out_dim)
        assert syn.rel_err(product(gpu, lambda o, xo: m.ProjectBatchToBuffer(o, xo, 1), x, out_dim), want) <= TOL
        m.Free()
    with pytest.raises(ck.CheckpointError, match="not found"):
        ck.UploadGGUFTensor(gpu, g, "nope")
    g.Close()
