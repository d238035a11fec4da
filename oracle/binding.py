"""ctypes/numpy front end of the CPU oracle (test infrastructure only).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
arm may import this module; the shipped package never does.
Function names follow the reference's Go functions they restate.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None

Q8_0 = 8   # loader/gguf/gguf.go:51
Q4_K = 12  # loader/gguf/gguf.go:54
Q5_K = 13  # loader/gguf/gguf.go:55
Q6_K = 14  # loader/gguf/gguf.go:56


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            path = _build.build()
        _lib = C.CDLL(path)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_e4m3_decode.restype = C.c_float
        _lib.orc_e4m3_decode.argtypes = [C.c_uint8]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def default_threads():
    return os.cpu_count() or 1


# --------------------------------------------------------------------- MLX
def mlx_validate(w_len, s_len, b_len, out_dim, in_dim, gs, groups, bits=4):
    return lib().orc_mlx_validate(C.c_long(w_len), C.c_long(s_len), C.c_long(b_len),
                                  out_dim, in_dim, gs, groups, bits) == 0


def mlx_dequant(w, scales, biases, out_dim, in_dim, gs, bits=4, nthreads=1, out=None):
    """mlx.DequantTo; returns None on malformed input (Go: false)."""
    w, scales, biases = _u32(w), _f32(scales), _f32(biases)
    if out is None:
        out = np.empty(max(out_dim * in_dim, 0), dtype=np.float32)
    rc = lib().orc_mlx_dequant(_p(out), C.c_long(out.size), _p(w), C.c_long(w.size), _p(scales),
                               _p(biases), C.c_long(min(scales.size, biases.size)), out_dim,
                               in_dim, gs, bits, nthreads)
    return out if rc == 0 else None


def mlx_gemv(x, w, scales, biases, out_dim, in_dim, gs, bits=4, nthreads=1, out=None):
    """mlx.GemvTo / GemvParallel; returns None on malformed input."""
    x, w, scales, biases = _f32(x), _u32(w), _f32(scales), _f32(biases)
    if out is None:
        out = np.empty(max(out_dim, 0), dtype=np.float32)
    rc = lib().orc_mlx_gemv(_p(out), C.c_long(out.size), _p(x), C.c_long(x.size), _p(w),
                            C.c_long(w.size), _p(scales), _p(biases),
                            C.c_long(min(scales.size, biases.size)), out_dim, in_dim, gs, bits,
                            nthreads)
    return out if rc == 0 else None


def mlx_gemm(x, batch, w, scales, biases, out_dim, in_dim, gs, bits=4, nthreads=1, out=None):
    """mlx.Gemm: x [batch,in] -> out [batch,out]; None on malformed input."""
    x, w, scales, biases = _f32(x), _u32(w), _f32(scales), _f32(biases)
    if out is None:
        out = np.empty(max(batch * out_dim, 0), dtype=np.float32)
    rc = lib().orc_mlx_gemm(_p(out), C.c_long(out.size), _p(x), C.c_long(x.size), batch, _p(w),
                            C.c_long(w.size), _p(scales), _p(biases),
                            C.c_long(min(scales.size, biases.size)), out_dim, in_dim, gs, bits,
                            nthreads)
    return out if rc == 0 else None


# -------------------------------------------------------------------- GGUF
def gguf_row_bytes(qtype, in_dim):
    return lib().orc_gguf_row_bytes(qtype, in_dim)


def gguf_dequant(raw, qtype, in_dim, out_dim, nthreads=1):
    raw = _u8(raw)
    out = np.empty(out_dim * in_dim, dtype=np.float32)
    rc = lib().orc_gguf_dequant(_p(out), C.c_long(out.size), _p(raw), C.c_long(raw.size), qtype,
                                in_dim, out_dim, nthreads)
    return out.reshape(out_dim, in_dim) if rc == 0 else None


def gguf_gemv(x, raw, qtype, in_dim, out_dim, batch=1, nthreads=1):
    """gemvGGUFQuantRowsPureGo per activation row: dequant row, sequential dot."""
    x, raw = _f32(x), _u8(raw)
    out = np.empty(batch * out_dim, dtype=np.float32)
    rc = lib().orc_gguf_gemv(_p(out), C.c_long(out.size), _p(x), C.c_long(x.size), batch,
                             _p(raw), C.c_long(raw.size), qtype, in_dim, out_dim, nthreads)
    return out if rc == 0 else None


# --------------------------------------------------------------------- GPTQ
def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def gptq_dequant_sym(qweight, gidx, scales, in_dim, out_dim):
    """q4.DequantSym (backends/simd/quant/q4/dequant.go:114-197): [out, in] row-major, or None when rejected."""
    qweight, gidx, scales = _i32(qweight), _i32(gidx), _f32(scales)
    out = np.empty(max(0, out_dim * in_dim), dtype=np.float32)
    rc = lib().orc_gptq_dequant_sym(_p(out), C.c_long(out.size), _p(qweight), C.c_long(qweight.size), _p(gidx),
                                    C.c_long(gidx.size), _p(scales), C.c_long(scales.size), in_dim, out_dim)
    return out.reshape(out_dim, in_dim) if rc == 0 else None


def gptq_gemm_sym(x, batch, qweight, gidx, scales, in_dim, out_dim):
    """q4.GemvSym / q4.GemmSym (gemv.go:76-94, gemm_sym_portable.go:7-150); None when rejected."""
    x, qweight, gidx, scales = _f32(x), _i32(qweight), _i32(gidx), _f32(scales)
    out = np.empty(max(0, batch * out_dim), dtype=np.float32)
    rc = lib().orc_gptq_gemm_sym(_p(out), C.c_long(out.size), _p(x), C.c_long(x.size), batch, _p(qweight),
                                 C.c_long(qweight.size), _p(gidx), C.c_long(gidx.size), _p(scales),
                                 C.c_long(scales.size), in_dim, out_dim)
    return out if rc == 0 else None


# --------------------------------------------------------------------- FP8
def e4m3_decode(code):
    return lib().orc_e4m3_decode(int(code) & 0xFF)


def e4m3_table():
    return np.array([e4m3_decode(i) for i in range(256)], dtype=np.float32)


def fp8_dequant(w, scale, out_dim, in_dim):
    w, scale = _u8(w), _f32(scale)
    out = np.empty(out_dim * in_dim, dtype=np.float32)
    rc = lib().orc_fp8_dequant(_p(out), _p(w), _p(scale), scale.size, out_dim, in_dim)
    return out.reshape(out_dim, in_dim) if rc == 0 else None


def fp8_gemv(x, w, scale, bias, out_dim, in_dim, avx2=True, nthreads=1):
    """fp8.Linear.GemvTo."""
    x, w, scale = _f32(x), _u8(w), _f32(scale)
    bias = None if bias is None else _f32(bias)
    out = np.empty(out_dim, dtype=np.float32)
    rc = lib().orc_fp8_gemv(_p(out), _p(x), _p(w), _p(scale), scale.size, _p(bias), out_dim,
                            in_dim, int(avx2), nthreads)
    return out if rc == 0 else None


def fp8_batch_gemv(x, batch, w, scale, bias, out_dim, in_dim, avx2=True, nthreads=1):
    """fp8.Linear.BatchGemvTo: x [batch,in] -> out [batch,out]."""
    x, w, scale = _f32(x), _u8(w), _f32(scale)
    bias = None if bias is None else _f32(bias)
    out = np.empty(batch * out_dim, dtype=np.float32)
    rc = lib().orc_fp8_batch_gemv(_p(out), _p(x), batch, _p(w), _p(scale), scale.size, _p(bias),
                                  out_dim, in_dim, int(avx2), nthreads)
    return out if rc == 0 else None


# --------------------------------------------------------------------- MoE
def softmax(x):
    x = _f32(x).copy()
    return x if lib().orc_softmax(_p(x), x.size) == 0 else None


def silu_mul(a, b):
    a, b = _f32(a), _f32(b)
    dst = np.empty_like(a)
    lib().orc_silu_mul(_p(dst), _p(a), _p(b), a.size)
    return dst


def moe_route(logits, top_k, norm_topk=True):
    logits = _f32(logits)
    ids = np.zeros(max(top_k, 1), dtype=np.int32)
    wts = np.zeros(max(top_k, 1), dtype=np.float32)
    n = lib().orc_moe_route(_p(logits), logits.size, top_k, int(norm_topk), _p(ids), _p(wts))
    return ids[:n].copy(), wts[:n].copy()


def moe_experts(x, hidden, inter, gs, gate, up, down, ids, weights):
    """gate/up/down are (w, scales, biases) with experts stacked on axis 0."""
    x = _f32(x)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = _f32(weights)
    out = np.empty(hidden, dtype=np.float32)
    gw, gsc, gb = _u32(gate[0]), _f32(gate[1]), _f32(gate[2])
    uw, usc, ub = _u32(up[0]), _f32(up[1]), _f32(up[2])
    dw, dsc, db = _u32(down[0]), _f32(down[1]), _f32(down[2])
    rc = lib().orc_moe_experts(_p(out), _p(x), hidden, inter, gs, _p(gw), _p(gsc), _p(gb),
                               _p(uw), _p(usc), _p(ub), _p(dw), _p(dsc), _p(db), _p(ids),
                               _p(weights), ids.size)
    return out if rc == 0 else None
