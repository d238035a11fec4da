"""Host-side mirror of the reference's GPU operator API (backends/nvidia/runtime) over the
C ABI of libgoph_b200.so.

Function and type names are the reference's Go names so that callers and tests read the
same.  Differences, both deliberate: (1) errors are raised as GophError instead of being
returned, and (2) there is no CPU fallback — where the reference's DevBuf operators fall
back to the CPU implementation when a launch fails (runtime/mlx.go:322-349), these raise.
Importing this module never touches the GPU; the first call that needs the library loads
it and fails loudly if it has not been built.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgoph_b200.so")

GGUF_Q8_0 = 8   # loader/gguf/gguf.go:51
GGUF_Q4_K = 12  # loader/gguf/gguf.go:54
GGUF_Q5_K = 13  # loader/gguf/gguf.go:55
GGUF_Q6_K = 14  # loader/gguf/gguf.go:56

# Every symbol include/goph_b200.h declares.
EXPORTS = [
    "goph_init", "goph_init_current_context", "goph_set_option", "goph_kernel_status", "goph_kernel_status_clear", "goph_last_error", "goph_sm_count", "goph_malloc", "goph_free", "goph_upload",
    "goph_download", "goph_memset", "goph_sync",
    "goph_mlx_program_create", "goph_mlx_program_create_pre", "goph_mlx_program_run", "goph_mlx_program_status", "goph_mlx_program_free",
    "goph_gptq_upload", "goph_gptq_free", "goph_gptq_resident_bytes", "goph_gptq_uses_mlx_kernels", "goph_gptq_gemm",
    "goph_gptq_dequant",
    "goph_mlx_upload", "goph_mlx_upload_dev", "goph_mlx_free", "goph_mlx_resident_bytes",
    "goph_mlx_dequant", "goph_mlx_gemv", "goph_mlx_gemm", "goph_mlx_gemm_bf16", "goph_mlx_gemm_multi", "goph_mlx_gemv_noalloc", "goph_mlx_gemv_noalloc_status", "goph_launch_count",
    "goph_mlx_gemm_host",
    "goph_gguf_upload", "goph_gguf_free", "goph_gguf_resident_bytes", "goph_gguf_dequant",
    "goph_gguf_project", "goph_gguf_project_pair", "goph_gguf_project_host",
    "goph_gguf_gate_up_gelu", "goph_gguf_gate_up_gelu_by_work", "goph_gguf_project_scatter", "goph_gguf_scatter_by_work",
    "goph_fp8_upload", "goph_fp8_free", "goph_fp8_resident_bytes", "goph_fp8_dequant", "goph_fp8_gemm", "goph_fp8_gemm_bf16",
    "goph_fp8_gemm_host",
    "goph_moe_create", "goph_moe_set_router", "goph_moe_set_expert", "goph_moe_free", "goph_moe_forward",
    "goph_moe_forward_logits", "goph_moe_last_routing",
    "goph_add_rmsnorm", "goph_qk_norm_rope_append", "goph_attn_decode", "goph_attn_decode_fused", "goph_silu_mul", "goph_argmax_advance", "goph_mlx_embed", "goph_mlx_gemv_pre",
    "goph_shard_rows", "goph_gather_create", "goph_gather_export", "goph_gather_open_peer", "goph_gather_attach_local",
    "goph_gather_free", "goph_gather_status", "goph_gather_shard_buffer", "goph_gather_all",
    "goph_mlx_gemm_allgather", "goph_gguf_project_allgather", "goph_fp8_gemm_allgather", "goph_moe_forward_sharded",
]


class GophError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("goph error %d: %s" % (code, text))
        self.code = code


_lib = None
_device = 0


def lib():
    """The loaded C-ABI library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        path = os.environ.get("GOPH_B200_LIB") or LIB_PATH  # the tuning build of the same library, when asked for
        if not os.path.exists(path):
            raise GophError(-1, "libgoph_b200.so is not built (run __graft_entry__.build()); "
                                "there is no CPU or PyTorch fallback")
        L = C.CDLL(path)
        L.goph_last_error.restype = C.c_char_p
        for name in ("goph_mlx_resident_bytes", "goph_gguf_resident_bytes", "goph_fp8_resident_bytes", "goph_gptq_resident_bytes"):
            getattr(L, name).restype = C.c_uint64
            getattr(L, name).argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise GophError(rc, lib().goph_last_error().decode("utf-8", "replace"))


def _vp(a):
    return a.ctypes.data_as(C.c_void_p)


def _stream_ptr(stream):
    if stream is None:
        return C.c_void_p(0)
    if hasattr(stream, "cuda_stream"):
        return C.c_void_p(stream.cuda_stream)
    return C.c_void_p(int(stream))


def init(device=0):
    """nvidia.Init + EnsureContext (runtime/runtime.go:142-274)."""
    global _device
    _check(lib().goph_init(int(device)))
    _device = int(device)
    return True


def InitCurrentContext():
    """Binds the library to the driver context that is current on this thread (the reference creates its
    own with cuCtxCreate, runtime/runtime.go:247) instead of the device's primary context."""
    global _device
    d = C.c_int(-1)
    _check(lib().goph_init_current_context(C.byref(d)))
    _device = d.value
    return _device


def device():
    return _device


def SetOption(name, value):
    """Tuning switches (the reference's GO_PHERENCE_* environment switches, model/gpu_forward.go:24-47)."""
    _check(lib().goph_set_option(name.encode(), int(value)))


def KernelStatus():
    """0 unless a bounded device-side wait has given up (see goph_kernel_status)."""
    v = C.c_int(0)
    _check(lib().goph_kernel_status(_device, C.byref(v)))
    return v.value


def KernelStatusClear():
    _check(lib().goph_kernel_status_clear(_device))


def SMCount():
    return lib().goph_sm_count(_device)


def Sync():
    """nvidia.SyncErr (runtime/runtime.go:563)."""
    _check(lib().goph_sync(_device))


class Buffer:
    """nvidia.Buffer{Ptr, Size} (runtime/runtime.go:291-295): a device allocation, Size in bytes."""

    def __init__(self, ptr, size, dev, owned=True):
        self.Ptr, self.Size, self.device, self._owned = ptr, size, dev, owned

    @property
    def n(self):
        return self.Size // 4

    def Upload(self, data):
        data = np.ascontiguousarray(data, dtype=np.float32)
        self._up(data)

    def UploadBytes(self, data):
        self._up(np.ascontiguousarray(data, dtype=np.uint8))

    def UploadUint32(self, data):
        self._up(np.ascontiguousarray(data, dtype=np.uint32))

    def _up(self, arr):
        if arr.nbytes > self.Size:
            raise GophError(1, "upload of %d bytes into a %d-byte buffer" % (arr.nbytes, self.Size))
        _check(lib().goph_upload(self.device, C.c_void_p(self.Ptr), _vp(arr), C.c_uint64(arr.nbytes)))

    def Download(self, n=None, dtype=np.float32):
        n = self.Size // np.dtype(dtype).itemsize if n is None else n
        out = np.empty(n, dtype=dtype)
        if out.nbytes > self.Size:
            raise GophError(1, "download of %d bytes from a %d-byte buffer" % (out.nbytes, self.Size))
        _check(lib().goph_download(self.device, _vp(out), C.c_void_p(self.Ptr), C.c_uint64(out.nbytes)))
        return out

    def Zero(self):
        _check(lib().goph_memset(self.device, C.c_void_p(self.Ptr), 0, C.c_uint64(self.Size)))

    def Free(self):
        """Idempotent, like Buffer.Free (runtime/runtime.go:323-359)."""
        if self.Ptr and self._owned:
            _check(lib().goph_free(self.device, C.c_void_p(self.Ptr)))
        self.Ptr, self.Size = 0, 0


def MallocBytes(n):
    """nvidia.MallocBytes (runtime/q8.go:166-177)."""
    p = C.c_void_p(0)
    _check(lib().goph_malloc(_device, C.c_uint64(int(n)), C.byref(p)))
    return Buffer(p.value, int(n), _device)


def Malloc(n_float32):
    """nvidia.Malloc (runtime/runtime.go:297)."""
    return MallocBytes(int(n_float32) * 4)


def wrap(ptr, size_bytes):
    """A Buffer over memory owned by someone else (e.g. a torch tensor's data_ptr())."""
    return Buffer(int(ptr), int(size_bytes), _device, owned=False)


def from_numpy(arr):
    arr = np.ascontiguousarray(arr)
    b = MallocBytes(max(arr.nbytes, 4))
    if arr.nbytes:
        _check(lib().goph_upload(b.device, C.c_void_p(b.Ptr), _vp(arr), C.c_uint64(arr.nbytes)))
    return b


# ------------------------------------------------------------------------------- MLX
class GPUMLXWeight:
    """nvidia.GPUMLXWeight (runtime/mlx.go:21-32)."""

    def __init__(self, handle, in_dim, out_dim, gs):
        self._h = handle
        self.InDim, self.OutDim, self.GroupSz, self.Groups = in_dim, out_dim, gs, in_dim // gs

    def ResidentBytes(self):
        return lib().goph_mlx_resident_bytes(self._h) if self._h else 0

    def Free(self):
        if self._h:
            _check(lib().goph_mlx_free(self._h))
            self._h = None


def UploadMLXWeight(weight, scales, biases, inDim, outDim, groupSize, wantNative=False):
    """nvidia.UploadMLXWeight (runtime/mlx.go:59).  wantNative is accepted for signature
    compatibility; there is one device layout and one kernel family here."""
    weight = np.ascontiguousarray(weight, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    biases = np.ascontiguousarray(biases, dtype=np.float32)
    h = C.c_void_p(0)
    _check(lib().goph_mlx_upload(_device, _vp(weight), C.c_uint64(weight.size), _vp(scales), _vp(biases),
                                 C.c_uint64(min(scales.size, biases.size)), int(inDim), int(outDim),
                                 int(groupSize), C.byref(h)))
    return GPUMLXWeight(h, int(inDim), int(outDim), int(groupSize))


def UploadMLXWeightNative(weight, scales, biases, inDim, outDim, groupSize):
    """nvidia.UploadMLXWeightNative (runtime/mlx.go:189)."""
    return UploadMLXWeight(weight, scales, biases, inDim, outDim, groupSize, True)


def _mlx_handle(w):
    if not isinstance(w, GPUMLXWeight) or not w._h:
        raise GophError(1, "nil or freed GPUMLXWeight")
    return w._h


def DequantMLX(out, w, stream=None):
    """mlx.DequantTo on the device (backends/mlx/dequant.go:30-42)."""
    _check(lib().goph_mlx_dequant(_mlx_handle(w), C.c_void_p(out.Ptr), C.c_uint64(out.n), _stream_ptr(stream)))


def GemvMLX(out, x, w, stream=None):
    """nvidia.GemvMLX (runtime/mlx.go:287)."""
    if out is None or x is None:
        raise GophError(1, "nil buffer")
    _check(lib().goph_mlx_gemv(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.n),
                               _mlx_handle(w), _stream_ptr(stream)))


def GemvMLXNoAlloc(out, x, w, stream=None):
    """out = W·x through goph_mlx_gemv_noalloc: the same product as GemvMLX for callers that cannot
    allocate device memory at this point (committed memory budget, no allocator synchronisation
    allowed mid-step, stream already being captured).  Tiled weights only, in_dim <= 16384, batch 1;
    calls that may overlap on the GPU must be ordered by the caller (they share one scratch array)."""
    if out is None or x is None:
        raise GophError(1, "nil buffer")
    _check(lib().goph_mlx_gemv_noalloc(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.n),
                                       _mlx_handle(w), _stream_ptr(stream)))


def LaunchCount():
    """Compute kernels launched through the library by this process so far (goph_launch_count)."""
    v = C.c_uint64(0)
    _check(lib().goph_launch_count(C.byref(v)))
    return v.value


def GemvMLXNoAllocStatus():
    """Status word of the allocation-free entry point's kernels on this device (0 = every wait completed)."""
    v = C.c_int(0)
    _check(lib().goph_mlx_gemv_noalloc_status(_device, C.byref(v)))
    return v.value


GemvMLXDirect = GemvMLX  # nvidia.GemvMLXDirect (runtime/mlx.go:455): same kernel here.


def GemmMLX(out, input, w, B, stream=None):
    """nvidia.GemmMLX (runtime/mlx.go:395)."""
    if out is None or input is None:
        raise GophError(1, "nil buffer")
    _check(lib().goph_mlx_gemm(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(input.Ptr),
                               C.c_uint64(input.n), _mlx_handle(w), int(B), _stream_ptr(stream)))


def to_bf16_bits(a):
    """f32 array -> uint16 bf16 bit patterns (round to nearest even)."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def GemmMLXBF16(out, input, w, B, stream=None):
    """nvidia.GemmMLX (runtime/mlx.go:395) with the activations held as bf16: `input` is a Buffer of
    B * inDim bf16 bit patterns (2 bytes each)."""
    if out is None or input is None:
        raise GophError(1, "nil buffer")
    _check(lib().goph_mlx_gemm_bf16(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(input.Ptr),
                                    C.c_uint64(input.Size // 2), _mlx_handle(w), int(B), _stream_ptr(stream)))


def GemmMLXMulti(outs, x, weights, B=1, stream=None):
    """mlx.Gemv2To generalised (backends/mlx/gemv.go:32-60): several weights, one x, one launch."""
    n = len(weights)
    if n != len(outs) or n == 0:
        raise GophError(1, "outs/weights length mismatch")
    op = (C.c_void_p * n)(*[o.Ptr for o in outs])
    wp = (C.c_void_p * n)(*[_mlx_handle(w) for w in weights])
    _check(lib().goph_mlx_gemm_multi(n, op, wp, C.c_void_p(x.Ptr), C.c_uint64(x.n), int(B), _stream_ptr(stream)))


def GemmMLXHost(x, w, B=1):
    """Host-slice form (x and result are numpy arrays), as the reference's slice operators."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(B * w.OutDim, dtype=np.float32)
    _check(lib().goph_mlx_gemm_host(_vp(out), C.c_uint64(out.size), _vp(x), C.c_uint64(x.size), _mlx_handle(w), int(B)))
    return out


# ------------------------------------------------------------------------------ GGUF
class GPUGGUFMatrix:
    """nvidia.GPUGGUFMatrix (runtime/gguf_matrix.go:11-17); also stands for GPUQ4KMatrix and
    GPUQ8_0Matrix (runtime/q4k.go:39-47, q8.go:20-25)."""

    def __init__(self, handle, qtype, in_dim, out_dim):
        self._h, self.QType, self.InDim, self.OutDim = handle, qtype, in_dim, out_dim

    def ResidentBytes(self):
        return lib().goph_gguf_resident_bytes(self._h) if self._h else 0

    def ProjectBatchToBuffer(self, out, x, batch, stream=None):
        """GPUGGUFMatrix.ProjectBatchToBuffer (runtime/gguf_matrix.go:121-135)."""
        if not self._h:
            raise GophError(1, "nil or freed GPUGGUFMatrix")
        if out is None or x is None:
            raise GophError(1, "nil buffer")
        _check(lib().goph_gguf_project(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr),
                                       C.c_uint64(x.n), int(batch), self._h, _stream_ptr(stream)))

    def Dequant(self, out, stream=None):
        if not self._h:
            raise GophError(1, "nil or freed GPUGGUFMatrix")
        _check(lib().goph_gguf_dequant(self._h, C.c_void_p(out.Ptr), C.c_uint64(out.n), _stream_ptr(stream)))

    def Free(self):
        if self._h:
            _check(lib().goph_gguf_free(self._h))
            self._h = None


def ProjectQ4PairToBuffers(outA, outB, x, batch, a, b, stream=None):
    """nvidia.ProjectQ4PairToBuffers (runtime/gguf_matrix.go:82-111): gate and up on one x."""
    if outA is None or outB is None or x is None or a is None or b is None:
        raise GophError(1, "nil buffer or matrix")
    _check(lib().goph_gguf_project_pair(C.c_void_p(outA.Ptr), C.c_uint64(outA.n), C.c_void_p(outB.Ptr), C.c_uint64(outB.n),
                                        C.c_void_p(x.Ptr), C.c_uint64(x.n), int(batch), a._h, b._h, _stream_ptr(stream)))


def _upload_gguf(qtype, raw, inDim, outDim):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    h = C.c_void_p(0)
    _check(lib().goph_gguf_upload(_device, int(qtype), _vp(raw), C.c_uint64(raw.size), int(inDim), int(outDim),
                                  C.byref(h)))
    return GPUGGUFMatrix(h, int(qtype), int(inDim), int(outDim))


def UploadGGUFMatrix(qtype, raw, inDim, outDim):
    """nvidia.UploadGGUFMatrix (runtime/gguf_matrix.go:19-39) for a QuantMatrix{QType, Raw, InDim, OutDim}."""
    return _upload_gguf(qtype, raw, inDim, outDim)


def UploadQ4KMatrixRaw(raw, inDim, outDim):
    """nvidia.UploadQ4KMatrixRaw / UploadQ4KMatrixRows (runtime/q4k.go:163-172)."""
    return _upload_gguf(GGUF_Q4_K, raw, inDim, outDim)


UploadQ4KMatrixRows = UploadQ4KMatrixRaw


def UploadQ8_0MatrixRows(raw, inDim, outDim):
    """nvidia.UploadQ8_0MatrixRows (runtime/q8.go:109)."""
    return _upload_gguf(GGUF_Q8_0, raw, inDim, outDim)


def _gguf_host(x, batch, m):
    if not isinstance(m, GPUGGUFMatrix) or not m._h:
        raise GophError(1, "nil or freed GPUGGUFMatrix")
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(batch * m.OutDim, dtype=np.float32)
    _check(lib().goph_gguf_project_host(_vp(out), C.c_uint64(out.size), _vp(x), C.c_uint64(x.size), int(batch), m._h))
    return out


def GemvQ4K(x, m):
    """nvidia.GemvQ4K (runtime/q4k.go:571) with host slices; returns out."""
    return _gguf_host(x, 1, m)


def GemvQ4KBatch(x, batch, m):
    """nvidia.GemvQ4KBatch (runtime/q4k.go:533)."""
    return _gguf_host(x, batch, m)


GemvQ8_0 = GemvQ4K            # nvidia.GemvQ8_0 (runtime/q8.go:277)
GemvQ8_0Batch = GemvQ4KBatch  # nvidia.GemvQ8_0Batch (runtime/q8.go:239)


def GemvQ4KBatchToBuffer(out, x, batch, m, stream=None):
    """nvidia.GemvQ4KBatchToBuffer (runtime/q4k.go:351)."""
    m.ProjectBatchToBuffer(out, x, batch, stream)


GemvQ8_0BatchToBuffer = GemvQ4KBatchToBuffer  # runtime/q8.go:225


def UploadQ5KMatrixRows(raw, inDim, outDim):
    """nvidia.UploadQ5KMatrixRows (runtime/qk.go:51): 176-byte super-blocks of 256 elements."""
    return _upload_gguf(GGUF_Q5_K, raw, inDim, outDim)


def UploadQ6KMatrixRows(raw, inDim, outDim):
    """nvidia.UploadQ6KMatrixRows (runtime/qk.go:55): 210-byte super-blocks of 256 elements."""
    return _upload_gguf(GGUF_Q6_K, raw, inDim, outDim)


def _want_qtype(m, qtype, name):
    if not isinstance(m, GPUGGUFMatrix) or not m._h or m.QType != qtype:
        raise GophError(1, "invalid %s matrix" % name)


def GateUpGELUQ4KBatchToBuffer(out, x, batch, intermediate, m, stream=None):
    """nvidia.GateUpGELUQ4KBatchToBuffer (runtime/q4k.go:338-352)."""
    _check(lib().goph_gguf_gate_up_gelu(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.n), int(batch),
                                        int(intermediate), m._h, _stream_ptr(stream)))


def GateUpGELUQ4KByWorkToBuffer(out, x, workExperts, workLen, intermediate, activeExperts, m, stream=None):
    """nvidia.GateUpGELUQ4KByWorkToBuffer (runtime/q4k.go:322-336); workExperts: device buffer of uint32."""
    _check(lib().goph_gguf_gate_up_gelu_by_work(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.n),
                                                C.c_void_p(workExperts.Ptr), int(workLen), int(intermediate),
                                                int(activeExperts), m._h, _stream_ptr(stream)))


def GemvQ8_0BatchScatter(dst, x, pos, weight, batch, m, stream=None):
    """nvidia.GemvQ8_0BatchScatter (runtime/q8.go:209-222); pos: device buffer of uint32, weight: of float32."""
    _check(lib().goph_gguf_project_scatter(C.c_void_p(dst.Ptr), C.c_uint64(dst.n), C.c_void_p(x.Ptr), C.c_uint64(x.n),
                                           C.c_void_p(pos.Ptr), C.c_void_p(weight.Ptr), int(batch), m._h, _stream_ptr(stream)))


def GemvQ8_0ScatterByWork(dst, x, workActive, workPos, workWeight, workLen, activeExperts, m, stream=None):
    """nvidia.GemvQ8_0ScatterByWork (runtime/q8.go:193-207)."""
    _check(lib().goph_gguf_scatter_by_work(C.c_void_p(dst.Ptr), C.c_uint64(dst.n), C.c_void_p(x.Ptr), C.c_uint64(x.n),
                                           C.c_void_p(workActive.Ptr), C.c_void_p(workPos.Ptr), C.c_void_p(workWeight.Ptr),
                                           int(workLen), int(activeExperts), m._h, _stream_ptr(stream)))


def GemvQ5KBatch(x, batch, m):
    """nvidia.GemvQ5KBatch (runtime/qk.go:392) with host slices; returns out."""
    _want_qtype(m, GGUF_Q5_K, "Q5_K")
    return _gguf_host(x, batch, m)


def GemvQ6KBatch(x, batch, m):
    """nvidia.GemvQ6KBatch (runtime/qk.go:396) with host slices; returns out."""
    _want_qtype(m, GGUF_Q6_K, "Q6_K")
    return _gguf_host(x, batch, m)


def GemvQ5KBatchToBuffer(out, x, batch, m, stream=None):
    """nvidia.GemvQ5KBatchToBuffer (runtime/qk.go:229)."""
    _want_qtype(m, GGUF_Q5_K, "Q5_K")
    m.ProjectBatchToBuffer(out, x, batch, stream)


def GemvQ6KBatchToBuffer(out, x, batch, m, stream=None):
    """nvidia.GemvQ6KBatchToBuffer (runtime/qk.go:285)."""
    _want_qtype(m, GGUF_Q6_K, "Q6_K")
    m.ProjectBatchToBuffer(out, x, batch, stream)


class MLXProgram:
    """A list of batch-1 MLX products run as one cooperative launch (goph_mlx_program_*).
    ops: [(x Buffer, [weights], [out Buffers])]; product k+1 may read what product k wrote.
    pre: optional list, one entry per product: None, or a dict with "op" (1: residual add + RMSNorm,
    2: SiLU(x) * b) and the operands "b", "w", "hidden" (Buffers or None) and "eps"."""

    def __init__(self, ops, pre=None):
        ws, outs, xs, counts = [], [], [], []
        for x, hs, os_ in ops:
            if len(hs) != len(os_) or not hs:
                raise GophError(1, "product needs as many outputs as weights")
            counts.append(len(hs)); xs.append(x.Ptr)
            ws += [_mlx_handle(h) for h in hs]; outs += [o.Ptr for o in os_]
        self._keep = (ops, pre)
        self.n = len(ops)
        h = C.c_void_p(0)
        n = len(ops)
        if pre is not None and len(pre) != n:
            raise GophError(1, "one pre entry per product")
        ptr = lambda b: b.Ptr if b is not None else None
        pick = lambda key: (C.c_void_p * n)(*[ptr(p.get(key)) if p else None for p in pre]) if pre is not None and n else None
        pre_ops = (C.c_int * n)(*[int(p["op"]) if p else 0 for p in pre]) if pre is not None and n else None
        pre_eps = (C.c_float * n)(*[float(p.get("eps", 0.0)) if p else 0.0 for p in pre]) if pre is not None and n else None
        _check(lib().goph_mlx_program_create_pre(_device, n, (C.c_int * len(counts))(*counts), (C.c_void_p * len(ws))(*ws),
                                                 (C.c_void_p * len(outs))(*outs), (C.c_void_p * len(xs))(*xs), pre_ops,
                                                 pick("b"), pick("w"), pick("hidden"), pre_eps, C.byref(h)))
        self._h = h

    def Run(self, stream=None):
        if not self._h:
            raise GophError(1, "freed product list")
        _check(lib().goph_mlx_program_run(self._h, _stream_ptr(stream)))

    def Status(self):
        st = C.c_int(0)
        _check(lib().goph_mlx_program_status(self._h, C.byref(st)))
        return st.value

    def Free(self):
        if self._h:
            _check(lib().goph_mlx_program_free(self._h))
            self._h = None


# ------------------------------------------------------------------------------- GPTQ
class GPUQuantWeight:
    """nvidia.GPUQuantWeight (runtime/q4.go:18-26)."""

    def __init__(self, handle, in_dim, out_dim, groups):
        self._h, self.InDim, self.OutDim, self.Groups = handle, in_dim, out_dim, groups

    def ResidentBytes(self):
        return int(lib().goph_gptq_resident_bytes(self._h)) if self._h else 0

    def UsesMLXKernels(self):
        return bool(lib().goph_gptq_uses_mlx_kernels(self._h)) if self._h else False

    def Dequant(self, out, stream=None):
        if not self._h:
            raise GophError(1, "nil or freed GPUQuantWeight")
        _check(lib().goph_gptq_dequant(self._h, C.c_void_p(out.Ptr), C.c_uint64(out.n), _stream_ptr(stream)))

    def Free(self):
        if self._h:
            _check(lib().goph_gptq_free(self._h))
            self._h = None


def UploadQuantWeight(qweight, gIdx, scales, inDim, outDim):
    """nvidia.UploadQuantWeight (runtime/q4.go:29-102)."""
    qweight = np.ascontiguousarray(qweight, dtype=np.int32)
    gIdx = np.ascontiguousarray(gIdx, dtype=np.int32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    h = C.c_void_p(0)
    _check(lib().goph_gptq_upload(_device, _vp(qweight), C.c_uint64(qweight.size), _vp(gIdx), C.c_uint64(gIdx.size),
                                  _vp(scales), C.c_uint64(scales.size), int(inDim), int(outDim), C.byref(h)))
    return GPUQuantWeight(h, int(inDim), int(outDim), scales.size // int(outDim))


def GemmQ4(out, x, w, B, stream=None):
    """nvidia.GemmQ4 (runtime/gemm_q4.go:24) on device buffers; raises where the reference would fall back to the CPU."""
    if not isinstance(w, GPUQuantWeight) or not w._h:
        raise GophError(1, "nil or freed GPUQuantWeight")
    _check(lib().goph_gptq_gemm(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.n), int(B), w._h,
                                _stream_ptr(stream)))


def GemvQ4(out, x, w, stream=None):
    """nvidia.GemvQ4 (runtime/q4.go:149)."""
    GemmQ4(out, x, w, 1, stream)


GemvQ4OrGemm = GemmQ4  # nvidia.GemvQ4OrGemm (runtime/gemm_q4.go:113): one entry point serves every batch


# ------------------------------------------------------------------------------- FP8
class GPUFP8E4M3Linear:
    """nvidia.GPUFP8E4M3Linear (runtime/fp8.go:35-44)."""

    def __init__(self, handle, out_dim, in_dim):
        self._h, self.OutDim, self.InDim = handle, out_dim, in_dim

    def ResidentBytes(self):
        return lib().goph_fp8_resident_bytes(self._h) if self._h else 0

    def Free(self):
        if self._h:
            _check(lib().goph_fp8_free(self._h))
            self._h = None


def UploadFP8E4M3Linear(weight, scale, bias, outDim, inDim):
    """nvidia.UploadFP8E4M3Linear (runtime/fp8.go:48)."""
    weight = np.ascontiguousarray(weight, dtype=np.uint8)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    bias_p, bias_n = C.c_void_p(0), 0
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        bias_p, bias_n = _vp(bias), bias.size
    h = C.c_void_p(0)
    _check(lib().goph_fp8_upload(_device, _vp(weight), C.c_uint64(weight.size), _vp(scale), int(scale.size),
                                 bias_p, int(bias_n), int(outDim), int(inDim), C.byref(h)))
    return GPUFP8E4M3Linear(h, int(outDim), int(inDim))


def _fp8_handle(w):
    if not isinstance(w, GPUFP8E4M3Linear) or not w._h:
        raise GophError(1, "nil or freed GPUFP8E4M3Linear")
    return w._h


def GemmFP8E4M3Buffer(out, x, batch, w, stream=None):
    """nvidia.GemmFP8E4M3Buffer (runtime/fp8.go:271)."""
    if out is None or x is None:
        raise GophError(1, "nil buffer")
    _check(lib().goph_fp8_gemm(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.n),
                               int(batch), _fp8_handle(w), _stream_ptr(stream)))


def GemmFP8E4M3BF16Buffer(out, x, batch, w, stream=None):
    """nvidia.GemmFP8E4M3Buffer (runtime/fp8.go:271) with the activations held as bf16: `x` is a Buffer
    of batch * inDim bf16 bit patterns."""
    if out is None or x is None:
        raise GophError(1, "nil buffer")
    _check(lib().goph_fp8_gemm_bf16(C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr), C.c_uint64(x.Size // 2),
                                    int(batch), _fp8_handle(w), _stream_ptr(stream)))


def GemvFP8E4M3Buffer(out, x, w, stream=None):
    """nvidia.GemvFP8E4M3Buffer (runtime/fp8.go:995)."""
    GemmFP8E4M3Buffer(out, x, 1, w, stream)


def GemmFP8E4M3(x, batch, w):
    """nvidia.GemmFP8E4M3 (runtime/fp8.go:180) with host slices; returns out."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(batch * w.OutDim, dtype=np.float32)
    _check(lib().goph_fp8_gemm_host(_vp(out), C.c_uint64(out.size), _vp(x), C.c_uint64(x.size), int(batch), _fp8_handle(w)))
    return out


def GemvFP8E4M3(x, w):
    """nvidia.GemvFP8E4M3 (runtime/fp8.go:158)."""
    return GemmFP8E4M3(x, 1, w)


def DequantFP8E4M3(out, w, stream=None):
    """fp8.Linear.DequantRowTo for every row (backends/simd/quant/fp8/fp8.go:181-198)."""
    _check(lib().goph_fp8_dequant(_fp8_handle(w), C.c_void_p(out.Ptr), C.c_uint64(out.n), _stream_ptr(stream)))


# ------------------------------------------------------------------------------ MoE
class GPUMoELayer:
    """The MoE state of one layer as model.moeForwardGPU uses it (model/moe_gpu.go:49-130):
    router weight, per-expert gate/up/down GPUMLXWeight, routing constants.  Experts left unset
    are not resident on this GPU and contribute nothing (per-GPU expert placement)."""

    def __init__(self, numExperts, hidden, inter, groupSize=64, topK=8, normTopK=True, maxTokens=32):
        h = C.c_void_p(0)
        _check(lib().goph_moe_create(_device, int(numExperts), int(hidden), int(inter), int(groupSize), int(topK),
                                     int(bool(normTopK)), int(maxTokens), C.byref(h)))
        self._h = h
        self.NumExperts, self.Hidden, self.Inter = int(numExperts), int(hidden), int(inter)
        self.TopK = min(int(topK) if topK > 0 else 8, int(numExperts))
        self._keep = {}

    def _handle(self):
        if not self._h:
            raise GophError(1, "nil or freed GPUMoELayer")
        return self._h

    def SetRouter(self, w):
        _check(lib().goph_moe_set_router(self._handle(), _mlx_handle(w)))
        self._keep["router"] = w

    def SetExpert(self, eid, gate, up, down):
        if gate is None and up is None and down is None:
            _check(lib().goph_moe_set_expert(self._handle(), int(eid), None, None, None))
            self._keep.pop(eid, None)
            return
        _check(lib().goph_moe_set_expert(self._handle(), int(eid), _mlx_handle(gate), _mlx_handle(up), _mlx_handle(down)))
        self._keep[eid] = (gate, up, down)

    def Forward(self, out, x, tokens=1, stream=None):
        """moeForwardGPU for `tokens` rows of x (model/moe_gpu.go:49)."""
        _check(lib().goph_moe_forward(self._handle(), C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr),
                                      C.c_uint64(x.n), int(tokens), _stream_ptr(stream)))

    def ForwardLogits(self, out, x, logits, tokens=1, stream=None):
        """The selected-expert projection with router logits supplied by the caller."""
        _check(lib().goph_moe_forward_logits(self._handle(), C.c_void_p(out.Ptr), C.c_uint64(out.n), C.c_void_p(x.Ptr),
                                             C.c_uint64(x.n), C.c_void_p(logits.Ptr), C.c_uint64(logits.n),
                                             int(tokens), _stream_ptr(stream)))

    def LastRouting(self, tokens=1):
        ids = np.empty(tokens * self.TopK, dtype=np.int32)
        wts = np.empty(tokens * self.TopK, dtype=np.float32)
        _check(lib().goph_moe_last_routing(self._handle(), int(tokens), _vp(ids), _vp(wts)))
        return ids.reshape(tokens, self.TopK), wts.reshape(tokens, self.TopK)

    def Free(self):
        if self._h:
            _check(lib().goph_moe_free(self._h))
            self._h = None
            self._keep = {}


# ------------------------------------------------------------------------------ row sharding
def ShardRows(outDim, rank, world, align=8):
    """Rows [lo, hi) of a projection owned by `rank` (goph_shard_rows)."""
    lo, hi = C.c_int(0), C.c_int(0)
    _check(lib().goph_shard_rows(int(outDim), int(rank), int(world), int(align), C.byref(lo), C.byref(hi)))
    return lo.value, hi.value


class Gather:
    """Exchange area of this rank for row-sharded outputs (no counterpart in the single-GPU reference)."""

    def __init__(self, rank, world, capacityFloats):
        h = C.c_void_p(0)
        _check(lib().goph_gather_create(_device, int(rank), int(world), C.c_uint64(int(capacityFloats)), C.byref(h)))
        self._h, self.rank, self.world, self.capacity, self.device = h, int(rank), int(world), int(capacityFloats), _device

    def Export(self):
        buf = (C.c_ubyte * 64)()
        _check(lib().goph_gather_export(self._h, buf))
        return bytes(buf)

    def OpenPeer(self, peerRank, handle):
        buf = (C.c_ubyte * 64)(*handle)
        _check(lib().goph_gather_open_peer(self._h, int(peerRank), buf))

    def AttachLocal(self, peer):
        _check(lib().goph_gather_attach_local(self._h, peer._h))

    def Connect(self, dist):
        """Exchanges the area tokens over an initialised torch.distributed group (host-side plumbing)."""
        handles = [None] * self.world
        dist.all_gather_object(handles, self.Export())
        for r, h in enumerate(handles):
            if r != self.rank:
                self.OpenPeer(r, h)
        dist.barrier()

    def Status(self):
        v = C.c_int(0)
        _check(lib().goph_gather_status(self._h, C.byref(v)))
        return v.value

    def ShardBuffer(self):
        p = C.c_void_p(0)
        _check(lib().goph_gather_shard_buffer(self._h, C.byref(p)))
        return Buffer(p.value, self.capacity * 4, self.device, owned=False)

    def _result(self, p, n):
        return Buffer(p.value, int(n) * 4, self.device, owned=False)

    def All(self, src, rows, per, total, rowStride, stream=None):
        """Every rank's block [rows x its width] side by side in every rank's result buffer."""
        p = C.c_void_p(0)
        _check(lib().goph_gather_all(self._h, C.c_void_p(src.Ptr if src is not None else 0), int(rows), int(per),
                                     C.c_int64(int(total)), C.c_int64(int(rowStride)), _stream_ptr(stream), C.byref(p)))
        return self._result(p, rows * rowStride)

    def GemmMLX(self, x, shard, B, rowLo, outDimFull, stream=None):
        """GemmMLX for a weight split by rows over the GPUs (shard None: this rank owns no rows);
        returns this rank's [B x outDimFull] buffer."""
        p = C.c_void_p(0)
        _check(lib().goph_mlx_gemm_allgather(self._h, _mlx_handle(shard) if shard is not None else None,
                                             C.c_void_p(x.Ptr), C.c_uint64(x.n), int(B),
                                             int(rowLo), int(outDimFull), _stream_ptr(stream), C.byref(p)))
        return self._result(p, B * outDimFull)

    def ProjectGGUF(self, x, shard, batch, rowLo, outDimFull, stream=None):
        p = C.c_void_p(0)
        _check(lib().goph_gguf_project_allgather(self._h, shard._h if shard is not None else None, C.c_void_p(x.Ptr),
                                                 C.c_uint64(x.n), int(batch),
                                                 int(rowLo), int(outDimFull), _stream_ptr(stream), C.byref(p)))
        return self._result(p, batch * outDimFull)

    def GemmFP8E4M3(self, x, shard, batch, rowLo, outDimFull, stream=None):
        p = C.c_void_p(0)
        _check(lib().goph_fp8_gemm_allgather(self._h, _fp8_handle(shard) if shard is not None else None,
                                             C.c_void_p(x.Ptr), C.c_uint64(x.n), int(batch),
                                             int(rowLo), int(outDimFull), _stream_ptr(stream), C.byref(p)))
        return self._result(p, batch * outDimFull)

    def MoEForward(self, layer, out, x, tokens, stream=None):
        _check(lib().goph_moe_forward_sharded(self._h, layer._handle(), C.c_void_p(out.Ptr), C.c_uint64(out.n),
                                              C.c_void_p(x.Ptr), C.c_uint64(x.n), int(tokens), int(layer.Hidden),
                                              _stream_ptr(stream)))

    def Free(self):
        if self._h:
            _check(lib().goph_gather_free(self._h))
            self._h = None


# ------------------------------------------------------------------------------ decode-step operations
def _ptr(b):
    return C.c_void_p(b.Ptr if b is not None else 0)


def AddRMSNorm(hidden, normed, a, b, weight, n, rows=1, eps=1e-6, stream=None):
    """hidden = a (+ b); normed = RMSNorm(hidden) * weight (simd.RMSNorm after the residual add)."""
    _check(lib().goph_add_rmsnorm(_device, _ptr(hidden), _ptr(normed), _ptr(a), _ptr(b), _ptr(weight), int(n), int(rows),
                                  C.c_float(eps), _stream_ptr(stream)))


def QKNormRoPEAppend(q, k, v, qNorm, kNorm, ropeTable, pos, kCache, vCache, maxSeq, heads, kvHeads, headDim, eps=1e-6, stream=None):
    _check(lib().goph_qk_norm_rope_append(_device, _ptr(q), _ptr(k), _ptr(v), _ptr(qNorm), _ptr(kNorm), _ptr(ropeTable),
                                          _ptr(pos), _ptr(kCache), _ptr(vCache), int(maxSeq), int(heads), int(kvHeads), int(headDim),
                                          C.c_float(eps), _stream_ptr(stream)))


def AttnDecode(out, q, kCache, vCache, pos, maxSeq, heads, kvHeads, headDim, scale, stream=None):
    _check(lib().goph_attn_decode(_device, _ptr(out), _ptr(q), _ptr(kCache), _ptr(vCache), _ptr(pos), int(maxSeq), int(heads),
                                  int(kvHeads), int(headDim), C.c_float(scale), _stream_ptr(stream)))


def SiLUMul(out, gate, up, n, stream=None):
    _check(lib().goph_silu_mul(_device, _ptr(out), _ptr(gate), _ptr(up), int(n), _stream_ptr(stream)))


def ArgmaxAdvance(logits, n, tok, pos, history, forced, historyCap, stream=None):
    _check(lib().goph_argmax_advance(_device, _ptr(logits), int(n), _ptr(tok), _ptr(pos), _ptr(history), _ptr(forced),
                                     int(historyCap), _stream_ptr(stream)))


def EmbedMLX(out, w, tok, stream=None):
    _check(lib().goph_mlx_embed(_ptr(out), C.c_uint64(out.n), _mlx_handle(w), _ptr(tok), _stream_ptr(stream)))


def GemvMLXPre(out, w, preOp, x, b, normW, hiddenOut, eps=1e-6, stream=None):
    """out = W . f(x): preOp 1 = RMSNorm(x (+ b)) * normW with hiddenOut = x (+ b); preOp 2 = silu(x) * b."""
    _check(lib().goph_mlx_gemv_pre(_ptr(out), C.c_uint64(out.n), _mlx_handle(w), int(preOp), _ptr(x), _ptr(b), _ptr(normW),
                                   _ptr(hiddenOut), C.c_float(eps), _stream_ptr(stream)))


def AttnDecodeFused(out, q, k, v, qNorm, kNorm, ropeTable, pos, kCache, vCache, maxSeq, heads, kvHeads, headDim, scale,
                    eps=1e-6, stream=None):
    """QKNormRoPEAppend + AttnDecode in one launch (q, k, v: raw projection outputs of the current position)."""
    _check(lib().goph_attn_decode_fused(_device, _ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(qNorm), _ptr(kNorm), _ptr(ropeTable),
                                        _ptr(pos), _ptr(kCache), _ptr(vCache), int(maxSeq), int(heads), int(kvHeads),
                                        int(headDim), C.c_float(scale), C.c_float(eps), _stream_ptr(stream)))
