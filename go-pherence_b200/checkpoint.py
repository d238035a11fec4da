"""Checkpoint files -> device layouts: safetensors (MLX affine, GPTQ, FP8 tensors) and GGUF.

Host-side mirror of the reference's loaders for the quantized projections:
  safetensors.Open / File.GetRaw / GetFloat32 / GetInt32 / Names   (loader/safetensors/safetensors.go:113-178, :217-253, :280-352, :514-553)
  mlx.LoadWeight                                                     (backends/mlx/load.go:12-108)
  gguf.Open / GGUF.Raw / TensorByName / MatrixFromTensor / TensorRawBytes
                                                                     (loader/gguf/gguf.go:116-277, :295-350, :410-480; quant_matrix.go:27-39)
followed by the upload the reference does right after (nvidia.UploadMLXWeight, UploadGGUFMatrix,
UploadQuantWeight).  Files are memory-mapped; tensor bytes go from the mapping straight into the
upload call (one host copy into the staging buffer of the C library, none in Python).
Validation follows the reference: a malformed file is refused before anything reaches the GPU.
"""
import json
import mmap
import os
import struct

import numpy as np


class CheckpointError(ValueError):
    pass


_MAX_INT = 2 ** 63 - 1   # Go's int on the reference's 64-bit targets


# ------------------------------------------------------------------------------ safetensors
_ST_SIZES = {"F32": 4, "I32": 4, "U32": 4, "F16": 2, "BF16": 2, "I16": 2, "U16": 2, "I64": 8, "U64": 8,
             "I8": 1, "U8": 1, "BOOL": 1, "F8_E4M3": 1, "F8_E4M3FN": 1, "F8_E5M2": 1}


class SafetensorsFile:
    """safetensors.File: an 8-byte little-endian header length, a JSON header, then tensor bytes."""

    def __init__(self, path):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise CheckpointError("safetensors: file too short")
        self._fd = open(path, "rb")
        self._map = mmap.mmap(self._fd.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            (hlen,) = struct.unpack_from("<Q", self._map, 0)
            if hlen > size - 8:
                raise CheckpointError("safetensors: header length %d exceeds file size" % hlen)
            try:
                header = json.loads(bytes(self._map[8:8 + hlen]).decode("utf-8"))
            except (ValueError, UnicodeDecodeError) as e:
                raise CheckpointError("safetensors: parse header: %s" % e)
            if not isinstance(header, dict):
                raise CheckpointError("safetensors: parse header: not an object")
            self._base = 8 + hlen
            data_len = size - self._base
            self.Tensors = {}
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                try:
                    dtype, shape = str(info["dtype"]), [int(d) for d in info["shape"]]
                    start, end = (int(v) for v in info["data_offsets"])
                except (KeyError, TypeError, ValueError) as e:
                    raise CheckpointError("safetensors: parse tensor %r: %s" % (name, e))
                _validate_st(name, dtype, shape, start, end, data_len)
                self.Tensors[name] = (dtype, shape, start, end)
        except Exception:
            self.Close()
            raise

    def Close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass   # a caller still holds a view of the mapping; it stays valid until released
            self._map = None
        if self._fd is not None:
            self._fd.close()
            self._fd = None

    def Names(self):
        return sorted(self.Tensors)

    def GetRaw(self, name):
        """-> (uint8 view of the mapping, dtype string, shape)."""
        if self._map is None:
            raise CheckpointError("safetensors: file closed")
        if name not in self.Tensors:
            raise CheckpointError("safetensors: tensor %r not found" % name)
        dtype, shape, start, end = self.Tensors[name]
        return np.frombuffer(self._map, dtype=np.uint8, count=end - start, offset=self._base + start), dtype, list(shape)

    def GetFloat32(self, name):
        raw, dtype, shape = self.GetRaw(name)
        return _to_f32(raw, dtype, name), shape

    def GetInt32(self, name):
        raw, dtype, shape = self.GetRaw(name)
        if dtype not in ("I32", "U32"):
            raise CheckpointError("safetensors: tensor %r dtype %s is not I32" % (name, dtype))
        return raw.view("<i4"), shape


def _validate_st(name, dtype, shape, start, end, data_len):
    if start < 0 or end < start or end > data_len:
        raise CheckpointError("safetensors: tensor %r invalid data offsets [%d,%d] for data length %d" % (name, start, end, data_len))
    numel = 1
    for d in shape:
        if d < 0:
            raise CheckpointError("safetensors: tensor %r invalid shape %s" % (name, shape))
        numel *= d
    es = _ST_SIZES.get(dtype, 0)
    if es and numel * es != end - start:
        raise CheckpointError("safetensors: tensor %r shape %s dtype %s expects %d bytes, got %d" % (name, shape, dtype, numel * es, end - start))


def _to_f32(raw, dtype, name):
    if dtype == "F32":
        if raw.size % 4:
            raise CheckpointError("%s F32 raw byte length %d is not divisible by 4" % (name, raw.size))
        return raw.view("<f4")
    if dtype == "F16":
        if raw.size % 2:
            raise CheckpointError("%s F16 raw byte length %d is not divisible by 2" % (name, raw.size))
        return raw.view("<f2").astype(np.float32)
    if dtype == "BF16":
        if raw.size % 2:
            raise CheckpointError("%s BF16 raw byte length %d is not divisible by 2" % (name, raw.size))
        return (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
    raise CheckpointError("unsupported dtype %s for %s" % (dtype, name))


class QuantWeight:
    """mlx.QuantWeight (backends/mlx/quant.go): host arrays of one MLX affine projection."""

    def __init__(self, weight, scales, biases, out_dim, in_dim, group_size, bits):
        self.Weight, self.Scales, self.Biases = weight, scales, biases
        self.OutDim, self.InDim, self.GroupSize, self.Bits = out_dim, in_dim, group_size, bits
        self.Groups = in_dim // group_size


def LoadWeight(f, prefix, outDim, inDim, groupSize, bits):
    """mlx.LoadWeight: `<prefix>.weight` (U32/I32, [out, in*bits/32]), `.scales`, `.biases` (F32/F16/BF16,
    [out, in/groupSize]).  The file's shape wins over the caller's dims when it has one."""
    if bits <= 0 or bits > 32 or 32 % bits != 0:
        raise CheckpointError("invalid MLX bits=%d" % bits)
    if groupSize <= 0:
        raise CheckpointError("invalid MLX groupSize=%d" % groupSize)
    pack = 32 // bits
    try:
        raw, dtype, shape = f.GetRaw(prefix + ".weight")
    except CheckpointError as e:
        raise CheckpointError("load %s.weight: %s" % (prefix, e))
    if raw.size % 4:
        raise CheckpointError("MLX weight raw byte length %d is not divisible by 4" % raw.size)
    if len(shape) == 2:
        so, sp = shape
        if so <= 0 or sp <= 0:
            raise CheckpointError("MLX weight invalid shape %s" % shape)
        if sp * pack > _MAX_INT:
            raise CheckpointError("MLX weight shape %s overflows inDim with packFactor=%d" % (shape, pack))
        if (sp * pack) % groupSize:
            raise CheckpointError("MLX weight shape %s implies inDim=%d not divisible by groupSize=%d" % (shape, sp * pack, groupSize))
        outDim, inDim = so, sp * pack
    elif len(shape) != 0:
        raise CheckpointError("MLX weight shape rank %d unsupported for %s.weight" % (len(shape), prefix))
    if inDim <= 0 or outDim <= 0:
        raise CheckpointError("invalid MLX dims outDim=%d inDim=%d" % (outDim, inDim))
    if inDim % pack:
        raise CheckpointError("MLX inDim=%d is not divisible by packFactor=%d" % (inDim, pack))
    if inDim % groupSize:
        raise CheckpointError("MLX inDim=%d is not divisible by groupSize=%d" % (inDim, groupSize))
    if dtype not in ("U32", "I32"):
        raise CheckpointError("MLX weight dtype %s not supported (expected U32/I32)" % dtype)
    weight = raw.view("<u4")
    want = outDim * (inDim // pack)
    if weight.size != want:
        raise CheckpointError("MLX weight shape mismatch: got %d, expected %d (%dx%d)" % (weight.size, want, outDim, inDim // pack))
    want_s = outDim * (inDim // groupSize)
    tables = []
    for suffix in (".scales", ".biases"):
        name = prefix + suffix
        try:
            r, dt, sh = f.GetRaw(name)
        except CheckpointError as e:
            raise CheckpointError("load %s: %s" % (name, e))
        t = _to_f32(r, dt, name)
        if sh:
            n = 1
            for d in sh:
                if d <= 0:
                    raise CheckpointError("%s invalid shape %s" % (name, sh))
                n *= d
                if n > _MAX_INT:
                    raise CheckpointError("%s shape %s element count overflows" % (name, sh))
            if n != t.size:
                raise CheckpointError("%s shape %s has %d elements, raw data has %d" % (name, sh, n, t.size))
        if t.size != want_s:
            raise CheckpointError("%s length mismatch: got %d, expected %d" % (name, t.size, want_s))
        tables.append(t)
    return QuantWeight(weight, tables[0], tables[1], outDim, inDim, groupSize, bits)


def UploadMLXFromSafetensors(rt, f, prefix, outDim=0, inDim=0, groupSize=64, bits=4):
    """LoadWeight then nvidia.UploadMLXWeight (runtime/mlx.go:57).  4-bit only, as the GPU path of the reference."""
    qw = LoadWeight(f, prefix, outDim, inDim, groupSize, bits)
    if qw.Bits != 4:
        raise CheckpointError("MLX bits=%d has no GPU layout (4-bit only)" % qw.Bits)
    return rt.UploadMLXWeight(qw.Weight, qw.Scales, qw.Biases, qw.InDim, qw.OutDim, qw.GroupSize, True)


def UploadGPTQFromSafetensors(rt, f, prefix):
    """`<prefix>.qweight` [in/8, out] I32, `.g_idx` [in] I32, `.scales` [groups, out] F16/F32 of a symmetric
    GPTQ checkpoint -> nvidia.UploadQuantWeight (runtime/q4.go:29)."""
    qweight, shape = f.GetInt32(prefix + ".qweight")
    if len(shape) != 2:
        raise CheckpointError("GPTQ qweight shape %s is not a matrix" % shape)
    gidx, _ = f.GetInt32(prefix + ".g_idx")
    scales, _ = f.GetFloat32(prefix + ".scales")
    return rt.UploadQuantWeight(qweight, gidx, scales, shape[0] * 8, shape[1])


def UploadFP8FromSafetensors(rt, f, prefix, scale_suffix=".weight_scale"):
    """`<prefix>.weight` [out, in] F8_E4M3, `<prefix><scale_suffix>` F32/BF16/F16 of length 1 or out, optional
    `<prefix>.bias` -> nvidia.UploadFP8E4M3Linear (runtime/fp8.go:48)."""
    raw, dtype, shape = f.GetRaw(prefix + ".weight")
    if dtype not in ("F8_E4M3", "F8_E4M3FN") or len(shape) != 2:
        raise CheckpointError("FP8 weight %s.weight dtype %s shape %s unsupported" % (prefix, dtype, shape))
    scale, _ = f.GetFloat32(prefix + scale_suffix)
    bias = f.GetFloat32(prefix + ".bias")[0] if prefix + ".bias" in f.Tensors else None
    return rt.UploadFP8E4M3Linear(raw, scale, bias, shape[0], shape[1])


# ------------------------------------------------------------------------------------ GGUF
# (elements, bytes) per block of each tensor type the reference sizes (loader/gguf/gguf.go:429-480)
_GGUF_BLOCKS = {0: (1, 4), 1: (1, 2), 30: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34),
                10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292)}
_MAX_STRING, _MAX_COUNT, _MAX_DIMS = 16 << 20, 1_000_000, 8
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


def TensorRawBytes(qtype, n):
    """gguf.TensorRawBytes: bytes of n elements of a tensor type; n must fill whole blocks."""
    if n < 0:
        raise CheckpointError("negative element count %d" % n)
    if qtype not in _GGUF_BLOCKS:
        raise CheckpointError("unsupported quant type %d" % qtype)
    if n == 0:
        return 0
    be, bb = _GGUF_BLOCKS[qtype]
    if n % be:
        raise CheckpointError("quant type %d: %d elements do not fill blocks of %d" % (qtype, n, be))
    return n // be * bb


class TensorInfo:
    def __init__(self, name, shape, qtype, offset):
        self.Name, self.Shape, self.QType, self.Offset = name, shape, qtype, offset   # Shape: innermost dimension first


class QuantMatrix:
    """gguf.QuantMatrix (loader/gguf/quant_matrix.go:13-24): rows of InDim elements, OutDim rows, raw blocks."""

    def __init__(self, name, qtype, raw, in_dim, out_dim):
        self.Name, self.QType, self.Raw, self.InDim, self.OutDim = name, qtype, raw, in_dim, out_dim

    def RowBytes(self):
        return TensorRawBytes(self.QType, self.InDim)


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos, self.size = buf, 0, len(buf)

    def take(self, fmt):
        n = struct.calcsize(fmt)
        if self.pos + n > self.size:
            raise CheckpointError("unexpected end of file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += n
        return v

    def string(self):
        n = self.take("<Q")
        if n > _MAX_STRING:
            raise CheckpointError("string length %d exceeds limit %d" % (n, _MAX_STRING))
        if n > self.size - self.pos:
            raise CheckpointError("unexpected end of file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, t, depth=0):
        if t in _SCALARS:
            v = self.take(_SCALARS[t])
            return bool(v) if t == 7 else v
        if t == 8:
            return self.string()
        if t == 9:
            if depth >= 1:
                raise CheckpointError("nested arrays exceed depth limit 1")
            et = self.take("<I")
            if et == 9:
                raise CheckpointError("nested arrays are unsupported")
            count = self.take("<Q")
            if count > _MAX_COUNT:
                raise CheckpointError("array count %d exceeds limit %d" % (count, _MAX_COUNT))
            return [self.value(et, depth + 1) for _ in range(count)]
        raise CheckpointError("unknown GGUFType %d" % t)


class GGUFFile:
    """gguf.GGUF: header, metadata and tensor index of a version 2 or 3 file; tensor data starts at the
    next multiple of 32 bytes after the index."""

    def __init__(self, path):
        self.path = path
        self._fd = open(path, "rb")
        size = os.path.getsize(path)
        self._map = mmap.mmap(self._fd.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        try:
            r = _Reader(self._map if self._map is not None else b"")
            try:
                magic = bytes(r.buf[0:4])
                r.pos = 4
                if len(magic) < 4:
                    raise CheckpointError("gguf: read magic: unexpected end of file")
                if magic != b"GGUF":
                    raise CheckpointError("gguf: bad magic %r" % magic)
                version = r.take("<I")
                if version not in (2, 3):
                    raise CheckpointError("gguf: unsupported version %d" % version)
                n_tensors, n_kv = r.take("<Q"), r.take("<Q")
                if n_tensors > _MAX_COUNT:
                    raise CheckpointError("gguf: tensor count %d exceeds limit %d" % (n_tensors, _MAX_COUNT))
                if n_kv > _MAX_COUNT:
                    raise CheckpointError("gguf: metadata count %d exceeds limit %d" % (n_kv, _MAX_COUNT))
                self.Meta = {}
                for i in range(n_kv):
                    key = r.string()
                    if key in self.Meta:
                        raise CheckpointError("gguf: duplicate metadata key %r" % key)
                    self.Meta[key] = r.value(r.take("<I"))
                self.Tensors = []
                for i in range(n_tensors):
                    name = r.string()
                    nd = r.take("<I")
                    if nd == 0 or nd > _MAX_DIMS:
                        raise CheckpointError("gguf: tensor[%d] %r rank %d exceeds limit %d" % (i, name, nd, _MAX_DIMS))
                    shape = [r.take("<Q") for _ in range(nd)]
                    qtype, offset = r.take("<I"), r.take("<Q")
                    self.Tensors.append(TensorInfo(name, shape, qtype, offset))
            except CheckpointError as e:
                raise CheckpointError(str(e) if str(e).startswith("gguf:") else "gguf: %s" % e)
            self.DataOffset = (r.pos + 31) // 32 * 32
            if self.DataOffset > size:
                raise CheckpointError("gguf: data offset %d exceeds file size %d" % (self.DataOffset, size))
            self._size = size
            for i, t in enumerate(self.Tensors):
                start, end = self._span(t)
                if end > size:
                    raise CheckpointError("gguf: tensor[%d] %r span [%d,%d) exceeds GGUF data length (file size %d)" % (i, t.Name, start, end, size))
        except Exception:
            self.Close()
            raise

    def _span(self, t):
        # rows are encoded one after another: every row of Shape[0] elements fills whole blocks
        rows = 1
        for d in t.Shape[1:]:
            rows *= d
        try:
            nbytes = TensorRawBytes(t.QType, t.Shape[0]) * rows
        except CheckpointError as e:
            raise CheckpointError("gguf: tensor %r: %s" % (t.Name, e))
        start = self.DataOffset + t.Offset
        return start, start + nbytes

    def Close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass
            self._map = None
        if self._fd is not None:
            self._fd.close()
            self._fd = None

    def TensorByName(self, name):
        for t in self.Tensors:
            if t.Name == name:
                return t
        return None

    def Raw(self, t):
        if self._map is None:
            raise CheckpointError("gguf: file closed")
        start, end = self._span(t)
        return np.frombuffer(self._map, dtype=np.uint8, count=end - start, offset=start)

    def MatrixFromTensor(self, t):
        if len(t.Shape) != 2:
            raise CheckpointError("gguf: tensor %r shape %s is not a matrix" % (t.Name, t.Shape))
        return QuantMatrix(t.Name, t.QType, self.Raw(t), int(t.Shape[0]), int(t.Shape[1]))

    def MetaUint32(self, key):
        v = self.Meta.get(key)
        return (int(v), True) if isinstance(v, int) and not isinstance(v, bool) and 0 <= v < 2 ** 32 else (0, False)

    def MetaString(self, key):
        v = self.Meta.get(key)
        return (v, True) if isinstance(v, str) else ("", False)


def UploadGGUFTensor(rt, g, name):
    """TensorByName + MatrixFromTensor + nvidia.UploadGGUFMatrix (runtime/gguf_matrix.go:19-39); Q8_0 goes
    through the same upload (nvidia.UploadQ8_0MatrixRows, runtime/q8.go:109)."""
    t = g.TensorByName(name)
    if t is None:
        raise CheckpointError("gguf: tensor %r not found" % name)
    m = g.MatrixFromTensor(t)
    return rt.UploadGGUFMatrix(m.QType, m.Raw, m.InDim, m.OutDim)
