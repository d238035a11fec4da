"""Writers of small safetensors and GGUF files for the checkpoint tests."""
import json
import struct

import numpy as np


def write_safetensors(path, tensors, metadata=None):
    """tensors: name -> (dtype string, shape, bytes)."""
    header, blobs, pos = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dtype, shape, data) in tensors.items():
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [pos, pos + len(data)]}
        blobs.append(data)
        pos += len(data)
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def _gguf_string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _gguf_value(v):
    if isinstance(v, bool):
        return 7, struct.pack("<B", int(v))
    if isinstance(v, str):
        return 8, _gguf_string(v)
    if isinstance(v, np.uint32):
        return 4, struct.pack("<I", int(v))
    if isinstance(v, np.uint64):
        return 10, struct.pack("<Q", int(v))
    if isinstance(v, np.float32):
        return 6, struct.pack("<f", float(v))
    if isinstance(v, list):
        parts = [_gguf_value(e) for e in v]
        return 9, struct.pack("<IQ", parts[0][0], len(parts)) + b"".join(p[1] for p in parts)
    raise TypeError(type(v))


def write_gguf(path, meta, tensors, version=3):
    """tensors: list of (name, shape innermost first, type id, bytes); data aligned to 32 bytes."""
    out = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta))
    for k, v in meta.items():
        t, payload = _gguf_value(v)
        out += _gguf_string(k) + struct.pack("<I", t) + payload
    pos, blobs = 0, []
    for name, shape, qtype, data in tensors:
        out += _gguf_string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", qtype, pos)
        pad = -len(data) % 32
        blobs.append(data + b"\0" * pad)
        pos += len(data) + pad
    out += b"\0" * (-len(out) % 32)
    with open(path, "wb") as f:
        f.write(out + b"".join(blobs))
