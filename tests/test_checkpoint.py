"""Checkpoint readers (safetensors, GGUF) and mlx.LoadWeight: CPU tests on files written here."""
import json
import struct

import numpy as np
import pytest

from helpers_checkpoint import write_gguf, write_safetensors


@pytest.fixture(scope="module")
def ck(pkg):
    return pkg.checkpoint


class FakeSource(dict):
    """The in-memory source of backends/mlx/loader_test.go:11-38."""

    def GetRaw(self, name):
        if name not in self:
            raise self.err("missing raw %s" % name)
        raw, dtype, shape = self[name]
        return np.frombuffer(raw, dtype=np.uint8), dtype, shape


def valid_source(ck):
    s = FakeSource()
    s.err = ck.CheckpointError
    s["proj.weight"] = (struct.pack("<2I", 0x76543210, 0xfedcba98), "U32", [2, 1])
    s["proj.scales"] = (struct.pack("<2f", 0.1, 0.2), "F32", [2, 1])
    s["proj.biases"] = (struct.pack("<2f", -0.1, -0.2), "F32", [2, 1])
    return s


def test_load_weight_reference_cases(ck):
    # backends/mlx/loader_test.go:68-170
    qw = ck.LoadWeight(valid_source(ck), "proj", 999, 999, 8, 4)
    assert (qw.OutDim, qw.InDim, qw.Groups, qw.Weight.size) == (2, 8, 1, 2)
    assert list(qw.Weight) == [0x76543210, 0xfedcba98]
    s = valid_source(ck)
    s["proj.scales"] = (struct.pack("<2H", 0x3c00, 0x4000), "F16", [2, 1])
    s["proj.biases"] = (struct.pack("<2H", 0xbf80, 0x3f00), "BF16", [2, 1])
    qw = ck.LoadWeight(s, "proj", 2, 8, 8, 4)
    assert list(qw.Scales) == [1, 2] and list(qw.Biases) == [-1, 0.5]
    for out_dim, in_dim, gs, bits, want in [(2, 8, 8, 0, "bits"), (2, 8, 8, 5, "bits"), (2, 8, 0, 4, "groupSize")]:
        with pytest.raises(ck.CheckpointError, match=want):
            ck.LoadWeight(valid_source(ck), "proj", out_dim, in_dim, gs, bits)
    s = valid_source(ck)
    s["proj.weight"] = (s["proj.weight"][0], "U32", [])
    with pytest.raises(ck.CheckpointError, match="inDim"):
        ck.LoadWeight(s, "proj", 2, 7, 8, 4)
    s = valid_source(ck)
    s["proj.scales"] = (struct.pack("<f", 0.1), "F32", [1, 1])
    with pytest.raises(ck.CheckpointError, match="length mismatch"):
        ck.LoadWeight(s, "proj", 2, 8, 8, 4)
    s = valid_source(ck)
    s["proj.biases"] = (struct.pack("<2f", -0.1, -0.2), "F32", [3, 1])
    with pytest.raises(ck.CheckpointError, match="shape"):
        ck.LoadWeight(s, "proj", 2, 8, 8, 4)
    s = valid_source(ck)
    s["proj.scales"] = (struct.pack("<2I", 1, 2), "I32", [2, 1])
    with pytest.raises(ck.CheckpointError, match="unsupported dtype I32"):
        ck.LoadWeight(s, "proj", 2, 8, 8, 4)
    max_int = 2 ** 63 - 1
    s = valid_source(ck)
    s["proj.weight"] = (s["proj.weight"][0], "U32", [2, max_int // 2 + 1])
    with pytest.raises(ck.CheckpointError, match="overflows"):
        ck.LoadWeight(s, "proj", 2, 8, 8, 4)
    s = valid_source(ck)
    s["proj.scales"] = (struct.pack("<2f", 0.1, 0.2), "F32", [max_int // 2 + 1, 3])
    with pytest.raises(ck.CheckpointError, match="overflows"):
        ck.LoadWeight(s, "proj", 2, 8, 8, 4)
    with pytest.raises(ck.CheckpointError, match="load other.weight"):
        ck.LoadWeight(valid_source(ck), "other", 2, 8, 8, 4)


def test_safetensors_round_trip(ck, pkg, tmp_path):
    w, s, b = pkg.synth.mlx_weight("ck", 24, 128, 64)
    bf16 = (s.view(np.uint32) >> 16).astype(np.uint16)
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, {"l.q.weight": ("U32", [24, 16], w.tobytes()), "l.q.scales": ("BF16", [24, 2], bf16.tobytes()),
                             "l.q.biases": ("F32", [24, 2], b.tobytes()), "aux": ("I64", [3], np.arange(3, dtype=np.int64).tobytes())},
                      metadata={"format": "mlx"})
    f = ck.SafetensorsFile(path)
    assert f.Names() == ["aux", "l.q.biases", "l.q.scales", "l.q.weight"]     # sorted, metadata skipped
    raw, dtype, shape = f.GetRaw("l.q.weight")
    assert dtype == "U32" and shape == [24, 16] and raw.tobytes() == w.tobytes()
    qw = ck.LoadWeight(f, "l.q", 0, 0, 64, 4)
    assert (qw.OutDim, qw.InDim, qw.Groups) == (24, 128, 2)
    assert np.array_equal(qw.Weight, w.reshape(-1)) and np.array_equal(qw.Biases, b.reshape(-1))
    assert np.array_equal(qw.Scales, s.reshape(-1))     # the synthetic scales are bf16 values
    with pytest.raises(ck.CheckpointError, match="not found"):
        f.GetRaw("nope")
    del raw, qw
    f.Close()
    with pytest.raises(ck.CheckpointError, match="closed"):
        f.GetRaw("aux")


def test_safetensors_rejects_malformed(ck, tmp_path):
    # loader/safetensors/safetensors_test.go:140-159 and the Open checks
    p = str(tmp_path / "bad.safetensors")

    def put(header, data=b"\0" * 16, hlen=None):
        h = json.dumps(header).encode()
        with open(p, "wb") as fh:
            fh.write(struct.pack("<Q", len(h) if hlen is None else hlen) + h + data)

    open(p, "wb").write(b"\0" * 7)
    with pytest.raises(ck.CheckpointError, match="too short"):
        ck.SafetensorsFile(p)
    put({}, hlen=1 << 40)
    with pytest.raises(ck.CheckpointError, match="header length"):
        ck.SafetensorsFile(p)
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(ck.CheckpointError, match="parse header"):
        ck.SafetensorsFile(p)
    put({"t": {"dtype": "F32", "shape": [4], "data_offsets": [8, 4]}})
    with pytest.raises(ck.CheckpointError, match="invalid data offsets"):
        ck.SafetensorsFile(p)
    put({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 32]}})
    with pytest.raises(ck.CheckpointError, match="invalid data offsets"):
        ck.SafetensorsFile(p)
    put({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 15]}})
    with pytest.raises(ck.CheckpointError, match="expects 16 bytes, got 15"):
        ck.SafetensorsFile(p)
    put({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}})
    with pytest.raises(ck.CheckpointError, match="expects 12 bytes"):
        ck.SafetensorsFile(p)
    put({"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 16]}})
    with pytest.raises(ck.CheckpointError, match="invalid shape"):
        ck.SafetensorsFile(p)
    put({"t": {"dtype": "F32"}})
    with pytest.raises(ck.CheckpointError, match="parse tensor"):
        ck.SafetensorsFile(p)


def test_gguf_round_trip(ck, pkg, tmp_path):
    q4 = pkg.synth.q4k_matrix("ck", 6, 512)
    q8 = pkg.synth.q8_0_matrix("ck", 5, 96)
    q6 = pkg.synth.q6k_matrix("ck", 3, 256)
    f32 = np.arange(7, dtype=np.float32)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, {"general.architecture": "llama", "llama.block_count": np.uint32(2), "general.alignment": np.uint32(32),
                      "tokens": ["a", "bc"], "rope": np.float32(1e6), "flag": True, "big": np.uint64(1 << 40)},
               [("blk.0.ffn_gate.weight", [512, 6], 12, q4.tobytes()), ("blk.0.attn_q.weight", [96, 5], 8, q8.tobytes()),
                ("output.weight", [256, 3], 14, q6.tobytes()), ("norm.weight", [7], 0, f32.tobytes())])
    g = ck.GGUFFile(path)
    assert g.DataOffset % 32 == 0
    assert g.MetaString("general.architecture") == ("llama", True) and g.MetaUint32("llama.block_count") == (2, True)
    assert g.Meta["tokens"] == ["a", "bc"] and g.Meta["flag"] is True and g.Meta["big"] == 1 << 40
    assert g.MetaUint32("general.architecture") == (0, False) and g.MetaString("missing") == ("", False)
    assert [t.Name for t in g.Tensors] == ["blk.0.ffn_gate.weight", "blk.0.attn_q.weight", "output.weight", "norm.weight"]
    m = g.MatrixFromTensor(g.TensorByName("blk.0.ffn_gate.weight"))
    assert (m.QType, m.InDim, m.OutDim, m.RowBytes()) == (12, 512, 6, 288) and m.Raw.tobytes() == q4.tobytes()
    m = g.MatrixFromTensor(g.TensorByName("blk.0.attn_q.weight"))
    assert (m.QType, m.InDim, m.OutDim, m.RowBytes()) == (8, 96, 5, 102) and m.Raw.tobytes() == q8.tobytes()
    m = g.MatrixFromTensor(g.TensorByName("output.weight"))
    assert (m.QType, m.RowBytes()) == (14, 210) and m.Raw.tobytes() == q6.tobytes()
    assert g.Raw(g.TensorByName("norm.weight")).view(np.float32).tolist() == f32.tolist()
    with pytest.raises(ck.CheckpointError, match="not a matrix"):
        g.MatrixFromTensor(g.TensorByName("norm.weight"))
    assert g.TensorByName("nope") is None
    del m
    g.Close()


def test_gguf_raw_byte_counts(ck):
    # loader/gguf/gguf.go:429-480
    for qt, n, want in [(0, 5, 20), (1, 5, 10), (30, 5, 10), (2, 64, 36), (8, 64, 68), (10, 256, 84), (11, 256, 110),
                        (12, 512, 288), (13, 256, 176), (14, 256, 210), (15, 256, 292), (12, 0, 0)]:
        assert ck.TensorRawBytes(qt, n) == want
    for qt, n in [(12, 255), (8, 33), (99, 32), (12, -1)]:
        with pytest.raises(ck.CheckpointError):
            ck.TensorRawBytes(qt, n)


def test_gguf_rejects_malformed(ck, tmp_path):
    # loader/gguf/hardening_test.go:12-140: caps on counts and strings, nested arrays, spans past the file
    p = str(tmp_path / "bad.gguf")
    head = lambda nt, nkv, version=3, magic=b"GGUF": magic + struct.pack("<IQQ", version, nt, nkv)
    string = lambda s: struct.pack("<Q", len(s)) + s.encode()
    cases = [
        (b"GG", "magic"),
        (head(0, 0, magic=b"GGML"), "bad magic"),
        (head(0, 0, version=1), "unsupported version 1"),
        (head(0, 1_000_001), "metadata count"),
        (head(1_000_001, 0), "tensor count"),
        (head(0, 1) + struct.pack("<Q", (16 << 20) + 1), "string length"),
        (head(0, 1) + string("general.architecture") + struct.pack("<IQ", 8, (16 << 20) + 1), "string length"),
        (head(0, 1) + string("tokens") + struct.pack("<IIQ", 9, 8, 1_000_001), "array count"),
        (head(0, 1) + string("bad") + struct.pack("<IIQ", 9, 9, 1), "nested arrays"),
        (head(0, 1) + string("bad") + struct.pack("<I", 77), "unknown GGUFType 77"),
        (head(0, 2) + (string("k") + struct.pack("<II", 4, 1)) * 2, "duplicate metadata key"),
        (head(0, 1) + string("k") + struct.pack("<I", 4), "end of file"),
        (head(1, 0) + string("t") + struct.pack("<I", 0), "rank 0"),
        (head(1, 0) + string("t") + struct.pack("<I", 9), "rank 9"),
        (head(1, 0) + string("t") + struct.pack("<IQQIQ", 2, 256, 4, 12, 0), "data offset 96 exceeds file size"),
        (head(1, 0) + string("t") + struct.pack("<IQQIQ", 2, 256, 4, 12, 0) + b"\0" * 200, "exceeds GGUF data length"),
        (head(1, 0) + string("t") + struct.pack("<IQQIQ", 2, 255, 4, 12, 0) + b"\0" * 4096, "do not fill blocks"),
        (head(1, 0) + string("t") + struct.pack("<IQQIQ", 2, 256, 4, 99, 0) + b"\0" * 4096, "unsupported quant type 99"),
    ]
    for data, want in cases:
        open(p, "wb").write(data)
        with pytest.raises(ck.CheckpointError, match=want):
            ck.GGUFFile(p)
    open(p, "wb").write(b"")
    with pytest.raises(ck.CheckpointError, match="magic"):
        ck.GGUFFile(p)
