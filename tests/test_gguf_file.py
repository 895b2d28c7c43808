"""GGUF ingest (gguf_file.rs / ggml_file.rs:180-228): header parsing, the reference's validation rules, and the path
from a file's block bytes to a device QTensor -- byte identity through ``data()`` and the same dequantized values
and products as the oracle gives for those bytes."""
import io
import struct

import numpy as np
import pytest

from lloom_b200 import gguf_file as G


def _weights(oracle, dt, n, k, seed):
    w = np.random.default_rng(seed).standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
    return oracle.quantize(dt, w, nthreads=4)


def _sample_file(oracle):
    tensors = [("blk.0.ffn_up.weight", 12, (48, 512), _weights(oracle, 12, 48, 512, 1).tobytes()),
               ("output.weight", 14, (40, 256), _weights(oracle, 14, 40, 256, 2).tobytes()),
               ("blk.0.attn_q.weight", 8, (33, 64), _weights(oracle, 8, 33, 64, 3).tobytes()),
               ("blk.0.attn_norm.weight", 0, (64,), np.arange(64, dtype=np.float32).tobytes())]
    meta = [("general.architecture", G.T_STRING, "llama"), ("llama.block_count", G.T_U32, 1),
            ("general.alignment", G.T_U32, 32), ("x.f", G.T_F32, 0.5), ("x.flag", G.T_BOOL, True),
            ("x.i64", G.T_I64, -5), ("tokenizer.ggml.tokens", G.T_ARRAY, (G.T_STRING, ["a", "bc", ""])),
            ("x.nested", G.T_ARRAY, (G.T_ARRAY, [(G.T_U8, [1, 2]), (G.T_U8, [])]))]
    f = io.BytesIO()
    G.write(f, meta, tensors)
    f.seek(0)
    return f, meta, tensors


def test_header_round_trip(oracle):
    f, meta, tensors = _sample_file(oracle)
    c = G.Content.read(f)
    assert c.version == 3 and c.tensor_data_offset % 32 == 0
    assert c.metadata["general.architecture"] == (G.T_STRING, "llama")
    assert c.metadata["llama.block_count"] == (G.T_U32, 1)
    assert c.metadata["x.i64"] == (G.T_I64, -5) and c.metadata["x.flag"] == (G.T_BOOL, True)
    assert c.metadata["tokenizer.ggml.tokens"] == (G.T_ARRAY, (G.T_STRING, ["a", "bc", ""]))
    assert c.metadata["x.nested"][1] == (G.T_ARRAY, [(G.T_U8, [1, 2]), (G.T_U8, [])])
    assert set(c.tensor_infos) == {t[0] for t in tensors}
    for name, dt, dims, data in tensors:
        info = c.tensor_infos[name]
        assert info.ggml_dtype == dt and info.shape == tuple(dims) and info.offset % 32 == 0
        start, size = info.validate_payload(f, c.tensor_data_offset)
        assert size == len(data)
        f.seek(start)
        assert f.read(size) == data  # the file holds the block stream as the device will
    c.validate_payloads(f)


def test_dims_are_stored_innermost_first(oracle):
    f, _, _ = _sample_file(oracle)
    raw = f.getvalue()
    name = b"blk.0.ffn_up.weight"
    at = raw.index(name) + len(name)
    nd, d0, d1 = struct.unpack_from("<IQQ", raw, at)
    assert (nd, d0, d1) == (2, 512, 48)  # k first, then n: the reader reverses (gguf_file.rs:626)


def test_reader_rejects_bad_files(oracle):
    f, _, _ = _sample_file(oracle)
    raw = f.getvalue()
    with pytest.raises(G.GgufError, match="unknown magic"):
        G.Content.read(io.BytesIO(b"XXXX" + raw[4:]))
    with pytest.raises(G.GgufError):
        G.Content.read(io.BytesIO(raw[:40]))  # header cut short
    # header intact, data section cut: parsing is lazy, the payload check is not
    c = G.Content.read(io.BytesIO(raw))
    cut = io.BytesIO(raw[: c.tensor_data_offset + 100])
    G.Content.read(cut)
    with pytest.raises(G.GgufError, match="remaining"):
        c.validate_payloads(cut)
    # more tensors / entries declared than the file could hold
    with pytest.raises(G.GgufError, match="needs at least"):
        G.Content.read(io.BytesIO(raw[:8] + struct.pack("<QQ", 1 << 20, 1 << 20) + raw[24:]))
    # five dimensions
    bad = io.BytesIO()
    bad.write(struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + struct.pack("<Q", 1) + b"t" + struct.pack("<I", 5) + b"\0" * 64)
    bad.seek(0)
    with pytest.raises(G.GgufError, match="dimensions"):
        G.Content.read(bad)
    # element count not a whole number of blocks
    odd = io.BytesIO()
    odd.write(struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + struct.pack("<Q", 1) + b"t" + struct.pack("<I", 1)
              + struct.pack("<Q", 100) + struct.pack("<IQ", 12, 0))
    odd.seek(0)
    with pytest.raises(G.GgufError, match="not divisible"):
        G.Content.read(odd)
    # zero alignment
    z = io.BytesIO()
    G.write(z, [("general.alignment", G.T_U32, 0)], [])
    z.seek(0)
    with pytest.raises(G.GgufError, match="alignment"):
        G.Content.read(z)


def test_third_party_writer_is_read(oracle, tmp_path):
    """A file written by the gguf package (independent of this repository's writer) parses to the same tensors."""
    gguf = pytest.importorskip("gguf")
    wq = _weights(oracle, 12, 16, 256, 7)
    path = tmp_path / "t.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("llama.block_count", 2)
    w.add_tensor("blk.0.ffn_down.weight", wq, raw_shape=wq.shape, raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with open(path, "rb") as f:
        c = G.Content.read(f)
        info = c.tensor_infos["blk.0.ffn_down.weight"]
        assert info.ggml_dtype == 12 and info.shape == (16, 256)
        start, size = info.validate_payload(f, c.tensor_data_offset)
        f.seek(start)
        assert f.read(size) == wq.tobytes()
    assert c.metadata["llama.block_count"] == (G.T_U32, 2)


@pytest.mark.gpu
def test_tensor_ingest_to_device(oracle, cuda_lib, tmp_path):
    import torch

    import lloom_b200 as lb

    f, _, tensors = _sample_file(oracle)
    path = tmp_path / "m.gguf"
    path.write_bytes(f.getvalue())
    dev = torch.device("cuda", 0)
    with open(path, "rb") as fh:
        c = G.Content.read(fh)
        for name, dt, dims, data in tensors[:3]:
            qt = c.tensor(fh, name, dev)
            assert qt.shape == tuple(dims) and int(qt.dtype()) == dt
            assert qt.data() == data  # packed byte identity (ggml_file_tests.rs:78-82)
            wq = np.frombuffer(data, dtype=np.uint8).reshape(dims[0], -1)
            assert qt.dequantize().cpu().numpy().tobytes() == oracle.dequantize(dt, wq, dims[1]).tobytes()
            x = np.random.default_rng(5).standard_normal((3, dims[1])).astype(np.float32)
            got = lb.QMatMul.from_qtensor(qt).forward(torch.from_numpy(x).to(dev)).cpu().numpy()
            ref = oracle.matmul(dt, x, wq, dims[0], nthreads=4)
            absum = oracle.matmul_absum(dt, x, wq, dims[0], nthreads=4)
            assert (np.abs(got.astype(np.float64) - ref) <= 1e-5 * absum + 1e-30).all()
        with pytest.raises(G.GgufError, match="no fallback"):
            c.tensor(fh, "blk.0.attn_norm.weight", dev)
        with pytest.raises(G.GgufError, match="cannot find"):
            c.tensor(fh, "missing", dev)


# ---- the reference's header-hardening cases (lloom-tensor/tests/gguf_tests.rs:10-112, 222-240), rebuilt byte by byte ----
def _header(tensor_count, kv_count, version=3):
    if version == 1:
        return struct.pack("<IIII", 0x46554747, 1, tensor_count, kv_count)
    return struct.pack("<IIQQ", 0x46554747, version, tensor_count, kv_count)


def _lp(s: bytes) -> bytes:
    return struct.pack("<Q", len(s)) + s


def _rejects(buf: bytes, msg: str):
    with pytest.raises(G.GgufError, match=msg):
        G.Content.read(io.BytesIO(buf))


def test_reference_header_hardening_cases():
    for version in (3, 1):  # empty_header_loads, empty_v1_header_loads
        c = G.Content.read(io.BytesIO(_header(0, 0, version)))
        assert not c.metadata and not c.tensor_infos
    _rejects(_header(0, 1 << 31), "metadata_kv_count")
    _rejects(_header(1 << 31, 0), "tensor_count")
    _rejects(_header(1, 0) + struct.pack("<Q", 1 << 31) + b"\0" * 64, "string length")
    _rejects(_header(0, 1) + _lp(b"k") + struct.pack("<IIQ", 9, 0, 1 << 31) + b"\0" * 64, "array length")
    _rejects(_header(1, 0) + _lp(b"t") + struct.pack("<I", 0xFFFFFFFF) + b"\0" * 64, "dimensions")
    nested = _header(0, 1) + _lp(b"k") + struct.pack("<I", 9)
    nested += struct.pack("<IQ", 9, 1) * 256 + struct.pack("<IQ", 0, 0)
    _rejects(nested, "nesting depth")
    _rejects(_header(1, 0) + struct.pack("<Q", 1 << 20) + b"\0" * 40, "remaining file bytes")  # string longer than the file


def test_reference_alignment_cases():
    def alignment_header(a):
        return _header(0, 1) + _lp(b"general.alignment") + struct.pack("<II", 4, a)

    _rejects(alignment_header(0), "alignment must be nonzero")
    for a in (1, 8, 24, 32):  # positive legacy alignments are kept, powers of two or not
        buf = alignment_header(a)
        assert G.Content.read(io.BytesIO(buf)).tensor_data_offset == -(-len(buf) // a) * a
