"""GGUF container reader / writer feeding ``QTensor`` straight from the file's block bytes.

Mirror of the reference's ``lloom-tensor/src/quantized/gguf_file.rs`` for the part of it that sits next to the
quantized matmul: ``Content.read`` (:537-662) parses the header -- magic and version (:52-77), metadata key/values
(:204-535), tensor infos with the dimensions reversed into row-major order (:591-636), the aligned start of the
data section from ``general.alignment`` (:638-653) -- with the reference's size caps (:12-20) and lazy payload
checks (:125-145, :664-669); ``Content.tensor`` (:671-683) reads one tensor's bytes and hands them to the device
slot exactly as stored (``qtensor_from_ggml`` -> ``QStorage::from_data``, ggml_file.rs:180-228): the file's block
stream IS the device layout, so ingest is one staged copy (pinned host buffer -> device), no repack.
``write`` (:749-) is the inverse for the same subset.  Tensor types other than Q8_0 / Q4_K / Q6_K are listed by
``read`` but refused by ``tensor``: there is no fallback path.
"""
from __future__ import annotations

import io
import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, Iterable, List, Sequence, Tuple

DEFAULT_ALIGNMENT = 32
GGUF_MAX_STRING_LENGTH = 1 << 30
GGUF_MAX_ARRAY_ELEMENTS = 1 << 30
GGUF_MAX_TENSOR_DIMS = 4
GGUF_MAX_VALUE_DEPTH = 64
_MAGICS = (0x46554747, 0x47475546)

# GGUF metadata value types (gguf_file.rs:204-235)
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
           T_U64: "<Q", T_I64: "<q", T_F64: "<d"}

# (block elements, block bytes) of every ggml type id a header may name (mod.rs:505-568, :663-715); only the
# first three can be loaded
_TYPE_GEOMETRY = {8: (32, 34), 12: (256, 144), 14: (256, 210),
                  0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 9: (32, 36),
                  10: (256, 84), 11: (256, 110), 13: (256, 176), 15: (256, 292), 30: (1, 2)}
LOADABLE = (8, 12, 14)


class GgufError(ValueError):
    pass


def _need(f: BinaryIO, n: int) -> bytes:
    b = f.read(n)
    if len(b) != n:
        raise GgufError(f"gguf: unexpected end of file (wanted {n} bytes, got {len(b)})")
    return b


@dataclass
class TensorInfo:
    """gguf_file.rs:81-171.  ``shape`` is row-major (the file stores innermost first); ``offset`` is relative to the
    data section."""

    ggml_dtype: int
    shape: Tuple[int, ...]
    offset: int

    def size_in_bytes(self) -> int:
        elems = 1
        for d in self.shape:
            elems *= int(d)
        if self.ggml_dtype not in _TYPE_GEOMETRY:
            raise GgufError(f"gguf: unknown ggml dtype {self.ggml_dtype}")
        block, nbytes = _TYPE_GEOMETRY[self.ggml_dtype]
        if elems % block != 0:
            raise GgufError(f"the number of elements {elems} is not divisible by the block size {block}")
        return elems // block * nbytes

    def validate_payload(self, f: BinaryIO, tensor_data_offset: int) -> Tuple[int, int]:
        """File extent check without reading the payload (:125-145).  Returns (start, size)."""
        size = self.size_in_bytes()
        start = tensor_data_offset + self.offset
        file_size = f.seek(0, io.SEEK_END)
        if start > file_size:
            raise GgufError(f"gguf: tensor offset {start} exceeds file size {file_size}, no remaining bytes")
        if size > file_size - start:
            raise GgufError(f"tensor needs {size} bytes at offset {start}, only {file_size - start} remaining in file")
        return start, size

    def read_bytes(self, f: BinaryIO, tensor_data_offset: int):
        """The tensor's block bytes in a pinned host buffer when CUDA is present (so that the upload is one
        asynchronous copy), else in ordinary memory; uint8 torch tensor."""
        import numpy as np
        import torch

        start, size = self.validate_payload(f, tensor_data_offset)
        host = torch.empty(size, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        f.seek(start)
        view = host.numpy()
        got = f.readinto(memoryview(view)) if hasattr(f, "readinto") else None
        if got is None:
            view[:] = np.frombuffer(_need(f, size), dtype=np.uint8)
        elif got != size:
            raise GgufError(f"gguf: unexpected end of file inside tensor data ({got} of {size} bytes)")
        return host

    def read(self, f: BinaryIO, tensor_data_offset: int, device):
        """:147-170 -> QTensor on ``device``."""
        from .quantized import GgmlDType, QTensor

        if self.ggml_dtype not in LOADABLE:
            raise GgufError(f"gguf: ggml dtype {self.ggml_dtype} is not one of Q8_0 / Q4_K / Q6_K (no fallback path)")
        if len(self.shape) != 2:
            raise GgufError(f"gguf: quantized tensor of rank {len(self.shape)}; the matmul slot takes [n, k]")
        return QTensor.from_data(self.read_bytes(f, tensor_data_offset), GgmlDType(self.ggml_dtype), self.shape, device)


class Content:
    """gguf_file.rs:173-178: ``version`` (1..3), ``metadata`` {key: (value_type, value)}, ``tensor_infos``
    {name: TensorInfo}, ``tensor_data_offset``."""

    def __init__(self, version: int, metadata: Dict[str, Tuple[int, Any]], tensor_infos: Dict[str, TensorInfo],
                 tensor_data_offset: int):
        self.version = version
        self.metadata = metadata
        self.tensor_infos = tensor_infos
        self.tensor_data_offset = tensor_data_offset

    # ---- reading ----
    @staticmethod
    def _length(f: BinaryIO, version: int) -> int:
        return struct.unpack("<I", _need(f, 4))[0] if version == 1 else struct.unpack("<Q", _need(f, 8))[0]

    @classmethod
    def _string(cls, f: BinaryIO, version: int, file_size: int) -> str:
        n = cls._length(f, version)
        if n > GGUF_MAX_STRING_LENGTH:
            raise GgufError(f"gguf: string length {n} exceeds max {GGUF_MAX_STRING_LENGTH}")
        if n > file_size - f.tell():
            raise GgufError(f"gguf: string length {n} exceeds remaining file bytes {file_size - f.tell()}")
        return _need(f, n).rstrip(b"\x00").decode("utf-8", errors="replace")

    @classmethod
    def _value(cls, f: BinaryIO, vtype: int, version: int, depth: int, file_size: int):
        if vtype in _SCALAR:
            fmt = _SCALAR[vtype]
            return struct.unpack(fmt, _need(f, struct.calcsize(fmt)))[0]
        if vtype == T_BOOL:
            b = _need(f, 1)[0]
            if b > 1:
                raise GgufError(f"gguf: unexpected bool value {b}")
            return bool(b)
        if vtype == T_STRING:
            return cls._string(f, version, file_size)
        if vtype == T_ARRAY:
            if depth >= GGUF_MAX_VALUE_DEPTH:
                raise GgufError(f"gguf: array nesting depth exceeds {GGUF_MAX_VALUE_DEPTH}")
            etype = struct.unpack("<I", _need(f, 4))[0]
            n = cls._length(f, version)
            if n > GGUF_MAX_ARRAY_ELEMENTS:
                raise GgufError(f"gguf: array length {n} exceeds max {GGUF_MAX_ARRAY_ELEMENTS}")
            if n > file_size - f.tell():  # every element takes at least one byte
                raise GgufError(f"gguf: array length {n} exceeds remaining file bytes")
            return (etype, [cls._value(f, etype, version, depth + 1, file_size) for _ in range(n)])
        raise GgufError(f"gguf: unknown value type {vtype}")

    @classmethod
    def read(cls, f: BinaryIO) -> "Content":
        start = f.tell()
        file_size = f.seek(0, io.SEEK_END)
        f.seek(start)
        magic, version = struct.unpack("<II", _need(f, 8))
        if magic not in _MAGICS:
            raise GgufError(f"unknown magic 0x{magic:08x}")
        if version not in (1, 2, 3):
            raise GgufError(f"gguf: unsupported version {version}")
        tensor_count = cls._length(f, version)
        kv_count = cls._length(f, version)
        if tensor_count > GGUF_MAX_ARRAY_ELEMENTS or kv_count > GGUF_MAX_ARRAY_ELEMENTS:
            raise GgufError(f"gguf: tensor_count {tensor_count} / metadata_kv_count {kv_count} exceed the maximum")
        prefix = 4 if version == 1 else 8
        needed = kv_count * (prefix + 4 + 1) + tensor_count * (prefix + 4 + 4 + 8)
        if needed > file_size - f.tell():
            raise GgufError(f"gguf: header declares {tensor_count} tensors and {kv_count} metadata entries, needs at "
                            f"least {needed} bytes, only {file_size - f.tell()} remaining")
        metadata: Dict[str, Tuple[int, Any]] = {}
        for _ in range(kv_count):
            key = cls._string(f, version, file_size)
            vtype = struct.unpack("<I", _need(f, 4))[0]
            metadata[key] = (vtype, cls._value(f, vtype, version, 0, file_size))
        infos: Dict[str, TensorInfo] = {}
        for _ in range(tensor_count):
            name = cls._string(f, version, file_size)
            nd = struct.unpack("<I", _need(f, 4))[0]
            if nd > GGUF_MAX_TENSOR_DIMS:
                raise GgufError(f"gguf: tensor '{name}' has {nd} dimensions, max is {GGUF_MAX_TENSOR_DIMS}")
            dims = struct.unpack(f"<{nd}I", _need(f, 4 * nd)) if version == 1 else struct.unpack(f"<{nd}Q", _need(f, 8 * nd))
            dtype, offset = struct.unpack("<IQ", _need(f, 12))
            info = TensorInfo(int(dtype), tuple(int(d) for d in reversed(dims)), int(offset))
            info.size_in_bytes()
            infos[name] = info
        position = f.tell()
        alignment = DEFAULT_ALIGNMENT
        if "general.alignment" in metadata:
            vtype, v = metadata["general.alignment"]
            if vtype in (T_U8, T_U16, T_U32) or (vtype in (T_I8, T_I16, T_I32) and v >= 0):
                alignment = int(v)
        if alignment == 0:
            raise GgufError("gguf: general.alignment must be nonzero")
        data_offset = position + (alignment - position % alignment) % alignment
        return cls(version, metadata, infos, data_offset)

    def validate_payloads(self, f: BinaryIO) -> None:
        for info in self.tensor_infos.values():
            info.validate_payload(f, self.tensor_data_offset)

    def tensor(self, f: BinaryIO, name: str, device):
        if name not in self.tensor_infos:
            raise GgufError(f"cannot find tensor info for {name}")
        return self.tensor_infos[name].read(f, self.tensor_data_offset, device)


# ---- writing (gguf_file.rs:695-: version 3, default alignment) ----
def _w_string(f: BinaryIO, s: str) -> None:
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def _w_value(f: BinaryIO, vtype: int, v) -> None:
    if vtype in _SCALAR:
        f.write(struct.pack(_SCALAR[vtype], v))
    elif vtype == T_BOOL:
        f.write(bytes([1 if v else 0]))
    elif vtype == T_STRING:
        _w_string(f, v)
    elif vtype == T_ARRAY:
        etype, items = v
        f.write(struct.pack("<IQ", etype, len(items)))
        for it in items:
            _w_value(f, etype, it)
    else:
        raise GgufError(f"gguf: unknown value type {vtype}")


def packed_offsets(sizes: Iterable[int], alignment: int = DEFAULT_ALIGNMENT) -> List[int]:
    """Offsets of tensors laid out back to back, each padded to the alignment (:704-718)."""
    out, off = [], 0
    for s in sizes:
        out.append(off)
        off += (int(s) + alignment - 1) // alignment * alignment
    return out


def write(f: BinaryIO, metadata: Sequence[Tuple[str, int, Any]], tensors: Sequence[Tuple[str, int, Sequence[int], bytes]]) -> None:
    """``metadata``: (key, value_type, value); ``tensors``: (name, ggml dtype id, row-major dims, packed block bytes)."""
    f.write(struct.pack("<IIQQ", _MAGICS[0], 3, len(tensors), len(metadata)))
    for key, vtype, v in metadata:
        _w_string(f, key)
        f.write(struct.pack("<I", vtype))
        _w_value(f, vtype, v)
    offsets = packed_offsets(len(t[3]) for t in tensors)
    for (name, dtype, dims, data), off in zip(tensors, offsets):
        info = TensorInfo(int(dtype), tuple(int(d) for d in dims), off)
        if info.size_in_bytes() != len(data):
            raise GgufError(f"gguf: tensor '{name}' has {len(data)} bytes, its shape and type need {info.size_in_bytes()}")
        _w_string(f, name)
        f.write(struct.pack("<I", len(dims)))
        f.write(struct.pack(f"<{len(dims)}Q", *reversed([int(d) for d in dims])))
        f.write(struct.pack("<IQ", int(dtype), off))
    pos = f.tell()
    f.write(b"\x00" * ((DEFAULT_ALIGNMENT - pos % DEFAULT_ALIGNMENT) % DEFAULT_ALIGNMENT))
    for (_, _, _, data), off in zip(tensors, offsets):
        f.write(data)
        f.write(b"\x00" * ((DEFAULT_ALIGNMENT - len(data) % DEFAULT_ALIGNMENT) % DEFAULT_ALIGNMENT))
