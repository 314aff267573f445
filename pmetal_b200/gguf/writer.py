"""GGUF v3 writer.

File layout (crates/pmetal-gguf/src/writer.rs:180-224,303-341,483-537 of the reference): header (magic, version,
u64 tensor count, u64 metadata count), metadata key/values in **sorted key order** always including
``general.alignment`` and ``general.quantization_version``, tensor infos (name, u32 ndim, dims fastest-first,
u32 ggml type, u64 offset), padding to the alignment, then tensor data in insertion order with every tensor but
the last padded to the alignment."""
from __future__ import annotations

import struct
from typing import BinaryIO, Dict, List, Sequence, Tuple

import numpy as np

from .types import GGUF_DEFAULT_ALIGNMENT, GGUF_MAGIC, GGUF_VERSION, GgmlType, ValueType, tensor_nbytes

_SCALAR_FMT = {ValueType.UINT8: "<B", ValueType.INT8: "<b", ValueType.UINT16: "<H", ValueType.INT16: "<h",
               ValueType.UINT32: "<I", ValueType.INT32: "<i", ValueType.FLOAT32: "<f", ValueType.BOOL: "<?",
               ValueType.UINT64: "<Q", ValueType.INT64: "<q", ValueType.FLOAT64: "<d"}


def _pack_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(vt: ValueType, v) -> bytes:
    if vt == ValueType.STRING:
        return _pack_string(v)
    if vt == ValueType.ARRAY:
        et, items = v
        out = [struct.pack("<IQ", int(et), len(items))]
        out.extend(_pack_value(et, x) for x in items)
        return b"".join(out)
    return struct.pack(_SCALAR_FMT[vt], v)


class GgufWriter:
    def __init__(self, alignment: int = GGUF_DEFAULT_ALIGNMENT):
        self.alignment = alignment
        self.meta: Dict[str, Tuple[ValueType, object]] = {}
        self.tensors: List[Tuple[str, Tuple[int, ...], GgmlType, bytes]] = []
        self.add_u32("general.alignment", alignment)
        self.add_u32("general.quantization_version", 2)

    # ---- metadata
    def add(self, key: str, vt: ValueType, value) -> "GgufWriter":
        self.meta[key] = (vt, value)
        return self

    def add_u32(self, key, v): return self.add(key, ValueType.UINT32, int(v))
    def add_i32(self, key, v): return self.add(key, ValueType.INT32, int(v))
    def add_u64(self, key, v): return self.add(key, ValueType.UINT64, int(v))
    def add_f32(self, key, v): return self.add(key, ValueType.FLOAT32, float(v))
    def add_bool(self, key, v): return self.add(key, ValueType.BOOL, bool(v))
    def add_string(self, key, v): return self.add(key, ValueType.STRING, str(v))

    def add_array(self, key, elem_type: ValueType, items: Sequence) -> "GgufWriter":
        return self.add(key, ValueType.ARRAY, (elem_type, list(items)))

    # ---- tensors
    def add_tensor_bytes(self, name: str, shape: Sequence[int], dtype: GgmlType, data) -> "GgufWriter":
        """``shape`` is the logical (row-major, slowest-first) shape; ``data`` the encoded bytes."""
        data = bytes(data) if not isinstance(data, (bytes, bytearray, memoryview)) else data
        n = 1
        for d in shape:
            n *= int(d)
        need = tensor_nbytes(GgmlType(dtype), n)
        if len(data) != need:
            raise ValueError(f"{name}: {len(data)} bytes given, {need} expected for {tuple(shape)} {GgmlType(dtype).name}")
        self.tensors.append((name, tuple(int(d) for d in shape), GgmlType(dtype), data))
        return self

    def add_tensor_f32(self, name: str, arr: np.ndarray, dtype: GgmlType = GgmlType.F32, threads: int = 0):
        from . import native
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        return self.add_tensor_bytes(name, arr.shape, dtype, native.quantize(arr, dtype, threads).tobytes())

    # ---- output
    def _pad(self, n: int) -> int:
        return (-n) % self.alignment

    def write(self, fh: BinaryIO) -> int:
        head = [struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(self.tensors), len(self.meta))]
        for key in sorted(self.meta):
            vt, v = self.meta[key]
            head.append(_pack_string(key) + struct.pack("<I", int(vt)) + _pack_value(vt, v))
        offset = 0
        for i, (name, shape, dtype, data) in enumerate(self.tensors):
            head.append(_pack_string(name) + struct.pack("<I", len(shape)) +
                        b"".join(struct.pack("<Q", d) for d in reversed(shape)) + struct.pack("<IQ", int(dtype), offset))
            offset += len(data)
            if i + 1 < len(self.tensors):
                offset += self._pad(len(data))
        blob = b"".join(head)
        fh.write(blob)
        fh.write(b"\0" * self._pad(len(blob)))
        written = len(blob) + self._pad(len(blob))
        for i, (_, _, _, data) in enumerate(self.tensors):
            fh.write(data)
            written += len(data)
            if i + 1 < len(self.tensors):
                pad = self._pad(len(data))
                fh.write(b"\0" * pad)
                written += pad
        return written

    def write_to(self, path: str) -> int:
        with open(path, "wb") as fh:
            return self.write(fh)
