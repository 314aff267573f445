"""GGUF reader (v2/v3), memory-mapped, with bounds checks suited to untrusted files.

Mirrors the checks of crates/pmetal-gguf/src/reader.rs (magic, version, string/array length caps, tensor extents
inside the file) and is the target of the fuzz-style tests."""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

from .types import BLOCK_GEOMETRY, GGUF_DEFAULT_ALIGNMENT, GGUF_MAGIC, GgmlType, ValueType, tensor_nbytes

MAX_STRING = 1 << 26        # 64 MiB: tokenizer merges are long but not that long
MAX_ARRAY = 1 << 28
MAX_DIMS = 8


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]        # logical, slowest-first
    dtype: GgmlType
    offset: int                   # relative to the data section
    nbytes: int

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class _Cursor:
    def __init__(self, buf, pos=0):
        self.buf, self.pos, self.end = buf, pos, len(buf)

    def take(self, n: int):
        if n < 0 or self.pos + n > self.end:
            raise GgufError(f"truncated file: need {n} bytes at offset {self.pos}, size {self.end}")
        b = self.buf[self.pos:self.pos + n]
        self.pos += n
        return b

    def unpack(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self, v2_32bit=False) -> str:
        n = self.unpack("<I" if v2_32bit else "<Q")
        if n > MAX_STRING:
            raise GgufError(f"string length {n} exceeds the cap")
        return bytes(self.take(n)).decode("utf-8", errors="replace")


_SCALARS = {ValueType.UINT8: "<B", ValueType.INT8: "<b", ValueType.UINT16: "<H", ValueType.INT16: "<h",
            ValueType.UINT32: "<I", ValueType.INT32: "<i", ValueType.FLOAT32: "<f", ValueType.BOOL: "<?",
            ValueType.UINT64: "<Q", ValueType.INT64: "<q", ValueType.FLOAT64: "<d"}


def _read_value(c: _Cursor, vt: int, depth=0):
    try:
        vt = ValueType(vt)
    except ValueError:
        raise GgufError(f"unknown metadata value type {vt}") from None
    if vt == ValueType.STRING:
        return c.string()
    if vt == ValueType.ARRAY:
        if depth > 2:
            raise GgufError("metadata arrays nested too deeply")
        et = c.unpack("<I")
        n = c.unpack("<Q")
        if n > MAX_ARRAY:
            raise GgufError(f"array length {n} exceeds the cap")
        if et in _SCALARS and ValueType(et) != ValueType.BOOL:
            fmt = _SCALARS[ValueType(et)]
            raw = c.take(n * struct.calcsize(fmt))
            return np.frombuffer(raw, dtype=np.dtype(fmt[1:]).newbyteorder("<")).tolist()
        return [_read_value(c, et, depth + 1) for _ in range(n)]
    return c.unpack(_SCALARS[vt])


class GgufFile:
    """Parsed GGUF file. ``tensor_bytes`` returns a zero-copy view; ``tensor_f32`` dequantises on the host."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 24:
            raise GgufError("file too small to be GGUF")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self._parse(memoryview(self._mm))

    @classmethod
    def from_bytes(cls, data: bytes) -> "GgufFile":
        self = cls.__new__(cls)
        self.path, self._fh, self._mm = "<bytes>", None, None
        if len(data) < 24:
            raise GgufError("file too small to be GGUF")
        self._parse(memoryview(data))
        return self

    def _parse(self, buf):
        self._buf = buf
        c = _Cursor(buf)
        if c.unpack("<I") != GGUF_MAGIC:
            raise GgufError("bad magic: not a GGUF file")
        self.version = c.unpack("<I")
        if self.version not in (2, 3):
            raise GgufError(f"unsupported GGUF version {self.version}")
        n_tensors, n_kv = c.unpack("<Q"), c.unpack("<Q")
        if n_tensors > (1 << 24) or n_kv > (1 << 24):
            raise GgufError("implausible tensor / metadata count")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = _read_value(c, c.unpack("<I"))
        self.alignment = int(self.metadata.get("general.alignment", GGUF_DEFAULT_ALIGNMENT)) or GGUF_DEFAULT_ALIGNMENT
        if self.alignment & (self.alignment - 1) or self.alignment > (1 << 20):
            raise GgufError(f"alignment {self.alignment} is not a sane power of two")
        infos: List[TensorInfo] = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.unpack("<I")
            if nd > MAX_DIMS:
                raise GgufError(f"tensor {name}: {nd} dimensions")
            dims = [c.unpack("<Q") for _ in range(nd)]
            tid, off = c.unpack("<I"), c.unpack("<Q")
            try:
                dt = GgmlType(tid)
            except ValueError:
                raise GgufError(f"tensor {name}: unknown ggml type {tid}") from None
            n = 1
            for d in dims:
                n *= d
                if n > (1 << 48):
                    raise GgufError(f"tensor {name}: implausible element count")
            if dt not in BLOCK_GEOMETRY:
                raise GgufError(f"tensor {name}: no block geometry for {dt.name}")
            infos.append(TensorInfo(name, tuple(reversed(dims)), dt, off, tensor_nbytes(dt, n)))
        self.data_start = c.pos + ((-c.pos) % self.alignment)
        for t in infos:
            if self.data_start + t.offset + t.nbytes > len(buf):
                raise GgufError(f"tensor {t.name}: data [{t.offset}, +{t.nbytes}) runs past the end of the file")
        self.tensors: Dict[str, TensorInfo] = {t.name: t for t in infos}
        self.tensor_order = [t.name for t in infos]

    def tensor_bytes(self, name: str) -> memoryview:
        t = self.tensors[name]
        a = self.data_start + t.offset
        return self._buf[a:a + t.nbytes]

    def tensor_f32(self, name: str, threads: int = 0) -> np.ndarray:
        from . import native
        t = self.tensors[name]
        raw = np.frombuffer(self.tensor_bytes(name), dtype=np.uint8)
        if t.dtype in (GgmlType.I8, GgmlType.I16, GgmlType.I32, GgmlType.I64, GgmlType.F64):
            np_t = {GgmlType.I8: np.int8, GgmlType.I16: np.int16, GgmlType.I32: np.int32, GgmlType.I64: np.int64,
                    GgmlType.F64: np.float64}[t.dtype]
            return raw.view(np_t).astype(np.float32).reshape(t.shape)
        return native.dequantize(raw, t.dtype, t.n_elements, threads).reshape(t.shape)

    def close(self):
        self._buf = None
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
        if self._fh is not None:
            self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
