"""Safetensors reader/writer with control over header bytes and tensor order.

File layout: u64 little-endian header length, UTF-8 JSON header, raw tensor bytes.
Each header entry is ``{"dtype", "shape", "data_offsets":[begin,end]}`` with offsets
relative to the start of the data section; ``__metadata__`` holds string pairs.

The adapter files of the reference are produced by MLX's writer
(crates/pmetal-bridge/cpp/bridge_training.cpp:235-245), which iterates an unordered
map, so the tensor order in those files is unspecified; this writer uses sorted key
order, tags ``{"format": "mlx"}`` when asked, and pads the header with spaces to an
8-byte boundary as the safetensors reference implementation does.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

_DT = {
    torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
    torch.bool: "BOOL",
}
if hasattr(torch, "float8_e4m3fn"):
    _DT[torch.float8_e4m3fn] = "F8_E4M3"
    _DT[torch.float8_e5m2] = "F8_E5M2"
if hasattr(torch, "uint32"):
    _DT[torch.uint32] = "U32"
    _DT[torch.uint16] = "U16"
_RDT = {v: k for k, v in _DT.items()}
_SIZE = {"F32": 4, "F16": 2, "BF16": 2, "F64": 8, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1,
         "F8_E4M3": 1, "F8_E5M2": 1, "U32": 4, "U16": 2}


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None,
              order: Optional[Iterable[str]] = None) -> None:
    names = list(order) if order is not None else sorted(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for n in names:
        t = tensors[n]
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(hj)))
        fh.write(hj)
        for n in names:
            fh.write(_raw_bytes(tensors[n]))
    os.replace(tmp, path)


def read_header(path: str) -> Tuple[dict, int]:
    with open(path, "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        if n > 100 * 1024 * 1024:
            raise ValueError("safetensors header too large")
        header = json.loads(fh.read(n).decode("utf-8"))
    return header, 8 + n


class LazyFile:
    """Memory-mapped safetensors file; tensors are materialised one at a time."""

    def __init__(self, path: str):
        self.path = path
        self.header, self.base = read_header(path)
        self.metadata = self.header.pop("__metadata__", {}) or {}
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for k, e in self.header.items():
            b, en = e["data_offsets"]
            n = int(np.prod(e["shape"])) if e["shape"] else 1
            if en < b or self.base + en > size or (en - b) != n * _SIZE[e["dtype"]]:
                raise ValueError(f"corrupt safetensors entry {k!r}")

    def keys(self):
        return list(self.header.keys())

    def info(self, name: str):
        e = self.header[name]
        return e["dtype"], tuple(e["shape"])

    def get(self, name: str) -> torch.Tensor:
        e = self.header[name]
        b, en = e["data_offsets"]
        dt = _RDT[e["dtype"]]
        if en == b:
            return torch.empty(e["shape"], dtype=dt)
        buf = bytearray(self._mm[self.base + b:self.base + en])
        return torch.frombuffer(buf, dtype=torch.uint8).view(dt).reshape(e["shape"])

    def close(self):
        if self._mm is not None:
            self._mm.close()
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def load_file(path: str) -> Dict[str, torch.Tensor]:
    with LazyFile(path) as f:
        return {k: f.get(k) for k in f.keys()}


def load_metadata(path: str) -> Dict[str, str]:
    header, _ = read_header(path)
    return header.get("__metadata__", {}) or {}


def load_file_parallel(path: str, names: Optional[Iterable[str]] = None, threads: int = 8,
                       pin: bool = False) -> Dict[str, torch.Tensor]:
    """Read tensors with several positional reads in flight (``csrc/host/runtime.cpp: pm_read_ranges``): each tensor gets
    its own (optionally pinned) buffer and worker threads fill them directly, large tensors split into 64 MiB pieces.
    ``names`` restricts the load to some tensors (a shard of a tensor-parallel or pipeline rank)."""
    import ctypes
    from . import hostlib
    header, base = read_header(path)
    header.pop("__metadata__", None)
    size = os.path.getsize(path)
    want = list(names) if names is not None else list(header)
    out: Dict[str, torch.Tensor] = {}
    offs, sizes, ptrs = [], [], []
    for k in want:
        e = header[k]
        b, en = e["data_offsets"]
        n = int(np.prod(e["shape"])) if e["shape"] else 1
        if en < b or base + en > size or (en - b) != n * _SIZE[e["dtype"]]:
            raise ValueError(f"corrupt safetensors entry {k!r}")
        t = torch.empty(e["shape"], dtype=_RDT[e["dtype"]], pin_memory=pin and en > b)
        out[k] = t
        if en > b:
            offs.append(base + b)
            sizes.append(en - b)
            ptrs.append(t.data_ptr())
    if offs:
        L = hostlib.load()
        L.pm_read_ranges.restype = ctypes.c_int
        L.pm_read_ranges.argtypes = [ctypes.c_char_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_int]
        n = len(offs)
        a_off = (ctypes.c_int64 * n)(*offs)
        a_size = (ctypes.c_int64 * n)(*sizes)
        a_ptr = (ctypes.c_void_p * n)(*ptrs)
        rc = L.pm_read_ranges(os.fsencode(path), n, a_off, a_size, a_ptr, int(threads))
        if rc != 0:
            raise OSError(-rc, f"reading {path}: {os.strerror(-rc)}")
    return out
