"""Importance-matrix files in llama.cpp's legacy binary layout: ``i32 n_entries`` then, per entry,
``i32 name_len, name bytes, i32 ncall, i32 nval, f32 values[nval]`` (values are sums over ``ncall`` chunks).

Reference: crates/pmetal-gguf/src/imatrix.rs:73-245 (load/save with the same sanity limits)."""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict

import numpy as np

MAX_ENTRIES = 100_000
MAX_NAME = 4096
MAX_VALUES = 1 << 28


@dataclass
class IMatrix:
    data: Dict[str, np.ndarray] = field(default_factory=dict)
    ncalls: Dict[str, int] = field(default_factory=dict)

    @classmethod
    def load(cls, path: str) -> "IMatrix":
        with open(path, "rb") as fh:
            buf = fh.read()
        return cls.from_bytes(buf)

    @classmethod
    def from_bytes(cls, buf: bytes) -> "IMatrix":
        pos = 0

        def i32():
            nonlocal pos
            if pos + 4 > len(buf):
                raise ValueError("imatrix: truncated file")
            v = struct.unpack_from("<i", buf, pos)[0]
            pos += 4
            return v
        n = i32()
        if not 0 <= n <= MAX_ENTRIES:
            raise ValueError(f"imatrix: invalid entry count {n}")
        out = cls()
        for k in range(n):
            ln = i32()
            if not 0 < ln <= MAX_NAME or pos + ln > len(buf):
                raise ValueError(f"imatrix: invalid name length {ln} at entry {k}")
            name = buf[pos:pos + ln].decode("utf-8")
            pos += ln
            ncall, nval = i32(), i32()
            if not 0 <= nval <= MAX_VALUES or pos + 4 * nval > len(buf):
                raise ValueError(f"imatrix: invalid value count {nval} at entry {k}")
            vals = np.frombuffer(buf, dtype="<f4", count=nval, offset=pos).astype(np.float32)
            pos += 4 * nval
            out.data[name] = vals / ncall if ncall > 0 else vals
            out.ncalls[name] = ncall
        return out

    def save(self, path: str) -> None:
        with open(path, "wb") as fh:
            fh.write(struct.pack("<i", len(self.data)))
            for name, vals in self.data.items():
                nb = name.encode("utf-8")
                nc = max(self.ncalls.get(name, 1), 1)
                fh.write(struct.pack("<i", len(nb)) + nb + struct.pack("<ii", nc, len(vals)))
                fh.write((np.asarray(vals, dtype=np.float32) * nc).astype("<f4").tobytes())

    def importance(self, name: str) -> float:
        v = self.data.get(name)
        return float(v.sum()) if v is not None else 0.0

    def accumulate(self, name: str, activations: np.ndarray) -> None:
        """Adds one calibration chunk: mean of squared activations per input column."""
        sq = np.mean(np.square(np.asarray(activations, dtype=np.float32).reshape(-1, activations.shape[-1])), axis=0)
        n = self.ncalls.get(name, 0)
        self.data[name] = sq if n == 0 else (self.data[name] * n + sq) / (n + 1)
        self.ncalls[name] = n + 1
