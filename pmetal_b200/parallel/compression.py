"""Gradient compression codecs and wire format (CPU, NumPy).

Restates crates/pmetal-distributed/src/compression.rs:21-480: top-k by magnitude (indices sorted, the
unsent part kept as residual for error feedback), random-k with an LCG and 1/p rescaling, dense
FP16 / BF16 / INT8 (absmax/127, truncation toward zero) / 1-bit (sign + mean |x|) quantisation;
PowerSGD is accepted and falls back to uncompressed, as in the reference. Serialised form:
``u32 original_size | u8 tag (0 full, 1 sparse, 2 fp16, 3 bf16, 4 int8, 5 one-bit) | payload`` (little-endian).
On NVLink the product path only casts in flight (bf16) inside the fused reduce kernel; these codecs
exist for API parity and for slow links.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np


@dataclass
class Compressed:
    original_size: int
    kind: str                    # full | sparse | fp16 | bf16 | int8 | onebit
    data: object
    scale: float = 0.0

    def compressed_bytes(self) -> int:
        if self.kind == "full":
            return self.data.size * 4
        if self.kind == "sparse":
            return self.data[0].size * 4 + self.data[1].size * 4
        if self.kind in ("fp16", "bf16"):
            return self.data.size * 2
        return self.data.size + 4

    def compression_ratio(self) -> float:
        return self.original_size * 4 / max(self.compressed_bytes(), 1)


def _to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = x.astype(np.float32).view(np.uint32)
    rounding = ((u >> 16) & 1) + 0x7FFF
    return ((u + rounding) >> 16).astype(np.uint16)


class GradientCompressor:
    def __init__(self, strategy: str = "none", ratio: float = 0.01, use_error_feedback: bool = True, seed: int = 42):
        self.strategy, self.ratio, self.use_ef = strategy, ratio, use_error_feedback
        self.error: Optional[np.ndarray] = None
        self.rng = seed & 0xFFFFFFFFFFFFFFFF

    def compress(self, grads: np.ndarray) -> Compressed:
        g = grads.astype(np.float32).reshape(-1)
        n = g.size
        work = g + self.error if (self.use_ef and self.error is not None and self.error.size == n) else g.copy()
        residual = None
        s = self.strategy
        if s in ("none", "powersgd"):
            out = Compressed(n, "full", work)
        elif s in ("topk", "top_k"):
            k = max(int(np.float32(n) * np.float32(self.ratio)), 1)
            idx = np.sort(np.argpartition(np.abs(work), n - k)[n - k:]).astype(np.uint32)
            out = Compressed(n, "sparse", (idx, work[idx]))
            residual = work.copy()
            residual[idx] = 0.0
        elif s == "random":
            idx, rng = [], self.rng
            p = np.float32(self.ratio)
            denom = np.float32(0xFFFFFFFF >> 1)
            for i in range(n):
                rng = (rng * 6364136223846793005 + 1) & 0xFFFFFFFFFFFFFFFF
                if np.float32(rng >> 33) / denom < p:
                    idx.append(i)
            self.rng = rng
            idx = np.array(idx, dtype=np.uint32)
            out = Compressed(n, "sparse", (idx, (work[idx] / p).astype(np.float32)))
            residual = work.copy()
            residual[idx] = 0.0
        elif s == "fp16":
            out = Compressed(n, "fp16", work.astype(np.float16).view(np.uint16))
        elif s == "bf16":
            out = Compressed(n, "bf16", _to_bf16_bits(work))
        elif s == "int8":
            m = float(np.abs(work).max()) if n else 0.0
            scale = 1.0 if m == 0.0 else m / 127.0
            out = Compressed(n, "int8", np.trunc(np.clip(work / np.float32(scale), -127, 127)).astype(np.int8), scale)
        elif s in ("onebit", "one_bit"):
            scale = float(np.abs(work).sum(dtype=np.float32) / np.float32(max(n, 1)))
            out = Compressed(n, "onebit", np.packbits(work > 0, bitorder="little"), scale)
        else:
            raise ValueError(f"unknown compression strategy {s!r}")
        if self.use_ef:
            self.error = residual
        return out

    @staticmethod
    def decompress(c: Compressed) -> np.ndarray:
        if c.kind == "full":
            return c.data.astype(np.float32)
        if c.kind == "sparse":
            out = np.zeros(c.original_size, dtype=np.float32)
            idx, val = c.data
            ok = idx < c.original_size
            out[idx[ok]] = val[ok]
            return out
        if c.kind == "fp16":
            return c.data.view(np.float16).astype(np.float32)
        if c.kind == "bf16":
            return (c.data.astype(np.uint32) << 16).view(np.float32)
        if c.kind == "int8":
            return c.data.astype(np.float32) * np.float32(c.scale)
        bits = np.unpackbits(c.data, bitorder="little")[:c.original_size]
        return np.where(bits == 1, np.float32(c.scale), np.float32(-c.scale)).astype(np.float32)


_TAGS = {"full": 0, "sparse": 1, "fp16": 2, "bf16": 3, "int8": 4, "onebit": 5}
_RTAGS = {v: k for k, v in _TAGS.items()}


def serialize(c: Compressed) -> bytes:
    head = struct.pack("<IB", c.original_size, _TAGS[c.kind])
    if c.kind == "full":
        return head + c.data.astype("<f4").tobytes()
    if c.kind == "sparse":
        idx, val = c.data
        return head + struct.pack("<I", idx.size) + idx.astype("<u4").tobytes() + val.astype("<f4").tobytes()
    if c.kind in ("fp16", "bf16"):
        return head + c.data.astype("<u2").tobytes()
    if c.kind == "int8":
        return head + struct.pack("<f", c.scale) + c.data.view(np.uint8).tobytes()
    return head + struct.pack("<f", c.scale) + c.data.tobytes()


def deserialize(buf: bytes) -> Compressed:
    if len(buf) < 5:
        raise ValueError("compressed gradient shorter than its header")
    n, tag = struct.unpack_from("<IB", buf, 0)
    if tag not in _RTAGS:
        raise ValueError(f"unknown compression tag {tag}")
    kind, body = _RTAGS[tag], memoryview(buf)[5:]
    if kind == "full":
        if len(body) != n * 4:
            raise ValueError("full payload length mismatch")
        return Compressed(n, kind, np.frombuffer(body, dtype="<f4").copy())
    if kind == "sparse":
        if len(body) < 4:
            raise ValueError("sparse payload truncated")
        (k,) = struct.unpack_from("<I", body, 0)
        if k > n or len(body) != 4 + 8 * k:
            raise ValueError("sparse payload length mismatch")
        idx = np.frombuffer(body[4:4 + 4 * k], dtype="<u4").copy()
        val = np.frombuffer(body[4 + 4 * k:], dtype="<f4").copy()
        return Compressed(n, kind, (idx, val))
    if kind in ("fp16", "bf16"):
        if len(body) != n * 2:
            raise ValueError("16-bit payload length mismatch")
        return Compressed(n, kind, np.frombuffer(body, dtype="<u2").copy())
    if len(body) < 4:
        raise ValueError("quantised payload truncated")
    (scale,) = struct.unpack_from("<f", body, 0)
    if kind == "int8":
        if len(body) != 4 + n:
            raise ValueError("int8 payload length mismatch")
        return Compressed(n, kind, np.frombuffer(body[4:], dtype=np.int8).copy(), scale)
    if len(body) != 4 + (n + 7) // 8:
        raise ValueError("one-bit payload length mismatch")
    return Compressed(n, kind, np.frombuffer(body[4:], dtype=np.uint8).copy(), scale)
