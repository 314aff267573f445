"""Offline teacher-logit cache with per-sequence compression (crates/pmetal-distill/src/offline.rs:27-760).

A cache directory holds ``metadata.json`` and one ``seq_{id}.npz`` per sequence. Compression methods: ``full`` (fp32),
``topk`` (k values + int32 indices per token; the rest of the distribution is spread uniformly on decompression so
probabilities still sum to one), ``int8`` / ``int4`` (one affine scale per tensor) and ``int8_per_token``."""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Dict

import numpy as np
import torch


@dataclass
class CacheMetadata:
    model: str = ""
    vocab_size: int = 0
    max_seq_len: int = 0
    compression: str = "topk"
    top_k: int = 64
    num_sequences: int = 0


class LogitCompressor:
    def __init__(self, method: str = "topk", top_k: int = 64):
        if method not in ("full", "topk", "int8", "int4", "int8_per_token"):
            raise ValueError(method)
        self.method, self.top_k = method, top_k

    def compress(self, logits: torch.Tensor) -> Dict[str, np.ndarray]:
        x = logits.detach().float().cpu()
        if self.method == "full":
            return {"kind": np.array("full"), "data": x.numpy()}
        if self.method == "topk":
            k = min(self.top_k, x.shape[-1])
            v, i = x.topk(k, -1)
            lse = torch.logsumexp(x, -1)
            return {"kind": np.array("topk"), "values": v.numpy(), "indices": i.to(torch.int32).numpy(),
                    "lse": lse.numpy(), "vocab": np.array(x.shape[-1])}
        if self.method == "int8_per_token":
            lo, hi = x.min(-1, keepdim=True).values, x.max(-1, keepdim=True).values
            sc = (hi - lo).clamp(min=1e-8) / 255
            q = ((x - lo) / sc).round().clamp(0, 255).to(torch.uint8)
            return {"kind": np.array("int8_per_token"), "q": q.numpy(), "meta": torch.cat([sc, lo], -1).numpy()}
        bits = 8 if self.method == "int8" else 4
        lo, hi = float(x.min()), float(x.max())
        sc = max(hi - lo, 1e-8) / (2 ** bits - 1)
        q = ((x - lo) / sc).round().clamp(0, 2 ** bits - 1).to(torch.uint8)
        if bits == 4:
            flat = q.reshape(-1)
            if flat.numel() % 2:
                flat = torch.cat([flat, flat.new_zeros(1)])
            q = (flat[0::2] | (flat[1::2] << 4))
        return {"kind": np.array(self.method), "q": q.numpy(), "scale": np.array(sc, np.float32),
                "zero": np.array(lo, np.float32), "shape": np.array(x.shape)}

    @staticmethod
    def decompress(blob: Dict[str, np.ndarray]) -> torch.Tensor:
        kind = str(blob["kind"])
        if kind == "full":
            return torch.from_numpy(blob["data"])
        if kind == "topk":
            v, i = torch.from_numpy(blob["values"]), torch.from_numpy(blob["indices"]).long()
            V = int(blob["vocab"])
            lse = torch.from_numpy(blob["lse"])
            k = v.shape[-1]
            # mass outside the top-k, spread uniformly over the remaining entries
            rest = (1 - torch.exp(v - lse[..., None]).sum(-1)).clamp(min=1e-12)
            fill = torch.log(rest / max(V - k, 1)) + lse
            out = fill[..., None].expand(*v.shape[:-1], V).clone()
            out.scatter_(-1, i, v)
            return out
        if kind == "int8_per_token":
            meta = torch.from_numpy(blob["meta"])
            return torch.from_numpy(blob["q"]).float() * meta[..., :1] + meta[..., 1:]
        shape = tuple(int(s) for s in blob["shape"])
        q = torch.from_numpy(blob["q"])
        if kind == "int4":
            q = torch.stack([q & 15, q >> 4], -1).reshape(-1)[: int(np.prod(shape))]
        return (q.float() * float(blob["scale"]) + float(blob["zero"])).reshape(shape)


class LogitCache:
    def __init__(self, cache_dir: str, compression: str = "topk", top_k: int = 64):
        self.dir = cache_dir
        os.makedirs(cache_dir, exist_ok=True)
        self.meta = CacheMetadata(compression=compression, top_k=top_k)
        self.comp = LogitCompressor(compression, top_k)

    @classmethod
    def load(cls, cache_dir: str) -> "LogitCache":
        with open(os.path.join(cache_dir, "metadata.json"), "r", encoding="utf-8") as fh:
            meta = CacheMetadata(**json.load(fh))
        c = cls(cache_dir, meta.compression, meta.top_k)
        c.meta = meta
        return c

    def _path(self, seq_id: int) -> str:
        return os.path.join(self.dir, f"seq_{seq_id}.npz")

    def cache_sequence(self, seq_id: int, logits: torch.Tensor) -> None:
        np.savez(self._path(seq_id), **self.comp.compress(logits))
        self.meta.num_sequences = max(self.meta.num_sequences, seq_id + 1)
        self.meta.vocab_size = logits.shape[-1]
        self.meta.max_seq_len = max(self.meta.max_seq_len, logits.shape[-2])

    def has_sequence(self, seq_id: int) -> bool:
        return os.path.exists(self._path(seq_id))

    def load_sequence(self, seq_id: int) -> torch.Tensor:
        with np.load(self._path(seq_id), allow_pickle=False) as z:
            return LogitCompressor.decompress({k: z[k] for k in z.files})

    def save_metadata(self) -> None:
        tmp = os.path.join(self.dir, "metadata.json.tmp")
        with open(tmp, "w", encoding="utf-8") as fh:
            json.dump(asdict(self.meta), fh, indent=2)
        os.replace(tmp, os.path.join(self.dir, "metadata.json"))

    def stats(self, seq_id: int) -> dict:
        raw = self.meta.vocab_size * 4
        size = os.path.getsize(self._path(seq_id))
        return {"compressed_bytes": size, "ratio_per_token_row": raw / max(size, 1)}
