"""Rotary-embedding frequency schedules shared by the fast decoder and the portable architectures.

The default, linear, llama3, yarn and dynamic-NTK variants produce one vector of inverse frequencies
[dim/2] and one attention factor (a scale on cos and sin); the native RoPE-table kernel consumes both.
Behaviour parity: pmetal-mlx/src/kernels/rope.rs (scaled and NTK-aware frequencies).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def rope_inv_freq(dim: int, theta: float, scaling: Optional[dict], max_position: int) -> Tuple[torch.Tensor, float]:
    """Inverse frequencies [dim/2] and the attention factor for the default, linear, dynamic-NTK, llama3, yarn and longrope variants."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if not scaling:
        return inv, 1.0
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    factor = float(scaling.get("factor", 1.0))
    if kind == "default":
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind in ("dynamic", "ntk"):
        # NTK-aware base stretch for the configured context: the base grows so that the lowest frequency
        # spans `factor` times the original window while the highest is left untouched.
        old = float(scaling.get("original_max_position_embeddings") or max_position)
        length = max(float(max_position), old)
        base = theta * ((factor * length / old) - (factor - 1.0)) ** (dim / (dim - 2.0))
        return 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim)), 1.0
    if kind in ("longrope", "su"):
        old = float(scaling.get("original_max_position_embeddings") or max_position)
        long = max_position > old
        ext = torch.tensor(scaling["long_factor" if long else "short_factor"], dtype=torch.float32)
        ratio = max_position / old
        att = scaling.get("attention_factor")
        if att is None:
            att = 1.0 if ratio <= 1.0 else math.sqrt(1.0 + math.log(ratio) / math.log(old))
        return inv / ext, float(att)
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        mid = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > old / lo, inv / factor, inv)
        is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        return torch.where(is_mid, mid, out), 1.0
    if kind == "yarn":
        old = float(scaling.get("original_max_position_embeddings") or max_position)
        beta_fast, beta_slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)
        mscale, mscale_all = scaling.get("mscale"), scaling.get("mscale_all_dim")

        def get_mscale(s, m=1.0):
            return 1.0 if s <= 1 else 0.1 * m * math.log(s) + 1.0
        if scaling.get("attention_factor") is not None:
            att = float(scaling["attention_factor"])
        elif mscale and mscale_all:
            att = get_mscale(factor, mscale) / get_mscale(factor, mscale_all)
        else:
            att = get_mscale(factor)

        def corr_dim(rot):
            return dim * math.log(old / (rot * 2 * math.pi)) / (2 * math.log(theta))
        low, high = corr_dim(beta_fast), corr_dim(beta_slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
        extra = 1 - ramp
        return (inv / factor) * (1 - extra) + inv * extra, att
    raise ValueError(f"unsupported rope scaling {kind!r}")
