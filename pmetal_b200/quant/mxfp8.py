"""MXFP8 block quantisation: 32 values share one power-of-two scale (E8M0 byte), elements are FP8 E4M3.

The second mode of the reference's ``quantize_mode`` (affine | mxfp8, crates/pmetal-bridge/cpp/bridge_training.cpp:249-291).
Layout: ``codes`` uint8 [..., K] holding E4M3 bit patterns and ``scales`` uint8 [..., K/32] holding the biased exponent
e (value 2^(e - 127)), as in the OCP microscaling specification. The scale is the smallest power of two that keeps the
block's absolute maximum within the E4M3 range: e = ceil(log2(amax / 448)) + 127, so nothing saturates."""
from __future__ import annotations

from typing import Tuple

import torch

BLOCK = 32
E4M3_MAX = 448.0


def quantize_mxfp8(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """float tensor [..., K] (K a multiple of 32) -> (codes uint8 [..., K], scales uint8 [..., K/32])."""
    if w.shape[-1] % BLOCK:
        raise ValueError(f"last dimension {w.shape[-1]} is not a multiple of {BLOCK}")
    x = w.float().reshape(*w.shape[:-1], -1, BLOCK)
    amax = x.abs().amax(-1, keepdim=True)
    e = torch.ceil(torch.log2(amax.clamp_min(2.0 ** -127) / E4M3_MAX))      # smallest power of two with amax / 2^e <= 448
    e = e.clamp(-127, 127)
    scaled = (x * torch.exp2(-e)).clamp(-E4M3_MAX, E4M3_MAX)
    codes = scaled.to(torch.float8_e4m3fn).view(torch.uint8).reshape(w.shape)
    scales = (e.squeeze(-1) + 127).to(torch.uint8)
    scales = torch.where(amax.squeeze(-1) == 0, torch.zeros_like(scales), scales)
    return codes, scales


def dequantize_mxfp8(codes: torch.Tensor, scales: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    x = codes.view(torch.float8_e4m3fn).float().reshape(*codes.shape[:-1], -1, BLOCK)
    s = torch.exp2(scales.float() - 127.0).unsqueeze(-1)
    return (x * s).reshape(codes.shape).to(dtype)


def quantize_mode(w: torch.Tensor, mode: str = "affine", bits: int = 4, group_size: int = 64):
    """``affine`` -> (packed, scales, biases) of :mod:`mlx_affine`; ``mxfp8`` -> (codes, scales)."""
    if mode == "mxfp8":
        return quantize_mxfp8(w)
    if mode == "affine":
        from .mlx_affine import pack_bits, quantize_affine
        q, scales, biases = quantize_affine(w, bits, group_size)
        return pack_bits(q, bits), scales, biases
    raise ValueError(f"unknown quantisation mode {mode!r} (affine | mxfp8)")
