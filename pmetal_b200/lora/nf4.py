"""4-bit NormalFloat (NF4), FP4 and int8 block quantisation of frozen base weights (QLoRA).

Bit-exact restatement of the reference quantiser (crates/pmetal-mlx/src/quantization/nf4.rs:18-280):
blocks of ``block_size`` (64) consecutive elements of the flattened tensor, per-block absmax floored at
1e-10, values normalised to [-1, 1] and mapped to the 16-entry NF4 codebook by the 15 midpoints, two
codes per byte with the *first* element in the high nibble, optional double quantisation of the absmax
vector to 8 bits (offset = min, scale = (max - min) / 255, round-to-nearest).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

NF4_BINS = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0],
    dtype=torch.float32)
NF4_THRESHOLDS = torch.tensor([
    -0.8480964004993439, -0.6106329262256622, -0.4599952697753906, -0.33967943489551544, -0.23460740596055984,
    -0.13791173324, -0.04552501812577248, 0.03979014977812767, 0.1202552503, 0.20352125167846680,
    0.29201376438140869, 0.38931253552436829, 0.50166341662406921, 0.64278691411018372, 0.86147841811180115],
    dtype=torch.float32)
# FP4 (E2M1) magnitudes; sign in the top bit of the nibble
FP4_BINS = torch.tensor([0.0, 0.0052083333, 0.6666667, 1.0, 0.3333333, 0.5, 0.1666667, 0.25,
                         -0.0, -0.0052083333, -0.6666667, -1.0, -0.3333333, -0.5, -0.1666667, -0.25],
                        dtype=torch.float32)


@dataclass
class QuantizedTensor:
    data: torch.Tensor                  # uint8 packed codes (4-bit schemes: numel/2) or int8 values
    absmax: Optional[torch.Tensor]      # fp32 per block (None when double-quantised)
    absmax_q: Optional[torch.Tensor]    # uint8 per block
    absmax_offset: float
    absmax_scale: float
    shape: tuple
    block_size: int
    scheme: str                         # nf4 | fp4 | int8

    def block_absmax(self) -> torch.Tensor:
        if self.absmax is not None:
            return self.absmax
        return self.absmax_q.float() * self.absmax_scale + self.absmax_offset

    def nbytes(self) -> int:
        n = self.data.numel()
        n += self.absmax.numel() * 4 if self.absmax is not None else self.absmax_q.numel()
        return n

    def to(self, device) -> "QuantizedTensor":
        mv = lambda t: None if t is None else t.to(device)
        return QuantizedTensor(mv(self.data), mv(self.absmax), mv(self.absmax_q), self.absmax_offset,
                               self.absmax_scale, self.shape, self.block_size, self.scheme)


def _codes_nf4(normed: torch.Tensor) -> torch.Tensor:
    # index = number of thresholds <= value  (value < t[i] tests in the reference's decision tree)
    return torch.bucketize(normed, NF4_THRESHOLDS.to(normed.device), right=True).to(torch.uint8)


def _codes_nearest(normed: torch.Tensor, bins: torch.Tensor) -> torch.Tensor:
    return (normed[:, None] - bins.to(normed.device)[None, :]).abs().argmin(dim=1).to(torch.uint8)


def quantize(w: torch.Tensor, scheme: str = "nf4", block_size: int = 64, double_quant: bool = False) -> QuantizedTensor:
    flat = w.detach().float().reshape(-1)
    n = flat.numel()
    nb = -(-n // block_size)
    pad = nb * block_size - n
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    blocks = flat.view(nb, block_size)
    if scheme == "int8":
        absmax = blocks.abs().amax(dim=1).clamp_min(1e-10)
        q = torch.round(blocks / absmax[:, None] * 127.0).clamp(-127, 127).to(torch.int8)
        data = q.view(-1)[:n].contiguous().view(torch.uint8)
    else:
        absmax = blocks.abs().amax(dim=1).clamp_min(1e-10)
        normed = (blocks / absmax[:, None]).clamp(-1.0, 1.0).reshape(-1)
        codes = _codes_nf4(normed) if scheme == "nf4" else _codes_nearest(normed, FP4_BINS)
        codes = codes[: n + (n % 2)] if pad else codes
        if codes.numel() % 2:
            codes = torch.cat([codes, codes.new_zeros(1)])
        data = ((codes[0::2] << 4) | codes[1::2]).contiguous()
    aq, off, sc, am = None, 0.0, 0.0, absmax
    if double_quant:
        off = float(absmax.min())
        sc = (float(absmax.max()) - off) / 255.0
        aq = (torch.round((absmax - off) / sc).clamp(0, 255).to(torch.uint8) if sc > 0
              else torch.zeros_like(absmax, dtype=torch.uint8))
        am = None
    return QuantizedTensor(data, am, aq, off, sc, tuple(w.shape), block_size, scheme)


def dequantize(q: QuantizedTensor, dtype=torch.float32) -> torch.Tensor:
    """Reference dequantiser (PyTorch ops; any device)."""
    n = 1
    for s in q.shape:
        n *= s
    absmax = q.block_absmax().float()
    if q.scheme == "fp8":         # E4M3 codes with one scale per block of 128 (models/fp8.py)
        vals = q.data.view(torch.float8_e4m3fn).float().reshape(-1)
        idx = torch.arange(n, device=q.data.device) // q.block_size
        return (vals[:n] * absmax[idx]).view(q.shape).to(dtype)
    if q.scheme == "int8":
        vals = q.data.view(torch.int8).float() / 127.0
    else:
        bins = (NF4_BINS if q.scheme == "nf4" else FP4_BINS).to(q.data.device)
        hi, lo = (q.data >> 4).long(), (q.data & 0xF).long()
        vals = torch.stack([bins[hi], bins[lo]], dim=1).reshape(-1)[:n]
    idx = torch.arange(n, device=q.data.device) // q.block_size
    return (vals[:n] * absmax[idx]).view(q.shape).to(dtype)
