"""TurboQuant-style KV-cache compression: random rotation + Lloyd-Max scalar codebooks (+ optional 1-bit QJL residual).

The reference compresses keys/values 4-6x with ~45 JIT Metal kernels (crates/pmetal-bridge/src/turboquant/* — rotation,
Lloyd-Max codebooks, QJL, host/GPU key stores; cpp/bridge_turboquant_*.cpp). The algorithm restated here:

1. a vector x in R^d (d a power of two) is scaled to unit norm and rotated by a random signed Walsh-Hadamard transform
   R = H D / sqrt(d) (D = random +-1 diagonal); after rotation every coordinate is close to N(0, 1/d);
2. each coordinate is quantised with the Lloyd-Max codebook of the standard normal at b bits (b = 1..4), computed once by
   Lloyd iterations; codes are bit-packed; the norm is kept in fp16;
3. optionally the quantisation residual is sketched with a 1-bit Johnson-Lindenstrauss transform (sign of a second random
   rotation, plus the residual norm), which makes inner-product estimates unbiased: <q, x> ~ <q, x_hat> + <q, r_hat>;
4. attention scores against compressed keys are computed in the rotated domain (rotate the query once), so keys are never
   de-rotated; values are de-rotated after the weighted sum.
The encode / decode / score paths are PyTorch tensor programs; a fused quantised-KV decode-attention kernel is not built."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised fast Walsh-Hadamard transform along the last dimension (power of two)."""
    d = x.shape[-1]
    assert d & (d - 1) == 0, "dimension must be a power of two"
    y = x.clone()
    h = 1
    while h < d:
        y = y.view(*x.shape[:-1], d // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], dim=-2).reshape(*x.shape)
        h *= 2
    return y


def lloyd_max_normal(bits: int, iters: int = 200) -> Tuple[torch.Tensor, torch.Tensor]:
    """(centroids [2^b], decision thresholds [2^b - 1]) of the MSE-optimal quantiser for N(0, 1)."""
    n = 1 << bits
    c = torch.linspace(-2.0, 2.0, n, dtype=torch.float64)
    sq2 = math.sqrt(2.0)

    def pdf(t):
        return torch.exp(-0.5 * t * t) / math.sqrt(2 * math.pi)

    def cdf(t):
        return 0.5 * (1 + torch.erf(t / sq2))
    for _ in range(iters):
        t = (c[:-1] + c[1:]) / 2
        lo = torch.cat([torch.tensor([-float("inf")], dtype=torch.float64), t])
        hi = torch.cat([t, torch.tensor([float("inf")], dtype=torch.float64)])
        mass = (cdf(hi) - cdf(lo)).clamp(min=1e-300)
        c = (pdf(lo) - pdf(hi)) / mass              # E[x | lo < x < hi]
    return c.float(), ((c[:-1] + c[1:]) / 2).float()


def pack_bits(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 codes [..., d] with values < 2^bits -> packed uint8 [..., d * bits / 8]."""
    d = codes.shape[-1]
    per = 8 // bits
    c = codes.view(*codes.shape[:-1], d // per, per).to(torch.int32)
    shifts = torch.arange(per, device=codes.device, dtype=torch.int32) * bits
    return (c << shifts).sum(-1).to(torch.uint8)


def unpack_bits(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    per = 8 // bits
    shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
    c = (packed.to(torch.int32)[..., None] >> shifts) & ((1 << bits) - 1)
    return c.reshape(*packed.shape[:-1], d).to(torch.uint8)


@dataclass
class Compressed:
    codes: torch.Tensor              # packed uint8 [..., d * bits / 8]
    norm: torch.Tensor               # fp16 [...]
    qjl: Optional[torch.Tensor] = None       # packed sign bits of the rotated residual [..., d / 8]
    res_norm: Optional[torch.Tensor] = None  # fp16 [...]

    def nbytes(self) -> int:
        n = self.codes.numel() + 2 * self.norm.numel()
        if self.qjl is not None:
            n += self.qjl.numel() + 2 * self.res_norm.numel()
        return n


class TurboQuant:
    def __init__(self, dim: int, bits: int = 4, qjl: bool = False, seed: int = 0, device="cpu"):
        assert bits in (1, 2, 4), "bit widths that divide a byte"
        self.d, self.bits, self.use_qjl = dim, bits, qjl
        g = torch.Generator().manual_seed(seed)
        self.sign = (torch.randint(0, 2, (dim,), generator=g) * 2 - 1).float().to(device)
        self.sign2 = (torch.randint(0, 2, (dim,), generator=g) * 2 - 1).float().to(device)
        c, t = lloyd_max_normal(bits)
        self.centroids, self.thresholds = c.to(device), t.to(device)

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return fwht(x.float() * self.sign) / math.sqrt(self.d)

    def unrotate(self, y: torch.Tensor) -> torch.Tensor:
        return fwht(y.float()) / math.sqrt(self.d) * self.sign

    def encode(self, x: torch.Tensor) -> Compressed:
        norm = x.float().norm(dim=-1)
        y = self.rotate(x) / norm.clamp(min=1e-12)[..., None] * math.sqrt(self.d)       # ~ N(0, 1) per coordinate
        codes = torch.bucketize(y, self.thresholds).to(torch.uint8)
        out = Compressed(pack_bits(codes, self.bits), norm.to(torch.float16))
        if self.use_qjl:
            res = y - self.centroids[codes.long()]
            s = fwht(res * self.sign2) / math.sqrt(self.d)
            out.qjl = pack_bits((s >= 0).to(torch.uint8), 1)
            out.res_norm = res.norm(dim=-1).to(torch.float16)
        return out

    def decode_rotated(self, c: Compressed) -> torch.Tensor:
        """Reconstruction in the rotated domain, scaled back to the original norm."""
        y = self.centroids[unpack_bits(c.codes, self.bits, self.d).long()]
        if c.qjl is not None:
            s = unpack_bits(c.qjl, 1, self.d).float() * 2 - 1
            # E[|g|] = sqrt(2/pi) for a unit-variance coordinate: the sign sketch scaled by the residual norm is an
            # unbiased estimate of the residual's direction in expectation over the second rotation
            r = fwht(s) / math.sqrt(self.d) * self.sign2 * (c.res_norm.float()[..., None] * math.sqrt(math.pi / 2) / math.sqrt(self.d))
            y = y + r
        return y * (c.norm.float()[..., None] / math.sqrt(self.d))

    def decode(self, c: Compressed) -> torch.Tensor:
        return self.unrotate(self.decode_rotated(c))

    def scores(self, q: torch.Tensor, keys: Compressed) -> torch.Tensor:
        """<q, k> for every compressed key without de-rotating the keys: q [..., d] -> [..., n_keys]."""
        return self.rotate(q) @ self.decode_rotated(keys).transpose(-1, -2)

    def attention(self, q: torch.Tensor, keys: Compressed, values: Compressed, scale: float) -> torch.Tensor:
        """Single-head decode attention over compressed K and V: q [nq, d] -> [nq, d]."""
        p = torch.softmax(self.scores(q, keys) * scale, -1)
        return self.unrotate(p @ self.decode_rotated(values))

    def compression_ratio(self, c: Compressed, n_vectors: int) -> float:
        return n_vectors * self.d * 2 / c.nbytes()
