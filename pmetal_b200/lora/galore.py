"""GaLore gradient low-rank projection and NEFTune embedding noise.

* ``GaLoreProjector`` (crates/pmetal-lora/src/galore.rs): every ``update_gap`` steps the projection basis of a 2-D
  gradient is refreshed from its truncated SVD; the optimiser runs on the projected gradient ``P^T G`` (or ``G Q``) and the
  update is projected back and scaled.
* ``neftune_noise`` (crates/pmetal-mlx NEFTune): uniform noise of magnitude alpha / sqrt(L * d) added to input embeddings
  during training."""
from __future__ import annotations

import math
from typing import Optional

import torch


class GaLoreProjector:
    def __init__(self, rank: int = 128, update_gap: int = 200, scale: float = 0.25, proj_type: str = "std"):
        self.rank, self.update_gap, self.scale, self.proj_type = rank, update_gap, scale, proj_type
        self.ortho: Optional[torch.Tensor] = None
        self.step = 0
        self.left = True

    def _refresh(self, g: torch.Tensor) -> None:
        m, n = g.shape
        self.left = (m <= n) if self.proj_type == "std" else (self.proj_type == "left")
        u, _, vh = torch.linalg.svd(g.float(), full_matrices=False)
        r = min(self.rank, min(m, n))
        self.ortho = u[:, :r].contiguous() if self.left else vh[:r].contiguous()

    def project(self, g: torch.Tensor) -> torch.Tensor:
        if self.ortho is None or self.step % self.update_gap == 0:
            self._refresh(g)
        self.step += 1
        return self.ortho.t() @ g.float() if self.left else g.float() @ self.ortho.t()

    def project_back(self, low: torch.Tensor) -> torch.Tensor:
        full = self.ortho @ low if self.left else low @ self.ortho
        return full * self.scale


def neftune_noise(embeddings: torch.Tensor, alpha: float = 5.0, training: bool = True,
                  generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """embeddings [..., L, d]."""
    if not training or alpha <= 0:
        return embeddings
    L, d = embeddings.shape[-2], embeddings.shape[-1]
    mag = alpha / math.sqrt(L * d)
    noise = (torch.rand(embeddings.shape, device=embeddings.device, generator=generator) * 2 - 1) * mag
    return embeddings + noise.to(embeddings.dtype)
