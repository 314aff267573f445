"""Sanity checks on freshly merged tensors, before anything is written (crates/pmetal-merge/src/sanity.rs:28-200).

Levels: ``off``; ``quick`` counts NaN and infinite values; ``full`` adds mean, population standard deviation, largest
magnitude and the fraction of exact zeros, and flags outliers (|mean| > 10 or std > 100). A tensor with a NaN or an
infinity fails the merge at once, so no poisoned shard reaches the disk."""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import List, Optional

import torch

LEVELS = ("off", "quick", "full")


@dataclass
class MergedTensorReport:
    name: str
    shape: List[int]
    n_elements: int
    n_nan: int
    n_inf: int
    mean: Optional[float] = None
    std: Optional[float] = None
    abs_max: Optional[float] = None
    sparsity: Optional[float] = None

    def is_corrupt(self) -> bool:
        return self.n_nan > 0 or self.n_inf > 0

    def is_outlier(self) -> bool:
        return self.mean is not None and (abs(self.mean) > 10.0 or (self.std or 0.0) > 100.0)

    def to_dict(self) -> dict:
        return asdict(self)


def check_tensor(name: str, tensor: torch.Tensor, level: str = "quick") -> Optional[MergedTensorReport]:
    """Report for one tensor (None at level ``off``); raises ``ValueError`` when it holds a NaN or an infinity."""
    if level not in LEVELS:
        raise ValueError(f"sanity level must be one of {LEVELS}")
    if level == "off":
        return None
    t = tensor.detach().float()
    rep = MergedTensorReport(name, list(t.shape), t.numel(), int(torch.isnan(t).sum()), int(torch.isinf(t).sum()))
    if rep.is_corrupt():
        raise ValueError(f"merged tensor {name} holds {rep.n_nan} NaN and {rep.n_inf} infinite values")
    if level == "full" and t.numel():
        rep.mean, rep.std = float(t.mean()), float(t.std(unbiased=False))
        rep.abs_max, rep.sparsity = float(t.abs().max()), float((t == 0).float().mean())
    return rep
