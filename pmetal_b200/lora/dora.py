"""DoRA — weight-decomposed low-rank adaptation (crates/pmetal-lora/src/dora.rs:20-330).

``W' = m * (W + s B A) / ||W + s B A||_row`` with a trainable magnitude ``m`` per output row initialised to the row norms
of ``W``. The norm is treated as a constant in the backward pass (detached), as in the reference and the paper's
recommended variant, so the extra cost is one row-norm of the merged weight per step.

``attach_dora`` adds ``dora_magnitude`` to every projection group that has LoRA factors and routes its forward through
the decomposed form: y = (m / n) * (x W^T + s (x A^T) B^T), which reuses the fused base+LoRA GEMM and applies the row
scale to its output."""
from __future__ import annotations

import torch
import torch.nn as nn


def row_norms(fl) -> torch.Tensor:
    """||W + s B A|| per output row, fp32, no graph."""
    with torch.no_grad():
        return fl.merged_weight().float().norm(dim=1).clamp(min=1e-8)


def attach_dora(model) -> int:
    n = 0
    for _, _, fl in model.fused_linears():
        if fl.lora_a is None or getattr(fl, "dora_magnitude", None) is not None:
            continue
        fl.dora_magnitude = nn.Parameter(row_norms(fl).to(fl.lora_a.device))
        base_forward = fl.forward

        def forward(x, residual=None, _fl=fl, _base=base_forward):
            y = _base(x, None)
            scale = (_fl.dora_magnitude / row_norms(_fl).to(_fl.dora_magnitude.device)).to(y.dtype)
            y = y * scale
            return y if residual is None else y + residual
        fl.forward = forward
        n += 1
    return n


def merged_dora_weight(fl) -> torch.Tensor:
    w = fl.merged_weight().float()
    return w * (fl.dora_magnitude.detach().float() / w.norm(dim=1).clamp(min=1e-8))[:, None]
