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
    """||W + s B A|| per output row, fp32, no graph.

    The merged weight is never formed. Per row, with G = A A^T (r x r):
        ||W + s B A||^2 = ||W||^2 + 2 s (W A^T) . B + s^2 B G B^T
    ``||W||^2`` is computed once (the base is frozen); ``W A^T`` is one skinny product per segment that reads W once
    in its stored precision. The result is cached until a factor changes (``_version`` of the two parameters), so
    gradient-accumulation micro-steps and evaluation passes reuse it."""
    with torch.no_grad():
        a, b = fl.lora_a, fl.lora_b
        key = (a._version, b._version, a.data_ptr(), b.data_ptr())
        hit = getattr(fl, "_dora_norm_cache", None)
        if hit is not None and hit[0] == key:
            return hit[1]
        if getattr(fl, "qweight", None) is not None:              # packed base: expand once for this computation
            from .nf4 import dequantize
            w = dequantize(fl.qweight, torch.float32)
            w_sq = (w * w).sum(1)
        else:
            w = fl.weight.detach()
            w_sq = getattr(fl, "_dora_w_sq", None)
            if w_sq is None or w_sq.device != w.device:
                w_sq = fl._dora_w_sq = (w.float() ** 2).sum(1)
        out = w_sq.clone()
        o = 0
        for i, sz in enumerate(fl.seg_sizes):
            ai = a[i * fl.r:(i + 1) * fl.r].detach()
            bi = b[o:o + sz].detach().float()
            wa = (w[o:o + sz] @ ai.to(w.dtype).t()).float()                     # [sz, r]
            g = ai.float() @ ai.float().t()                                     # [r, r]
            out[o:o + sz] += 2.0 * fl.scale * (wa * bi).sum(1) + fl.scale ** 2 * ((bi @ g) * bi).sum(1)
            o += sz
        n = out.clamp(min=0).sqrt().clamp(min=1e-8)
        fl._dora_norm_cache = (key, n)
        return n


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
