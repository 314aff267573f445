"""TAID — temporally adaptive interpolated distillation (crates/pmetal-distill/src/taid.rs:64-580).

The student is trained against ``p_I = alpha p_T + (1 - alpha) p_S`` (student term detached). ``alpha`` follows a
schedule from ``initial_alpha`` to ``final_alpha`` (linear / cosine / exponential / 4-step / constant, clamped) and is
raised per sample by difficulty: ``alpha_i = base + sigmoid(scale * KL_i(p_T || p_S) - 5) * (max_alpha - base)``."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class TaidConfig:
    initial_alpha: float = 0.9
    final_alpha: float = 0.5
    schedule: str = "cosine"          # linear | cosine | exponential | step | constant
    temperature: float = 2.0
    difficulty_aware: bool = True
    difficulty_scale: float = 0.2
    min_alpha: float = 0.1
    max_alpha: float = 0.99
    loss_type: str = "kl"             # kl | ce
    hard_target_weight: float = 0.0


class TaidDistiller:
    def __init__(self, cfg: TaidConfig = TaidConfig()):
        self.cfg = cfg

    def base_alpha(self, step: int, total_steps: int) -> float:
        c = self.cfg
        if total_steps == 0:
            return c.initial_alpha
        p = step / total_steps
        rng = c.initial_alpha - c.final_alpha
        if c.schedule == "linear":
            a = c.initial_alpha - rng * p
        elif c.schedule == "cosine":
            a = c.final_alpha + rng * 0.5 * (1 + math.cos(math.pi * p))
        elif c.schedule == "exponential":
            a = c.initial_alpha * math.exp(math.log(c.final_alpha / c.initial_alpha) * p)
        elif c.schedule == "step":
            a = (c.initial_alpha if p < 0.25 else c.initial_alpha - rng * 0.33 if p < 0.5
                 else c.initial_alpha - rng * 0.66 if p < 0.75 else c.final_alpha)
        else:
            a = c.initial_alpha
        return min(max(a, c.min_alpha), c.max_alpha)

    def difficulty_alpha(self, pt: torch.Tensor, ps: torch.Tensor, base: float) -> torch.Tensor:
        """pt, ps: [B, T, V] probabilities. Returns per-sample alpha [B]."""
        c = self.cfg
        if not c.difficulty_aware:
            return torch.full((pt.shape[0],), base, device=pt.device)
        kl = (pt * torch.log(pt / (ps + 1e-10) + 1e-30)).sum(-1).sum(-1)
        nd = torch.sigmoid(c.difficulty_scale * kl - 5.0)
        return (base + nd * (c.max_alpha - base)).clamp(c.min_alpha, c.max_alpha)

    def loss(self, teacher_logits, student_logits, step: int, total_steps: int, labels=None, mask=None):
        """Logits [B, T, V]. Returns (loss, mean alpha)."""
        c = self.cfg
        T = c.temperature
        ls = F.log_softmax(student_logits.float() / T, -1)
        pt = F.softmax(teacher_logits.float() / T, -1)
        ps = ls.exp()
        alpha = self.difficulty_alpha(pt, ps.detach(), self.base_alpha(step, total_steps))
        a = alpha.view(-1, 1, 1)
        target = a * pt + (1 - a) * ps.detach()
        if c.loss_type == "ce":
            per = -(target * ls).sum(-1)
        else:
            per = (target * (torch.log(target.clamp(min=1e-30)) - ls)).sum(-1)
        if mask is not None:
            m = mask.to(per.dtype)
            soft = (per * m).sum() / m.sum().clamp(min=1)
        else:
            soft = per.mean()
        loss = soft * T * T
        if c.hard_target_weight > 0 and labels is not None:
            hard = F.cross_entropy(student_logits.float().reshape(-1, student_logits.shape[-1]), labels.reshape(-1),
                                   ignore_index=-100)
            loss = (1 - c.hard_target_weight) * loss + c.hard_target_weight * hard
        return loss, float(alpha.mean())
