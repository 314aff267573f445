"""Knowledge-distillation trainer: online (teacher forward every step), offline (cached, compressed teacher logits) and
progressive (temperature annealed from ``temperature`` to ``final_temperature``).

loss = alpha * soft(student, teacher; T) + (1 - alpha) * CE(student, labels); defaults alpha 0.5, T 2.0 as in the
reference CLI (crates/pmetal/src/cli/distill.rs; trainer crates/pmetal-trainer/src/distillation.rs, config
crates/pmetal-distill/src/config.rs). On CUDA the soft term of the KL family runs through the fused chunked kernel, so
neither model's full logits are materialised."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import losses as L
from .offline import LogitCache
from .taid import TaidConfig, TaidDistiller


@dataclass
class DistillConfig:
    method: str = "online"            # online | offline | progressive
    loss_type: str = "kl"             # any key of losses.LOSSES, or "taid"
    alpha: float = 0.5
    temperature: float = 2.0
    final_temperature: float = 1.0
    hidden_loss_weight: float = 0.0
    hidden_loss_kind: str = "mse"
    learning_rate: float = 2e-5
    max_grad_norm: float = 1.0
    total_steps: int = 1000
    chunk: int = 2048
    cache_dir: Optional[str] = None
    rationale: bool = False           # entropy-weighted KL that stresses the reasoning tokens
    rationale_weight: float = 1.0
    reasoning_markers: Optional[tuple] = None   # (start token id, end token id): only tokens inside the span count


class DistillTrainer:
    def __init__(self, student, teacher, cfg: DistillConfig, optimizer=None, taid: Optional[TaidConfig] = None):
        from ..trainer.optimizer import FlatAdamW, attach_shadows
        self.student, self.teacher, self.cfg = student, teacher, cfg
        self.device = next(student.parameters()).device
        shadow = torch.bfloat16 if (self.device.type == "cuda" and self._fast(student)) else None
        self.opt = optimizer or FlatAdamW(student.named_parameters(), lr=cfg.learning_rate, weight_decay=0.0,
                                          max_grad_norm=cfg.max_grad_norm, shadow_dtype=shadow)
        if shadow is not None:
            attach_shadows(student, self.opt)
        self.taid = TaidDistiller(taid or TaidConfig(temperature=cfg.temperature)) if cfg.loss_type == "taid" else None
        self.cache = LogitCache.load(cfg.cache_dir) if (cfg.method == "offline" and cfg.cache_dir) else None
        self.step_count = 0

    def temperature(self) -> float:
        c = self.cfg
        if c.method != "progressive":
            return c.temperature
        p = min(self.step_count / max(c.total_steps, 1), 1.0)
        return c.temperature + (c.final_temperature - c.temperature) * p

    @staticmethod
    def _fast(model) -> bool:
        """The hand-written decoder (flat token batches, ``head_weight``); everything else is a config-driven architecture
        that takes [batch, tokens] and applies its own read-out (logit scale, soft cap) in ``logits``."""
        return hasattr(model, "head_weight") and hasattr(model, "fused_linears")

    def _hidden(self, model, ids, grad):
        T = ids.numel()
        with (torch.enable_grad() if grad else torch.no_grad()):
            if not self._fast(model):
                return model.forward_hidden(ids.reshape(1, -1))[0]
            pos = torch.arange(T, dtype=torch.int32, device=ids.device)
            cu = torch.tensor([0, T], dtype=torch.int32, device=ids.device)
            return model.forward_hidden(ids.reshape(-1), pos, cu, torch.zeros(T, dtype=torch.int32, device=ids.device))

    def _logits(self, model, h):
        if self._fast(model):
            return h.float() @ model.head_weight().float().t()
        return model.logits(h).float()

    def loss(self, input_ids: torch.Tensor, labels: torch.Tensor, seq_id: Optional[int] = None):
        """One sequence [T] (callers pack or loop). Labels -100 are ignored; position t predicts labels[t+1]."""
        c = self.cfg
        T = self.temperature()
        hs = self._hidden(self.student, input_ids, True)[:-1]
        tgt = labels.reshape(-1)[1:]
        mask = tgt != -100
        both_fast = self._fast(self.student) and self._fast(self.teacher)
        ws = self.student.head_weight() if self._fast(self.student) else None
        stats = {}
        if self.cache is not None and seq_id is not None and self.cache.has_sequence(seq_id):
            t_logits = self.cache.load_sequence(seq_id).to(self.device)[:-1]
            soft = L.LOSSES[c.loss_type](self._logits(self.student, hs), t_logits, T, mask)
        else:
            ht = self._hidden(self.teacher, input_ids, False)[:-1]
            if c.rationale:
                tw = None
                if c.reasoning_markers is not None:
                    span = L.reasoning_mask(input_ids.reshape(-1), *c.reasoning_markers)[1:]
                    tw = span if bool(span.any()) else None
                soft = L.rationale_kl(self._logits(self.student, hs), self._logits(self.teacher, ht), T, mask,
                                      c.rationale_weight, tw)
            elif self.taid is not None:
                s_logits = self._logits(self.student, hs).unsqueeze(0)
                t_logits = self._logits(self.teacher, ht).unsqueeze(0)
                soft, a = self.taid.loss(t_logits, s_logits, self.step_count, c.total_steps, mask=mask.unsqueeze(0))
                stats["taid_alpha"] = a
            elif both_fast and c.loss_type in ("kl", "forward_kl", "reverse_kl", "js", "jsd", "soft_ce", "tvd"):
                soft = L.fused_kd_loss(hs, ws, ht, self.teacher.head_weight(), mask, T, c.loss_type, 0.5, c.chunk)
            else:
                soft = L.LOSSES[c.loss_type](self._logits(self.student, hs), self._logits(self.teacher, ht), T, mask)
            if c.hidden_loss_weight > 0 and hs.shape[-1] == ht.shape[-1]:
                soft = soft + c.hidden_loss_weight * L.hidden_state_loss(hs, ht, c.hidden_loss_kind, mask=mask)
        from ..ops import functional as ops
        if not mask.any():
            hard = hs.sum() * 0
        elif ws is not None:
            hard = ops.causal_lm_loss(hs, ws, tgt)
        else:
            hard = torch.nn.functional.cross_entropy(self._logits(self.student, hs), tgt, ignore_index=-100)
        total = c.alpha * soft + (1 - c.alpha) * hard
        stats.update(soft=float(soft.detach()), hard=float(hard.detach()), temperature=T)
        return total, stats

    def step(self, input_ids, labels, seq_id: Optional[int] = None) -> dict:
        self.opt.zero_grad()
        loss, stats = self.loss(input_ids.to(self.device), labels.to(self.device), seq_id)
        loss.backward()
        gn = self.opt.step(1.0)
        self.step_count += 1
        stats.update(loss=float(loss.detach()), grad_norm=float(gn))
        return stats

    @torch.no_grad()
    def build_cache(self, sequences, cache_dir: str, compression: str = "topk", top_k: int = 64) -> LogitCache:
        cache = LogitCache(cache_dir, compression, top_k)
        for i, ids in enumerate(sequences):
            ids = torch.as_tensor(ids, dtype=torch.int64, device=self.device)
            h = self._hidden(self.teacher, ids, False)
            cache.cache_sequence(i, self._logits(self.teacher, h))
        cache.save_metadata()
        return cache
