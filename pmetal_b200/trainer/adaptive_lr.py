"""Adaptive learning-rate controller and runtime control file.

Behaviour follows crates/pmetal-trainer/src/adaptive_lr.rs:112-1061: an EMA (0.97) of the loss with
variance tracking; a z-score spike (> 3.5 sigma) multiplies the LR by 0.3 for a 10-step cooldown; a
plateau (no improvement >= 1e-4 for 100 steps) halves it, at most 5 times; a positive loss slope over
two consecutive 40-step windows (divergence) multiplies it by 0.7 with an 80-step cooldown, at most 4
times; nothing fires during the warm-up grace (first 30 % of training); with rollback enabled (LoRA
preset: on, max 3, x0.5) a divergence first restores the best snapshot; when every budget is used the
run stops early. The file ``.lr_control.json`` is polled every 10 steps for
``{"action": "set_lr"|"reduce_lr"|"reset_lr"|"save_checkpoint"|"graceful_stop", ...}`` and removed
once consumed. NaN/inf losses are treated as spikes.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Optional


@dataclass
class AdaptiveLrConfig:
    enabled: bool = True
    ema_alpha: float = 0.97
    spike_threshold: float = 3.5
    spike_cooldown_steps: int = 10
    spike_reduction_factor: float = 0.3
    plateau_patience: int = 100
    plateau_factor: float = 0.5
    plateau_min_delta: float = 1e-4
    plateau_max_reductions: int = 5
    divergence_window: int = 40
    divergence_factor: float = 0.7
    divergence_slope_threshold: float = 0.005
    divergence_confirmation: int = 2
    divergence_cooldown_steps: int = 80
    max_divergence_reductions: int = 4
    min_lr: float = 1e-7
    control_poll_interval: int = 10
    rollback_enabled: bool = False
    max_rollbacks: int = 5
    rollback_lr_factor: float = 0.5
    warmup_fraction: float = 0.30

    @classmethod
    def for_lora(cls) -> "AdaptiveLrConfig":
        return cls(rollback_enabled=True, warmup_fraction=0.30, max_rollbacks=3, rollback_lr_factor=0.5)

    @classmethod
    def for_distillation(cls) -> "AdaptiveLrConfig":
        return cls(spike_threshold=3.0, spike_cooldown_steps=15, plateau_patience=50, divergence_window=30,
                   divergence_slope_threshold=0.003, divergence_cooldown_steps=60, warmup_fraction=0.15)


class AdaptiveLrController:
    def __init__(self, config: Optional[AdaptiveLrConfig] = None, total_steps: int = 10_000,
                 control_file: Optional[str] = None):
        self.cfg = config or AdaptiveLrConfig()
        self.total_steps = total_steps
        self.control_file = control_file
        self.ema: Optional[float] = None
        self.var = 0.0
        self.scale = 1.0                 # multiplicative factor applied to the scheduled LR
        self.manual_lr: Optional[float] = None
        self.spike_cooldown = 0
        self.best_ema = math.inf
        self.since_best = 0
        self.plateau_reductions = 0
        self.window: list = []
        self.prev_window_mean: Optional[float] = None
        self.diverging_windows = 0
        self.divergence_cooldown = 0
        self.divergence_reductions = 0
        self.rollbacks = 0
        self.n = 0

    @classmethod
    def lora_preset(cls, control_file: Optional[str] = None, total_steps: int = 10_000) -> "AdaptiveLrController":
        return cls(AdaptiveLrConfig.for_lora(), total_steps, control_file)

    # ------------------------------------------------------------------ control file
    def poll_control(self) -> Optional[dict]:
        p = self.control_file
        if not p or not os.path.exists(p):
            return None
        try:
            with open(p, "r", encoding="utf-8") as fh:
                cmd = json.load(fh)
            os.remove(p)
        except (OSError, ValueError):
            return None
        return cmd if isinstance(cmd, dict) and "action" in cmd else None

    # ------------------------------------------------------------------ per-step observation
    def effective_lr(self, scheduled: float) -> float:
        if self.manual_lr is not None:
            return max(self.manual_lr, self.cfg.min_lr)
        return max(scheduled * self.scale, self.cfg.min_lr)

    def observe(self, step: int, loss: float, scheduled_lr: float) -> Optional[dict]:
        """Feed one loss value; returns an action dict for the training loop or None."""
        c = self.cfg
        if not c.enabled:
            return None
        self.n += 1
        if c.control_poll_interval and step % c.control_poll_interval == 0:
            cmd = self.poll_control()
            if cmd:
                a = cmd["action"]
                if a == "set_lr":
                    self.manual_lr = float(cmd["value"])
                    return {"action": "set_lr", "lr": self.effective_lr(scheduled_lr)}
                if a == "reduce_lr":
                    self.scale *= float(cmd.get("factor", 0.5))
                    return {"action": "set_lr", "lr": self.effective_lr(scheduled_lr)}
                if a == "reset_lr":
                    self.manual_lr, self.scale = None, 1.0
                    return {"action": "reset_lr"}
                if a in ("save_checkpoint", "graceful_stop"):
                    return {"action": a}
        bad = not math.isfinite(loss)
        in_warmup = step < c.warmup_fraction * self.total_steps
        action = None
        if self.ema is None:
            if bad:
                return None
            self.ema = loss
            self.best_ema = loss
            return None
        std = math.sqrt(max(self.var, 1e-12))
        z = (loss - self.ema) / std if (std > 1e-6 and not bad) else (math.inf if bad else 0.0)
        # ---- spike
        if self.spike_cooldown > 0:
            self.spike_cooldown -= 1
            if self.spike_cooldown == 0 and self._spiked:
                self.scale /= c.spike_reduction_factor
                self._spiked = False
                action = {"action": "set_lr", "lr": self.effective_lr(scheduled_lr)} if self.scale != 1.0 or self.manual_lr else {"action": "reset_lr"}
        elif (z > c.spike_threshold or bad) and not in_warmup and self.n > 10:
            self.scale *= c.spike_reduction_factor
            self.spike_cooldown = c.spike_cooldown_steps
            self._spiked = True
            action = {"action": "set_lr", "lr": self.effective_lr(scheduled_lr), "reason": "spike"}
        if bad:
            return action
        # ---- EMA update (spikes are not folded into the statistics)
        if not (z > c.spike_threshold):
            d = loss - self.ema
            self.ema += (1 - c.ema_alpha) * d
            self.var = c.ema_alpha * (self.var + (1 - c.ema_alpha) * d * d)
        # ---- best tracking / plateau
        if self.ema < self.best_ema - c.plateau_min_delta:
            self.best_ema, self.since_best = self.ema, 0
            if c.rollback_enabled and not in_warmup and action is None:
                action = {"action": "snapshot"}
        else:
            self.since_best += 1
            if (self.since_best >= c.plateau_patience and not in_warmup
                    and self.plateau_reductions < c.plateau_max_reductions):
                self.scale *= c.plateau_factor
                self.plateau_reductions += 1
                self.since_best = 0
                action = {"action": "set_lr", "lr": self.effective_lr(scheduled_lr), "reason": "plateau"}
        # ---- divergence: slope between consecutive window means
        self.window.append(loss)
        if self.divergence_cooldown > 0:
            self.divergence_cooldown -= 1
        if len(self.window) >= c.divergence_window:
            mean = sum(self.window) / len(self.window)
            self.window = []
            if self.prev_window_mean is not None and not in_warmup and self.divergence_cooldown == 0:
                slope = (mean - self.prev_window_mean) / max(abs(self.prev_window_mean), 1e-8)
                self.diverging_windows = self.diverging_windows + 1 if slope > c.divergence_slope_threshold else 0
                if self.diverging_windows >= c.divergence_confirmation:
                    self.diverging_windows = 0
                    self.divergence_cooldown = c.divergence_cooldown_steps
                    if c.rollback_enabled and self.rollbacks < c.max_rollbacks:
                        self.rollbacks += 1
                        self.scale *= c.rollback_lr_factor
                        action = {"action": "rollback", "lr": self.effective_lr(scheduled_lr)}
                    elif self.divergence_reductions < c.max_divergence_reductions:
                        self.divergence_reductions += 1
                        self.scale *= c.divergence_factor
                        action = {"action": "set_lr", "lr": self.effective_lr(scheduled_lr), "reason": "divergence"}
                    else:
                        action = {"action": "early_stop", "reason": "divergence budget exhausted"}
            self.prev_window_mean = mean
        if action and action.get("action") == "set_lr" and self.scale == 1.0 and self.manual_lr is None:
            action = {"action": "reset_lr"}
        return action

    _spiked = False
