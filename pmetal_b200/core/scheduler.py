"""Learning-rate schedules with linear warm-up from ``min_lr``.

Values match the reference scheduler (crates/pmetal-core/src/scheduler.rs:83-146):
constant, linear, cosine, cosine-with-restarts, polynomial and warmup-stable-decay.
"""
from __future__ import annotations

import math


class LearningRateScheduler:
    def __init__(self, base_lr: float, total_steps: int, warmup_steps: int = 0, scheduler_type: str = "cosine",
                 min_lr: float = 0.0, num_restarts: int = 1, stable_ratio: float = 0.7,
                 polynomial_power: float = 1.0):
        self.base_lr = float(base_lr)
        self.min_lr = float(min_lr)
        self.total_steps = int(total_steps)
        self.warmup_steps = int(warmup_steps)
        self.scheduler_type = scheduler_type
        self.num_restarts = int(num_restarts)
        self.stable_ratio = min(max(float(stable_ratio), 0.0), 1.0)
        self.polynomial_power = max(float(polynomial_power), 0.1)
        self.current_step = 0

    @classmethod
    def from_training_config(cls, cfg, total_steps: int | None = None) -> "LearningRateScheduler":
        # total steps default to 10 000 when max_steps is unset (training_loop/mod.rs:530)
        total = total_steps if total_steps is not None else (cfg.max_steps or 10_000)
        warm = cfg.warmup_steps
        if cfg.warmup_ratio is not None:
            warm = int(total * cfg.warmup_ratio)
        return cls(cfg.learning_rate, total, warm, cfg.lr_scheduler, cfg.min_lr or 0.0,
                   cfg.cosine_num_restarts or 1, cfg.wsd_stable_ratio if cfg.wsd_stable_ratio is not None else 0.7,
                   cfg.polynomial_power or 1.0)

    def get_lr(self, step: int) -> float:
        span = self.base_lr - self.min_lr
        if step < self.warmup_steps:
            return self.min_lr + span * (step / max(self.warmup_steps, 1))
        decay_steps = max(self.total_steps - self.warmup_steps, 0)
        cur = max(step - self.warmup_steps, 0)
        if decay_steps == 0:
            return self.base_lr
        progress = min(cur / decay_steps, 1.0)
        t = self.scheduler_type
        if t == "constant":
            return self.base_lr
        if t == "linear":
            return self.min_lr + span * (1.0 - progress)
        if t == "cosine":
            return self.min_lr + span * 0.5 * (1.0 + math.cos(math.pi * progress))
        if t == "cosine_with_restarts":
            n = max(self.num_restarts, 1)
            cycle = -(-decay_steps // n)
            cp = (cur % cycle) / cycle if cycle > 0 else 0.0
            return self.min_lr + span * 0.5 * (1.0 + math.cos(math.pi * cp))
        if t == "polynomial":
            return self.min_lr + span * (1.0 - progress) ** self.polynomial_power
        if t == "wsd":
            stable = int(decay_steps * self.stable_ratio)
            if cur < stable:
                return self.base_lr
            phase = max(decay_steps - stable, 0)
            dp = min((cur - stable) / phase, 1.0) if phase > 0 else 1.0
            return self.min_lr + span * (1.0 - dp)
        raise ValueError(f"unknown scheduler {t!r}")

    def current_lr(self) -> float:
        return self.get_lr(self.current_step)

    def step(self) -> None:
        self.current_step += 1

    def set_step(self, step: int) -> None:
        self.current_step = int(step)

    def is_complete(self) -> bool:
        return self.current_step >= self.total_steps
