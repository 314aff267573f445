"""Metric records passed to callbacks (reference: crates/pmetal-core/src/types.rs:170-290)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class StepMetrics:
    step: int = 0
    epoch: int = 0
    total_epochs: int = 0
    total_steps: int = 0
    loss: float = 0.0
    lr: float = 0.0
    tok_sec: float = 0.0
    # The four Apple-Neural-Engine timing fields of the reference record are kept
    # (always 0.0 here) so that consumers of the JSONL stream see the same keys.
    ane_fwd_ms: float = 0.0
    ane_bwd_ms: float = 0.0
    rmsnorm_ms: float = 0.0
    cblas_ms: float = 0.0
    adam_ms: float = 0.0
    total_ms: float = 0.0
    tokens: int = 0
    grad_norm: Optional[float] = None


@dataclass
class EvalMetrics:
    loss: float = 0.0
    perplexity: float = 0.0
    accuracy: Optional[float] = None
