"""Training callbacks (reference: crates/pmetal-core/src/traits.rs:73-120,
crates/pmetal-trainer/src/callbacks.rs:34-516)."""
from __future__ import annotations

import datetime
import json
import logging
import sys
from typing import List, Optional

from .types import EvalMetrics, StepMetrics

log = logging.getLogger("pmetal")


def _ts() -> str:
    return datetime.datetime.now(datetime.timezone.utc).isoformat()


class TrainingCallback:
    def on_train_start(self) -> None: ...
    def on_train_end(self) -> None: ...
    def on_epoch_start(self, epoch: int) -> None: ...
    def on_epoch_end(self, epoch: int, metrics: EvalMetrics) -> None: ...
    def on_step_start(self, step: int) -> None: ...
    def on_step_end(self, step: int, loss: float) -> None: ...
    def on_step_end_with_metrics(self, metrics: StepMetrics) -> None:
        self.on_step_end(metrics.step, metrics.loss)
    def on_eval(self, metrics: EvalMetrics) -> None: ...
    def on_save(self, path: str) -> None: ...
    def should_stop(self) -> bool:
        return False


class CompositeCallback(TrainingCallback):
    def __init__(self, callbacks: Optional[List[TrainingCallback]] = None):
        self.callbacks = list(callbacks or [])

    def add(self, cb: TrainingCallback) -> None:
        self.callbacks.append(cb)

    def __getattribute__(self, name):
        if name.startswith("on_"):
            cbs = object.__getattribute__(self, "callbacks")

            def fan(*a, **k):
                for cb in cbs:
                    getattr(cb, name)(*a, **k)
            return fan
        return object.__getattribute__(self, name)

    def should_stop(self) -> bool:
        return any(cb.should_stop() for cb in self.callbacks)


class LoggingCallback(TrainingCallback):
    def __init__(self, every: int = 10):
        self.every = max(1, every)

    def on_step_end_with_metrics(self, m: StepMetrics) -> None:
        if m.step % self.every == 0 or m.step == 1:
            gn = f" grad_norm {m.grad_norm:.3f}" if m.grad_norm is not None else ""
            log.info("step %d/%d loss %.4f lr %.3e %.0f tok/s%s", m.step, m.total_steps, m.loss, m.lr, m.tok_sec, gn)


class ProgressCallback(TrainingCallback):
    """Single-line textual progress on stderr (stands in for the reference's indicatif bar)."""

    def __init__(self, stream=None):
        self.stream = stream or sys.stderr

    def on_step_end_with_metrics(self, m: StepMetrics) -> None:
        self.stream.write(f"\r[{m.step}/{m.total_steps}] loss={m.loss:.4f} lr={m.lr:.2e} {m.tok_sec:.0f} tok/s")
        self.stream.flush()

    def on_train_end(self) -> None:
        self.stream.write("\n")


class TensorBoardCallback(TrainingCallback):
    """Scalars per step (loss, learning rate, tokens/s, gradient norm) and per evaluation into a TensorBoard event
    directory (crates/pmetal-trainer/src/callbacks.rs, the ``tensorboard`` feature). Needs the ``tensorboard`` package;
    construction raises ImportError without it."""

    def __init__(self, log_dir: str):
        from torch.utils.tensorboard import SummaryWriter
        self.writer = SummaryWriter(log_dir)

    def on_step_end_with_metrics(self, m: StepMetrics) -> None:
        w = self.writer
        w.add_scalar("train/loss", m.loss, m.step)
        w.add_scalar("train/lr", m.lr, m.step)
        w.add_scalar("train/tokens_per_sec", m.tok_sec, m.step)
        if m.grad_norm is not None:
            w.add_scalar("train/grad_norm", m.grad_norm, m.step)

    def on_eval(self, metrics) -> None:
        step = getattr(metrics, "step", 0)
        for k in ("loss", "perplexity", "accuracy"):
            v = getattr(metrics, k, None) if not isinstance(metrics, dict) else metrics.get(k)
            if v is not None:
                self.writer.add_scalar(f"eval/{k}", float(v), step)

    def on_train_end(self) -> None:
        self.writer.flush()
        self.writer.close()


class MetricsJsonCallback(TrainingCallback):
    """JSON-lines metrics file with the reference's keys and flush cadence
    (callbacks.rs:217-316: every step for the first 20, then every fifth)."""

    def __init__(self, path: str, run_name: Optional[str] = None, config: Optional[dict] = None):
        self._fh = open(path, "w", encoding="utf-8")
        self.run_name, self.config = run_name, config
        self.current_epoch = 0

    def _write(self, entry: dict, flush: bool = True) -> None:
        self._fh.write(json.dumps(entry) + "\n")
        if flush:
            self._fh.flush()

    def on_train_start(self) -> None:
        e = {"event": "train_start", "timestamp": _ts()}
        if self.run_name:
            e["run_name"] = self.run_name
        if self.config is not None:
            e["config"] = self.config
        self._write(e)

    def on_train_end(self) -> None:
        self._write({"event": "train_end", "timestamp": _ts()})

    def on_epoch_start(self, epoch: int) -> None:
        self.current_epoch = epoch

    def on_epoch_end(self, epoch: int, metrics: EvalMetrics) -> None:
        self._write({"event": "epoch_end", "epoch": epoch, "loss": metrics.loss,
                     "perplexity": metrics.perplexity, "timestamp": _ts()})

    def on_step_end(self, step: int, loss: float) -> None:
        self._write({"step": step, "epoch": self.current_epoch, "loss": loss, "timestamp": _ts()},
                    flush=step <= 20 or step % 5 == 0)

    def on_step_end_with_metrics(self, m: StepMetrics) -> None:
        self._write({"step": m.step, "epoch": m.epoch, "total_epochs": m.total_epochs, "total_steps": m.total_steps,
                     "loss": m.loss, "lr": m.lr, "tok_sec": m.tok_sec, "ane_fwd_ms": m.ane_fwd_ms,
                     "ane_bwd_ms": m.ane_bwd_ms, "rmsnorm_ms": m.rmsnorm_ms, "cblas_ms": m.cblas_ms,
                     "adam_ms": m.adam_ms, "total_ms": m.total_ms, "tokens": m.tokens, "grad_norm": m.grad_norm,
                     "timestamp": _ts()}, flush=m.step <= 20 or m.step % 5 == 0)

    def on_save(self, path: str) -> None:
        self._write({"event": "checkpoint_saved", "path": str(path), "timestamp": _ts()})

    def close(self) -> None:
        self._fh.close()


class EventSinkCallback(TrainingCallback):
    """Forwards step metrics into a job-event sink (``--log-events``)."""

    def __init__(self, sink, job_id: str):
        self.sink, self.job_id = sink, job_id

    def on_step_end_with_metrics(self, m: StepMetrics) -> None:
        from .events import JobEvent
        self.sink.emit(JobEvent.metric(self.job_id, "step", step=m.step, total_steps=m.total_steps, loss=m.loss, lr=m.lr,
                                       tok_sec=m.tok_sec, tokens_per_s=m.tok_sec, grad_norm=m.grad_norm))
