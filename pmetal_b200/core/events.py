"""Job event stream: tagged JSON lines shared by CLI, dashboards and tool servers.

Wire format follows the reference's ``JobEvent`` enum, tagged with ``"event"`` in
snake_case (crates/pmetal-core/src/events.rs:291-420):

    {"event":"started","job_id":"abc","kind":"train","ts":1700000000}
    {"event":"phase","job_id":"abc","phase":{"phase":"training"}}
    {"event":"metric","job_id":"abc","payload":{"kind":"step","step":1,"loss":2.31}}
"""
from __future__ import annotations

import json
import threading
import time
from typing import Any, Callable, Dict, Iterable, List, Optional

JOB_KINDS = ("train", "distill", "grpo", "rlkd", "embed_train", "pretrain", "serve", "infer", "bench", "eval",
             "quantize", "merge", "fuse", "dataset", "download", "cluster")
PHASES = ("resolving_model", "resolving_dataset", "loading_tokenizer", "tokenizing_dataset", "loading_model",
          "training", "distilling", "generating_teacher_logits", "calibrating", "quantizing", "merging", "saving",
          "evaluating", "generating", "serving")


def _now() -> int:
    return int(time.time())


class JobEvent(dict):
    """A dict with constructors for each event kind."""

    @classmethod
    def started(cls, job_id: str, kind: str) -> "JobEvent":
        return cls(event="started", job_id=job_id, kind=kind, ts=_now())

    @classmethod
    def phase(cls, job_id: str, phase: str, **extra) -> "JobEvent":
        return cls(event="phase", job_id=job_id, phase={"phase": phase, **extra})

    @classmethod
    def metric(cls, job_id: str, kind: str = "step", **payload) -> "JobEvent":
        return cls(event="metric", job_id=job_id, payload={"kind": kind, **payload})

    @classmethod
    def token(cls, job_id: str, token: str, index: int) -> "JobEvent":
        return cls(event="token", job_id=job_id, token=token, index=index)

    @classmethod
    def log(cls, job_id: str, level: str, line: str) -> "JobEvent":
        return cls(event="log", job_id=job_id, level=level, line=line)

    @classmethod
    def progress(cls, job_id: str, current: int, total: Optional[int] = None, label: str = "") -> "JobEvent":
        return cls(event="progress", job_id=job_id, progress={"current": current, "total": total, "label": label})

    @classmethod
    def completed(cls, job_id: str, **summary) -> "JobEvent":
        return cls(event="completed", job_id=job_id, summary=summary, ts=_now())

    @classmethod
    def failed(cls, job_id: str, error: str) -> "JobEvent":
        return cls(event="failed", job_id=job_id, error=error, ts=_now())

    @classmethod
    def cancelled(cls, job_id: str) -> "JobEvent":
        return cls(event="cancelled", job_id=job_id, ts=_now())

    def to_json(self) -> str:
        return json.dumps(self, separators=(",", ":"))

    @classmethod
    def from_json(cls, line: str) -> "JobEvent":
        d = json.loads(line)
        if "event" not in d:
            raise ValueError("not a job event")
        return cls(d)


class JobEventSink:
    def emit(self, ev: JobEvent) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class NullSink(JobEventSink):
    def emit(self, ev: JobEvent) -> None:
        pass


class JsonlSink(JobEventSink):
    """Append events to a file, one JSON object per line, flushed per event."""

    def __init__(self, path: str):
        self._fh = open(path, "a", encoding="utf-8")
        self._lock = threading.Lock()

    def emit(self, ev: JobEvent) -> None:
        with self._lock:
            self._fh.write(ev.to_json() + "\n")
            self._fh.flush()

    def close(self) -> None:
        self._fh.close()


class MemorySink(JobEventSink):
    def __init__(self):
        self.events: List[JobEvent] = []

    def emit(self, ev: JobEvent) -> None:
        self.events.append(ev)


class JobStatus:
    """State derived from an event stream: idle → running(phase) → completed | failed | cancelled."""

    def __init__(self):
        self.state = "idle"
        self.phase: Optional[str] = None
        self.last_metric: Optional[Dict[str, Any]] = None
        self.error: Optional[str] = None
        self.summary: Optional[Dict[str, Any]] = None

    def apply(self, ev: JobEvent) -> "JobStatus":
        e = ev["event"]
        if e == "started":
            self.state = "running"
        elif e == "phase":
            self.phase = ev["phase"]["phase"]
        elif e == "metric":
            self.last_metric = ev["payload"]
        elif e == "completed":
            self.state, self.summary = "completed", ev.get("summary")
        elif e == "failed":
            self.state, self.error = "failed", ev.get("error")
        elif e == "cancelled":
            self.state = "cancelled"
        return self

    @classmethod
    def fold(cls, events: Iterable[JobEvent]) -> "JobStatus":
        st = cls()
        for ev in events:
            st.apply(ev)
        return st
