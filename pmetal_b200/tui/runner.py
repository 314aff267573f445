"""Child-process job runner for the terminal front end.

Each job is ``python -m pmetal_b200.cli --log-events FILE <argv>`` in its own process group; its combined output goes to
a log file and its progress is read back from the event file (the same stream ``dashboard`` follows). Counterpart of
crates/pmetal/src/tui/command_runner.rs (spawn, tail, cancel)."""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class Job:
    job_id: int
    command: str
    argv: List[str]
    log_path: str
    events_path: str
    proc: Optional[subprocess.Popen] = None
    started: float = field(default_factory=time.time)
    ended: Optional[float] = None
    state: str = "running"                  # running | finished | failed | cancelled
    returncode: Optional[int] = None
    metrics: Dict[str, float] = field(default_factory=dict)
    history: Dict[str, List[float]] = field(default_factory=dict)       # per metric name, in arrival order
    _ev_pos: int = 0

    def elapsed(self) -> float:
        return (self.ended or time.time()) - self.started

    def tail(self, n: int = 20) -> List[str]:
        try:
            with open(self.log_path, "rb") as fh:
                fh.seek(0, os.SEEK_END)
                size = fh.tell()
                fh.seek(max(0, size - 16384))
                return fh.read().decode("utf-8", "replace").splitlines()[-n:]
        except OSError:
            return []

    def poll_events(self) -> None:
        """Fold the event lines written since the last call into ``metrics`` / ``history``."""
        try:
            with open(self.events_path, "r", encoding="utf-8") as fh:
                fh.seek(self._ev_pos)
                chunk = fh.read()
        except OSError:
            return
        keep = chunk.rfind("\n") + 1                      # a partly written last line waits for the next poll
        self._ev_pos += len(chunk[:keep].encode("utf-8"))
        for ln in chunk[:keep].splitlines():
            try:
                ev = json.loads(ln)
            except ValueError:
                continue
            if ev.get("event") != "metric":
                continue
            for k, v in (ev.get("payload") or {}).items():
                if isinstance(v, (int, float)) and not isinstance(v, bool):
                    self.metrics[k] = v
                    self.history.setdefault(k, []).append(float(v))


class JobRunner:
    """Starts, follows and cancels command-line jobs. ``python`` and ``module`` can be replaced in tests."""

    def __init__(self, workdir: Optional[str] = None, python: Optional[str] = None, module: str = "pmetal_b200.cli"):
        self.workdir = workdir or tempfile.mkdtemp(prefix="pmetal-tui-")
        self.python = python or sys.executable
        self.module = module
        self.jobs: List[Job] = []

    def start(self, command: str, argv: List[str]) -> Job:
        jid = len(self.jobs) + 1
        log = os.path.join(self.workdir, f"job{jid}.log")
        events = os.path.join(self.workdir, f"job{jid}.events.jsonl")
        cmd = [self.python, "-m", self.module, "--log-events", events] + list(argv)
        out = open(log, "wb")
        try:
            proc = subprocess.Popen(cmd, stdout=out, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL,
                                    start_new_session=True)
        finally:
            out.close()
        job = Job(jid, command, list(argv), log, events, proc)
        self.jobs.append(job)
        return job

    def poll(self) -> None:
        for j in self.jobs:
            j.poll_events()
            if j.state == "running" and j.proc is not None:
                rc = j.proc.poll()
                if rc is not None:
                    j.returncode, j.ended = rc, time.time()
                    j.state = "finished" if rc == 0 else "failed"
                    j.poll_events()

    def cancel(self, job: Job, grace: float = 5.0) -> None:
        """SIGTERM to the job's own process group, SIGKILL after ``grace`` seconds."""
        if job.state != "running" or job.proc is None:
            return
        try:
            os.killpg(job.proc.pid, signal.SIGTERM)
            try:
                job.proc.wait(grace)
            except subprocess.TimeoutExpired:
                os.killpg(job.proc.pid, signal.SIGKILL)
                job.proc.wait(grace)
        except ProcessLookupError:
            pass
        job.returncode, job.ended, job.state = job.proc.returncode, time.time(), "cancelled"

    def running(self) -> List[Job]:
        return [j for j in self.jobs if j.state == "running"]

    def shutdown(self) -> None:
        for j in self.running():
            self.cancel(j, grace=2.0)
