"""Runtime auto-tuner with a persistent JSON cache (the counterpart of the reference's "Tuna",
crates/pmetal-metal/src/tuna.rs:1-20, which caches tuned tile sizes under ~/.cache/pmetal/tuna/).

``Tuner.tune(key, candidates, run)`` times ``run(candidate)`` for every candidate with CUDA events (warm-up, median of
``iters``), remembers the winner under ``key`` (shape, dtype, device name) and writes the cache atomically. The GEMM
wrapper consults it for the tile width when ``PMETAL_TUNA=1``; otherwise static heuristics are used."""
from __future__ import annotations

import json
import os
import statistics
import tempfile
from typing import Callable, Dict, Hashable, Optional, Sequence


def default_cache_path() -> str:
    base = os.environ.get("PMETAL_TUNA_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "pmetal_b200", "tuna")
    return os.path.join(base, "tuna.json")


class Tuner:
    def __init__(self, path: Optional[str] = None, iters: int = 10, warmup: int = 3):
        self.path, self.iters, self.warmup = path or default_cache_path(), iters, warmup
        self.table: Dict[str, dict] = {}
        try:
            with open(self.path, "r", encoding="utf-8") as fh:
                self.table = json.load(fh)
        except (OSError, ValueError):
            self.table = {}

    @staticmethod
    def make_key(op: str, *parts: Hashable) -> str:
        dev = "cpu"
        try:
            import torch
            if torch.cuda.is_available():
                dev = torch.cuda.get_device_name(torch.cuda.current_device())
        except ImportError:
            pass
        return "|".join([op, dev] + [str(p) for p in parts])

    def lookup(self, key: str):
        e = self.table.get(key)
        return None if e is None else e["best"]

    def _time(self, fn: Callable[[], None]) -> float:
        import torch
        if not torch.cuda.is_available():
            import time
            for _ in range(self.warmup):
                fn()
            ts = []
            for _ in range(self.iters):
                t0 = time.perf_counter()
                fn()
                ts.append((time.perf_counter() - t0) * 1e3)
            return statistics.median(ts)
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    def tune(self, key: str, candidates: Sequence, run: Callable[[object], None]):
        hit = self.lookup(key)
        if hit is not None and hit in list(candidates):
            return hit
        timings = {}
        for c in candidates:
            try:
                timings[c] = self._time(lambda c=c: run(c))
            except Exception:          # a candidate that is invalid for this shape simply loses
                continue
        if not timings:
            raise RuntimeError(f"no candidate ran for {key}")
        best = min(timings, key=timings.get)
        self.table[key] = {"best": best, "ms": {str(k): round(v, 5) for k, v in timings.items()}}
        self.save()
        return best

    def save(self) -> None:
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=os.path.dirname(self.path), suffix=".tmp")
        with os.fdopen(fd, "w", encoding="utf-8") as fh:
            json.dump(self.table, fh, indent=1, sort_keys=True)
        os.replace(tmp, self.path)


_GLOBAL: Optional[Tuner] = None


def global_tuner() -> Tuner:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = Tuner()
    return _GLOBAL
