"""NVTX ranges for timeline profilers (Nsight Systems, the PyTorch profiler).

Off by default: ``PMETAL_NVTX=1`` turns the ranges on. ``with nvtx.range("train_step"):`` marks a host-side span; the
kernels launched inside appear under it on the timeline. The ranges sit at phase level (data, forward + backward,
optimiser step, prefill, decode step), which is what the per-step timing fields of the metrics stream report as numbers
(the reference exposes Metal captures and per-phase stopwatches for the same purpose: crates/pmetal-bridge/cpp/bridge.cpp:605-609,
crates/pmetal-metal/src/ane/profiler.rs)."""
from __future__ import annotations

import contextlib
import os

_ON = None


def enabled() -> bool:
    global _ON
    if _ON is None:
        on = os.environ.get("PMETAL_NVTX") == "1"
        if on:
            try:
                import torch
                on = torch.cuda.is_available()
            except Exception:
                on = False
        _ON = on
    return _ON


def set_enabled(on: bool) -> None:
    global _ON
    _ON = bool(on)


@contextlib.contextmanager
def range(name: str):
    if not enabled():
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def mark(name: str) -> None:
    if enabled():
        import torch
        torch.cuda.nvtx.mark(name)
