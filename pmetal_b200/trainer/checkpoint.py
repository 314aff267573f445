"""Checkpoint directory management.

Layout (crates/pmetal-trainer/src/checkpoint.rs:30-560):

    <output>/checkpoints/step_N/{lora_weights.safetensors, metadata.json}
    <output>/checkpoints/latest            text file naming the newest step dir
    <output>/checkpoints/best/             copy of the best-eval checkpoint
    <output>/checkpoints/best_snapshot.safetensors   atomic tmp+rename

Only the newest ``keep`` step directories are retained. The reference does not save
optimizer state for LoRA runs; here ``optimizer.pt`` and ``rng.pt`` are written as
extra files beside the adapter so the adapter file itself stays the same.
Writes happen on a background thread which is joined before the next save and on close.
"""
from __future__ import annotations

import dataclasses
import datetime
import json
import os
import shutil
import threading
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..utils import safetensors_io as st


@dataclass
class CheckpointMetadata:
    step: int
    epoch: int
    running_loss: float
    learning_rate: float
    best_val_loss: Optional[float] = None
    model_config: Optional[str] = None
    training_config: Optional[str] = None
    seed: int = 42
    timestamp: str = ""

    def __post_init__(self):
        if not self.timestamp:
            self.timestamp = datetime.datetime.now(datetime.timezone.utc).isoformat()


class CheckpointManager:
    def __init__(self, checkpoint_dir: str, keep: int = 3, async_write: bool = True):
        self.dir, self.keep, self.async_write = checkpoint_dir, keep, async_write
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        os.makedirs(checkpoint_dir, exist_ok=True)

    # ------------------------------------------------------------------ save
    def save(self, tensors: Dict[str, torch.Tensor], meta: CheckpointMetadata, extra: Optional[dict] = None,
             is_best: bool = False) -> str:
        self.wait()
        path = os.path.join(self.dir, f"step_{meta.step}")
        cpu = {k: v.detach().to("cpu", copy=True) for k, v in tensors.items()}   # snapshot before going async

        def work():
            try:
                os.makedirs(path, exist_ok=True)
                st.save_file(cpu, os.path.join(path, "lora_weights.safetensors"), metadata={"format": "mlx"})
                with open(os.path.join(path, "metadata.json"), "w", encoding="utf-8") as fh:
                    json.dump(dataclasses.asdict(meta), fh, indent=2)
                if extra:
                    for name, obj in extra.items():
                        torch.save(obj, os.path.join(path, name))
                tmp = os.path.join(self.dir, "latest.tmp")
                with open(tmp, "w", encoding="utf-8") as fh:
                    fh.write(f"step_{meta.step}")
                os.replace(tmp, os.path.join(self.dir, "latest"))
                if is_best:
                    best = os.path.join(self.dir, "best")
                    if os.path.isdir(best):
                        shutil.rmtree(best)
                    shutil.copytree(path, best)
                self._cleanup()
            except BaseException as e:  # surfaced on the next wait()
                self._error = e

        if self.async_write:
            self._thread = threading.Thread(target=work, name="pmetal-checkpoint", daemon=True)
            self._thread.start()
        else:
            work()
            self.wait()
        return path

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            e, self._error = self._error, None
            raise RuntimeError(f"checkpoint write failed: {e}") from e

    close = wait

    def _steps(self):
        out = []
        for d in os.listdir(self.dir):
            if d.startswith("step_") and d[5:].isdigit() and os.path.isdir(os.path.join(self.dir, d)):
                out.append(int(d[5:]))
        return sorted(out)

    def _cleanup(self) -> None:
        steps = self._steps()
        for s in steps[:-self.keep] if self.keep > 0 else []:
            shutil.rmtree(os.path.join(self.dir, f"step_{s}"), ignore_errors=True)

    # ------------------------------------------------------------------ best snapshot
    def save_best_snapshot(self, tensors: Dict[str, torch.Tensor]) -> None:
        st.save_file({k: v.detach().cpu() for k, v in tensors.items()},
                     os.path.join(self.dir, "best_snapshot.safetensors"))

    def load_best_snapshot(self) -> Optional[Dict[str, torch.Tensor]]:
        p = os.path.join(self.dir, "best_snapshot.safetensors")
        return st.load_file(p) if os.path.exists(p) else None

    # ------------------------------------------------------------------ load
    def latest_path(self) -> Optional[str]:
        self.wait()
        marker = os.path.join(self.dir, "latest")
        if os.path.exists(marker):
            with open(marker, "r", encoding="utf-8") as fh:
                p = os.path.join(self.dir, fh.read().strip())
            if os.path.isdir(p):
                return p
        steps = self._steps()
        return os.path.join(self.dir, f"step_{steps[-1]}") if steps else None

    @staticmethod
    def load(path: str):
        with open(os.path.join(path, "metadata.json"), "r", encoding="utf-8") as fh:
            meta = CheckpointMetadata(**json.load(fh))
        tensors = st.load_file(os.path.join(path, "lora_weights.safetensors"))
        extra = {}
        for name in ("optimizer.pt", "rng.pt"):
            p = os.path.join(path, name)
            if os.path.exists(p):
                # tensors, lists, numbers and strings only: a checkpoint directory must not be able to run code
                extra[name] = torch.load(p, map_location="cpu", weights_only=True)
        return tensors, meta, extra
