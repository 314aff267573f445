"""Supervised fine-tuning loop (padded and packed batches).

Semantics kept from the reference (crates/pmetal-trainer/src/training_loop/mod.rs:267-1524,
run_packed.rs:12-401, step_functions.rs:35-342):

* loss = mean over non-ignored tokens of the shifted causal-LM cross-entropy;
* gradient accumulation scales each micro-batch by 1/accum;
* global-norm clipping, then (data-parallel) gradient mean, then AdamW — the clip
  comes *before* the reduction as in the reference, ``clip_after_reduce=True`` selects
  the order that clips the averaged gradient instead;
* learning rate is set from the schedule before every optimizer step;
* running loss is an exponential moving average (0.99 / 0.01);
* tokens/s counts real (non-padding) tokens;
* only rank 0 writes checkpoints.

On a CUDA device the whole micro-step can be replayed from a CUDA graph after one
eager warm-up step (the analogue of the reference's compiled path, run_compiled.rs:31-330).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional

import torch

from ..core.callbacks import CompositeCallback, TrainingCallback
from ..core.config import TrainingConfig
from ..core.scheduler import LearningRateScheduler
from ..core.types import EvalMetrics, StepMetrics
from ..data.packing import PackedTensors
from .optimizer import FlatAdamW, attach_shadows


@dataclass
class LoopState:
    step: int = 0
    epoch: int = 0
    running_loss: float = 0.0
    best_val_loss: Optional[float] = None
    tokens_seen: int = 0


class TrainingLoop:
    def __init__(self, model, cfg: TrainingConfig, callbacks: Optional[List[TrainingCallback]] = None,
                 dist=None, loraplus_ratio: Optional[float] = None, clip_after_reduce: bool = False,
                 checkpoint_manager=None, adaptive_lr=None, total_steps: Optional[int] = None):
        self.model, self.cfg = model, cfg
        self.cb = CompositeCallback(callbacks)
        self.dist = dist
        self.clip_after_reduce = clip_after_reduce
        self.ckpt = checkpoint_manager
        self.adaptive = adaptive_lr
        dev = next(model.parameters()).device
        self.device = dev
        shadow = torch.bfloat16 if dev.type == "cuda" else None
        fused_dist = dist is not None and getattr(dist, "fused", False)
        self.opt = FlatAdamW(model.named_parameters(), lr=cfg.learning_rate, weight_decay=cfg.weight_decay,
                             embedding_lr=cfg.embedding_learning_rate or 5e-5, loraplus_ratio=loraplus_ratio,
                             max_grad_norm=cfg.max_grad_norm, shadow_dtype=shadow)
        if fused_dist:
            dist.bind_optimizer(self.opt)
        if shadow is not None:
            attach_shadows(model, self.opt)
        self.sched = LearningRateScheduler.from_training_config(cfg, total_steps)
        self.state = LoopState()
        self.lr_override: Optional[float] = None
        self.should_stop = False
        self._accum = 0
        self._t_last = None
        self._tok_since = 0

    # ------------------------------------------------------------------ one micro-batch
    def _loss_for(self, batch) -> torch.Tensor:
        if isinstance(batch, PackedTensors):
            return self.model.loss(batch.input_ids, batch.labels, batch.position_ids, batch.cu_seqlens,
                                   batch.seq_start)
        return self.model.loss(batch["input_ids"], batch["labels"])

    def current_lr(self) -> float:
        return self.lr_override if self.lr_override is not None else self.sched.get_lr(self.state.step)

    def micro_step(self, batch) -> torch.Tensor:
        """Forward + backward of one micro-batch; gradients accumulate in the flat buffer."""
        if self._accum == 0:
            self.opt.zero_grad()
        loss = self._loss_for(batch)
        loss.backward()
        self._accum += 1
        return loss.detach()

    def optimizer_step(self) -> torch.Tensor:
        ga = max(self._accum, 1)
        self.opt.set_lr(self.current_lr())
        if self.dist is not None and self.dist.world_size > 1:
            gnorm = self.dist.reduce_and_step(self.opt, 1.0 / ga, self.clip_after_reduce)
        else:
            gnorm = self.opt.step(1.0 / ga)
        self._accum = 0
        self.state.step += 1
        return gnorm

    def train_step(self, batch) -> (torch.Tensor, Optional[torch.Tensor]):
        from ..utils import nvtx
        with nvtx.range("forward_backward"):
            loss = self.micro_step(batch)
        if self._accum >= self.cfg.gradient_accumulation_steps:
            with nvtx.range("optimizer_step"):
                return loss, self.optimizer_step()
        return loss, None

    # ------------------------------------------------------------------ CUDA-graph step
    def enable_cuda_graph(self, example: PackedTensors) -> None:
        """Capture forward + backward + (reduce) + optimizer of one fixed-shape packed batch into a CUDA graph.

        One eager step on ``example`` runs first (it is a real optimizer step). Later calls of
        ``train_step_graphed`` copy the batch into the static input buffers, stage the learning rate and
        bias corrections on the device and replay the graph. Requires gradient_accumulation_steps == 1.
        """
        assert self.device.type == "cuda" and self.cfg.gradient_accumulation_steps == 1
        ex = example.to(self.device)
        self._g_in = PackedTensors(ex.input_ids.clone(), ex.labels.clone(), ex.position_ids.clone(),
                                   ex.cu_seqlens.clone(), ex.seq_start.clone(), ex.total_tokens, ex.num_sequences,
                                   ex.max_seqlen)
        self.opt.device_hparams = True
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.opt.set_lr(self.current_lr())
            self.opt.push_hparams(self.opt.step_count + 1)
            self.train_step(self._g_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        from ..ops import native
        n0 = native.LAUNCHES
        with torch.cuda.graph(self._graph):
            loss = self.micro_step(self._g_in)
            gn = self.optimizer_step()
        self.launches_per_graph = native.LAUNCHES - n0
        self.opt.step_count -= 1          # capture records the work without running it
        self.state.step -= 1
        self._g_loss, self._g_gnorm = loss, gn

    def train_step_graphed(self, batch: PackedTensors):
        from ..utils import nvtx
        gi = self._g_in
        with nvtx.range("stage_batch"):
            gi.input_ids.copy_(batch.input_ids, non_blocking=True)
            gi.labels.copy_(batch.labels, non_blocking=True)
            gi.position_ids.copy_(batch.position_ids, non_blocking=True)
            gi.seq_start.copy_(batch.seq_start, non_blocking=True)
            self.opt.set_lr(self.current_lr())
            self.opt.step_count += 1
            self.opt.push_hparams(self.opt.step_count)
        with nvtx.range("train_step_graph"):
            self._graph.replay()
        self.state.step += 1
        return self._g_loss, self._g_gnorm

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate(self, batches: Iterable) -> EvalMetrics:
        was = self.model.training
        self.model.eval()
        tot, n = 0.0, 0
        for b in batches:
            b = self._to_device(b)
            tot += float(self._loss_for(b))
            n += 1
        self.model.train(was)
        loss = tot / max(n, 1)
        return EvalMetrics(loss=loss, perplexity=math.exp(min(loss, 50.0)))

    def _to_device(self, batch):
        if isinstance(batch, PackedTensors):
            return batch.to(self.device) if batch.input_ids.device != self.device else batch
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}

    # ------------------------------------------------------------------ full run
    def run(self, loader, eval_loader=None, num_epochs: Optional[int] = None) -> LoopState:
        cfg = self.cfg
        epochs = num_epochs if num_epochs is not None else cfg.num_epochs
        per_epoch = max(len(loader) // max(cfg.gradient_accumulation_steps, 1), 1)
        total_steps = cfg.max_steps or per_epoch * epochs
        self.model.train()
        self.cb.on_train_start()
        if self.dist is not None:
            self.dist.barrier()
        self._t_last = time.perf_counter()
        is_master = self.dist is None or self.dist.rank == 0
        done = False
        for epoch in range(self.state.epoch, epochs):
            self.state.epoch = epoch
            if hasattr(loader, "set_epoch"):
                loader.set_epoch(epoch)
            self.cb.on_epoch_start(epoch)
            for batch in loader:
                batch = self._to_device(batch)
                ntok = batch.total_tokens if isinstance(batch, PackedTensors) else int(batch.get("tokens", 0))
                self.cb.on_step_start(self.state.step)
                loss, gnorm = self.train_step(batch)
                self._tok_since += ntok
                if gnorm is None:
                    continue
                lossf = float(loss)
                if self.dist is not None and self.dist.world_size > 1:
                    lossf = self.dist.mean_scalar(lossf)
                st = self.state
                st.running_loss = lossf if st.step == 1 else 0.99 * st.running_loss + 0.01 * lossf
                st.tokens_seen += self._tok_since
                now = time.perf_counter()
                dt = max(now - self._t_last, 1e-9)
                m = StepMetrics(step=st.step, epoch=epoch, total_epochs=epochs, total_steps=total_steps, loss=lossf,
                                lr=self.opt.lr, tok_sec=self._tok_since / dt, total_ms=dt * 1e3,
                                tokens=self._tok_since, grad_norm=float(gnorm))
                self._t_last, self._tok_since = now, 0
                self.cb.on_step_end_with_metrics(m)
                if self.adaptive is not None:
                    self._apply_adaptive(self.adaptive.observe(st.step, lossf, self.sched.get_lr(st.step)))
                if eval_loader is not None and cfg.eval_steps and st.step % cfg.eval_steps == 0:
                    em = self.evaluate(eval_loader)
                    self.cb.on_eval(em)
                    if st.best_val_loss is None or em.loss < st.best_val_loss:
                        st.best_val_loss = em.loss
                if cfg.save_steps and st.step % cfg.save_steps == 0:
                    if self.dist is not None:                 # every rank: sharded optimizer state is collected first
                        self.dist.gather_optimizer_state(self.opt)
                    if self.ckpt is not None and is_master:
                        self.save_checkpoint()
                if (cfg.max_steps and st.step >= cfg.max_steps) or self.cb.should_stop() or self.should_stop:
                    done = True
                    break
            self.cb.on_epoch_end(epoch, EvalMetrics(loss=self.state.running_loss,
                                                    perplexity=math.exp(min(self.state.running_loss, 50.0))))
            if self.dist is not None:
                self.dist.barrier()
            if done:
                break
        if self.ckpt is not None:
            self.ckpt.wait()
        self.cb.on_train_end()
        return self.state

    def _apply_adaptive(self, action) -> None:
        if action is None:
            return
        kind = action.get("action")
        if kind == "set_lr":
            self.lr_override = action["lr"]
        elif kind == "reset_lr":
            self.lr_override = None
        elif kind in ("early_stop", "graceful_stop"):
            self.should_stop = True
        elif kind == "save_checkpoint" and self.ckpt is not None:
            self.save_checkpoint()
        elif kind == "rollback" and self.ckpt is not None:
            snap = self.ckpt.load_best_snapshot()
            if snap is not None:
                self.load_lora_tensors(snap)
            self.lr_override = action.get("lr", self.lr_override)
        elif kind == "snapshot" and self.ckpt is not None:
            from ..lora.adapter import lora_state_dict
            self.ckpt.save_best_snapshot(lora_state_dict(self.model))

    def save_checkpoint(self, is_best: bool = False) -> str:
        from ..lora.adapter import lora_state_dict
        from .checkpoint import CheckpointMetadata
        st = self.state
        meta = CheckpointMetadata(step=st.step, epoch=st.epoch, running_loss=st.running_loss,
                                  learning_rate=self.opt.lr, best_val_loss=st.best_val_loss, seed=self.cfg.seed)
        path = self.ckpt.save(lora_state_dict(self.model), meta,
                              extra={"optimizer.pt": self.opt.state_dict(),
                                     "rng.pt": {"cpu": torch.get_rng_state()}}, is_best=is_best)
        self.cb.on_save(path)
        return path

    @torch.no_grad()
    def load_lora_tensors(self, tensors) -> None:
        import os
        import tempfile
        from ..lora.adapter import load_adapter
        from ..utils import safetensors_io as st
        with tempfile.TemporaryDirectory() as d:
            p = os.path.join(d, "lora_weights.safetensors")
            st.save_file(tensors, p)
            load_adapter(self.model, p)
        self.opt.sync_shadow()

    def resume(self, path: str) -> None:
        """Restore LoRA parameters and step/epoch (plus optimizer moments when present)."""
        from .checkpoint import CheckpointManager
        tensors, meta, extra = CheckpointManager.load(path)
        self.load_lora_tensors(tensors)
        self.state.step, self.state.epoch = meta.step, meta.epoch
        self.state.running_loss, self.state.best_val_loss = meta.running_loss, meta.best_val_loss
        if "optimizer.pt" in extra:
            self.opt.load_state_dict(extra["optimizer.pt"])
