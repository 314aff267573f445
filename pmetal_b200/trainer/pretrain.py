"""Full-parameter pre-training loop over token shards (crates/pmetal-trainer/src/pretrain/*).

Every parameter trains (bf16 compute shadows of fp32 masters in the flat AdamW buffer), the loss is next-token
cross-entropy plus an optional z-loss ``z_coef * mean(logsumexp(logits)^2)`` (over the positions that have a target) that
keeps the softmax normaliser near one,
and a checkpoint holds model, optimiser state, step and data position so a run resumes exactly."""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass
from typing import Iterable, Optional

import torch

from ..core.scheduler import LearningRateScheduler


@dataclass
class PretrainConfig:
    learning_rate: float = 3e-4
    min_lr: float = 3e-5
    warmup_steps: int = 100
    max_steps: int = 1000
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    z_loss_coef: float = 1e-4
    seq_len: int = 2048
    micro_batch: int = 4
    gradient_accumulation_steps: int = 1
    lr_scheduler: str = "cosine"
    checkpoint_every: int = 0
    output: str = "./pretrain-output"


class PretrainTrainer:
    def __init__(self, model, cfg: PretrainConfig, dist=None, overlap_reduce: bool = False,
                 reduce_dtype: Optional[torch.dtype] = None, bucket_mb: float = 32.0):
        """``overlap_reduce``: all-reduce the gradient bucket by bucket while backward is still running
        (parallel/overlap.py) instead of after it; ``reduce_dtype=torch.bfloat16`` halves the bytes on the wire."""
        from .optimizer import FlatAdamW, attach_shadows
        self.model, self.cfg, self.dist = model, cfg, dist
        self.device = model.embed_tokens.device
        for p in model.parameters():
            p.requires_grad_(True)
        shadow = torch.bfloat16 if self.device.type == "cuda" else None
        self.opt = FlatAdamW(model.named_parameters(), lr=cfg.learning_rate, weight_decay=cfg.weight_decay,
                             max_grad_norm=cfg.max_grad_norm, shadow_dtype=shadow)
        if dist is not None and getattr(dist, "fused", False):
            dist.bind_optimizer(self.opt)
        if shadow is not None:
            attach_shadows(model, self.opt)
        self.reducer = None
        if overlap_reduce and dist is not None and dist.world_size > 1 and not getattr(dist, "fused", False):
            from ..parallel.overlap import OverlappedGradReducer
            self.reducer = OverlappedGradReducer(self.opt, model, group=dist.group, bucket_mb=bucket_mb,
                                                 reduce_dtype=reduce_dtype)
        self.sched = LearningRateScheduler(cfg.learning_rate, cfg.max_steps, cfg.warmup_steps, cfg.lr_scheduler,
                                           min_lr=cfg.min_lr)
        self.step_count = 0
        self.tokens_seen = 0
        self.data_state: Optional[dict] = None      # position of the training stream, saved with every checkpoint

    def _batch(self, windows):
        import numpy as np
        ids = torch.as_tensor(np.asarray(windows), dtype=torch.int64, device=self.device)
        return ids if ids.dim() == 2 else ids[None]

    def _native_path(self) -> bool:
        """Dense decoder without biases on a GPU with the kernels loaded: embedding, norms, projections, attention and
        the loss all read the bf16 shadows and write fp32 gradients into the flat buffer. Anything else (mixture-of-
        experts layers, biases, CPU) takes the PyTorch operators under autocast."""
        if not hasattr(self, "_native_ok"):
            from ..models.decoder import MLP
            from ..ops import functional as ops
            m = self.model
            self._native_ok = bool(
                self.device.type == "cuda" and getattr(m.embed_tokens, "shadow", None) is not None
                and ops.native_enabled(m.embed_tokens.shadow) and m.cfg.final_logit_softcap <= 0
                and all(isinstance(layer.mlp, MLP) for layer in m.layers)
                and all(fl.bias is None for _, _, fl in m.fused_linears()))
        return self._native_ok

    def _loss(self, ids):
        """(loss to differentiate, cross entropy, z term) of a [B, L] batch; next-token targets inside each window. The z
        term is the mean of logsumexp(logits)^2 over the positions that have a target."""
        from ..ops import functional as ops
        import contextlib
        tgt = torch.full_like(ids, -100)
        tgt[:, :-1] = ids[:, 1:]
        head = self.model.head_weight()
        if self._native_path():
            h = self.model.forward_hidden(ids)
            return ops.linear_cross_entropy_z(h, head, tgt.reshape(-1), self.cfg.z_loss_coef)
        amp = torch.autocast("cuda", dtype=torch.bfloat16) if self.device.type == "cuda" else contextlib.nullcontext()
        with ops.force_reference(), amp:
            h = self.model.forward_hidden(ids)
            return ops.linear_cross_entropy_z(h, head, tgt.reshape(-1), self.cfg.z_loss_coef)

    @torch.no_grad()
    def evaluate(self, dataset: Iterable, max_batches: int = 20) -> dict:
        """Mean cross entropy and perplexity over up to ``max_batches`` micro-batches of held-out windows."""
        was_training = self.model.training
        self.model.eval()
        batch, losses = [], []
        for window in dataset:
            batch.append(window)
            if len(batch) < self.cfg.micro_batch:
                continue
            losses.append(float(self._loss(self._batch(batch))[1]))
            batch = []
            if len(losses) >= max_batches:
                break
        if was_training:
            self.model.train()
        mean = sum(losses) / max(len(losses), 1)
        return {"eval_loss": mean, "eval_perplexity": math.exp(min(mean, 50.0)), "eval_batches": len(losses)}

    def train_step(self, windows) -> dict:
        """One optimiser step. ``windows`` holds ``micro_batch x gradient_accumulation_steps`` windows; every micro-batch
        contributes ``1 / accumulation`` of the gradient."""
        c = self.cfg
        acc = max(c.gradient_accumulation_steps, 1)
        if acc > 1 and len(windows) > c.micro_batch:
            self.opt.set_lr(self.sched.get_lr(self.step_count))
            self.opt.zero_grad()
            ce_sum, zl_sum, n_tok, parts = 0.0, 0.0, 0, [windows[i:i + c.micro_batch] for i in range(0, len(windows), c.micro_batch)]
            for j, part in enumerate(parts):
                ids = self._batch(part)
                loss, ce, zl = self._loss(ids)
                if self.reducer is not None and j == len(parts) - 1:
                    self.reducer.arm()                       # only the last micro-batch leaves final gradients
                (loss / len(parts)).backward()
                ce_sum += float(ce.detach()) / len(parts)
                zl_sum += float(zl.detach()) / len(parts)
                n_tok += ids.numel()
            if self.reducer is not None:
                gn = self.reducer.finish_and_step(1.0)
            elif self.dist is not None and self.dist.world_size > 1:
                gn = self.dist.reduce_and_step(self.opt, 1.0)
            else:
                gn = self.opt.step(1.0)
            self.step_count += 1
            self.tokens_seen += n_tok
            return {"step": self.step_count, "loss": ce_sum, "z_loss": zl_sum, "grad_norm": float(gn), "lr": self.opt.lr,
                    "tokens": self.tokens_seen}
        self.opt.set_lr(self.sched.get_lr(self.step_count))
        self.opt.zero_grad()
        ids = self._batch(windows)
        B, L = ids.shape
        loss, ce, zl = self._loss(ids)
        if self.reducer is not None:
            self.reducer.arm()
        loss.backward()
        if self.reducer is not None:
            gn = self.reducer.finish_and_step(1.0)
        elif self.dist is not None and self.dist.world_size > 1:
            gn = self.dist.reduce_and_step(self.opt, 1.0)
        else:
            gn = self.opt.step(1.0)
        self.step_count += 1
        self.tokens_seen += B * L
        return {"step": self.step_count, "loss": float(ce.detach()), "z_loss": float(zl.detach()),
                "grad_norm": float(gn), "lr": self.opt.lr, "tokens": self.tokens_seen}

    def run(self, dataset: Iterable, on_step=None, eval_dataset=None, eval_every: int = 0, eval_batches: int = 20) -> dict:
        c = self.cfg
        batch, last = [], {}
        per_step = c.micro_batch * max(c.gradient_accumulation_steps, 1)
        if self.data_state is not None and hasattr(dataset, "load_state_dict"):
            dataset.load_state_dict(self.data_state)            # resume exactly where the checkpointed run stopped reading
        if self.step_count >= c.max_steps:
            return last
        for window in dataset:
            batch.append(window)
            if len(batch) < per_step:
                continue
            last = self.train_step(batch)
            batch = []
            if hasattr(dataset, "state_dict"):
                self.data_state = dataset.state_dict()
            if eval_dataset is not None and eval_every and self.step_count % eval_every == 0:
                last = {**last, **self.evaluate(eval_dataset, eval_batches)}
            if on_step:
                on_step(last)
            if c.checkpoint_every and self.step_count % c.checkpoint_every == 0:
                self.save_checkpoint(os.path.join(c.output, f"step_{self.step_count}"))
            if self.step_count >= c.max_steps:
                break
        return last

    def save_checkpoint(self, path: str) -> None:
        from ..utils import safetensors_io as st
        os.makedirs(path, exist_ok=True)
        sd = {k: v.detach().cpu().contiguous() for k, v in self.model.hf_state_dict(merged=False).items()}
        st.save_file(sd, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
        o = self.opt.state_dict()
        st.save_file({k: v.detach().cpu().contiguous() for k, v in o.items() if isinstance(v, torch.Tensor)},
                     os.path.join(path, "optimizer.safetensors"))
        with open(os.path.join(path, "trainer_state.json"), "w", encoding="utf-8") as fh:
            json.dump({"step": self.step_count, "tokens_seen": self.tokens_seen, "config": asdict(self.cfg),
                       "data_state": self.data_state,
                       "optimizer_scalars": {k: v for k, v in o.items() if not isinstance(v, torch.Tensor)}}, fh, indent=2)

    def load_checkpoint(self, path: str) -> None:
        from ..utils import safetensors_io as st
        # parameters are views of the optimiser's flat fp32 buffer, so loading into the model updates the masters
        self.model.load_hf_state_dict(st.load_file(os.path.join(path, "model.safetensors")), strict=False)
        with open(os.path.join(path, "trainer_state.json"), "r", encoding="utf-8") as fh:
            state = json.load(fh)
        o = dict(st.load_file(os.path.join(path, "optimizer.safetensors")))
        o.update(state.get("optimizer_scalars", {}))
        self.opt.load_state_dict(o)
        self.opt.sync_shadow()
        self.step_count, self.tokens_seen = state["step"], state["tokens_seen"]
        self.data_state = state.get("data_state")
