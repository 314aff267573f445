"""Masked-diffusion language-model training and sampling (LLaDA / MDLM) and the DFlash draft objective.

Forward process: every token is replaced by the mask token independently with probability t ~ U(min_noise, 1) (in SFT
mode only response tokens, i.e. labels != ignore, are eligible). Training loss: cross-entropy of the model's prediction
at the masked positions, mean over them, divided by t for the ELBO weighting. Sampling: start from all-mask, for
``num_steps`` steps predict every masked position, then re-mask a fraction s / t of the generated span -- the least
confident predictions, random ones, or everything beyond the current block (semi-autoregressive).
Reference: crates/pmetal-trainer/src/diffusion.rs:32-160 (schedules, config), :183-357 (forward process, loss),
:845-960 (sampler). The model is called bidirectionally: any module mapping ids [B, T] -> logits [B, T, V] without a
causal mask works (``BidirectionalLM`` wraps the portable decoder for that).

DFlash draft training (crates/pmetal-trainer/src/dflash_training.rs:49-206): mask a block of the sequence, run the
frozen target over prefix + masked block with hidden-state taps, feed the taps of the block positions and the target's
embedding of the masked block to the draft, project through the target's head and take cross-entropy against the true
tokens of positions 1 .. B-1 of the block (position 0 is the seed slot)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def noise_alpha(schedule: str, t: float) -> float:
    """Fraction of tokens kept at time t."""
    if schedule == "linear":
        return 1.0 - t
    if schedule == "polynomial2":
        return (1.0 - t) ** 2
    if schedule == "cosine":
        return math.cos(math.pi / 2 * t)
    raise ValueError(schedule)


@dataclass
class DiffusionConfig:
    mask_token_id: int
    noise_schedule: str = "linear"
    num_inference_steps: int = 64
    remasking: str = "low_confidence"        # low_confidence | random | semi_autoregressive
    block_size: int = 32                     # semi-autoregressive block
    use_elbo_loss: bool = True
    sft_mode: bool = False
    min_noise_level: float = 1e-4
    sampling_temperature: float = 1.0
    ignore_index: int = -100
    seed: int = 42


def forward_process(x0: torch.Tensor, t: float, mask_token_id: int, generator: Optional[torch.Generator] = None,
                    eligible: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(x_t, mask): each eligible position is masked independently with probability t."""
    u = torch.rand(x0.shape, generator=generator, device=x0.device if generator is None or generator.device == x0.device else "cpu")
    mask = (u.to(x0.device) < t)
    if eligible is not None:
        mask = mask & eligible
    return torch.where(mask, torch.full_like(x0, mask_token_id), x0), mask


def diffusion_loss(logits: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor, t: float, use_elbo: bool = True,
                   ignore_index: int = -100) -> torch.Tensor:
    """Mean over masked, non-ignored positions of -log p(target), divided by t when ``use_elbo``."""
    V = logits.shape[-1]
    valid = mask & (targets != ignore_index) & (targets >= 0) & (targets < V)
    n = int(valid.sum())
    if n == 0:
        return logits.sum() * 0.0
    lp = torch.log_softmax(logits.float(), -1).gather(-1, targets.clamp(min=0)[..., None]).squeeze(-1)
    loss = -(lp * valid).sum()
    if use_elbo and t > 1e-4:
        loss = loss / t
    return loss / n


class BidirectionalLM(nn.Module):
    """Runs a ``GenericDecoderLM`` without the causal mask (every position sees the whole sequence)."""

    def __init__(self, lm):
        super().__init__()
        self.lm = lm

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        from ..models.architectures import generic
        orig = generic.build_mask
        generic.build_mask = lambda kind, q_pos, k_pos, window, chunk: torch.ones(
            q_pos.shape[0], 1, q_pos.shape[1], k_pos.shape[1], dtype=torch.bool, device=q_pos.device)
        try:
            return self.lm(ids)
        finally:
            generic.build_mask = orig


class DiffusionTrainer:
    def __init__(self, model: nn.Module, cfg: DiffusionConfig, lr: float = 1e-4, weight_decay: float = 0.0):
        self.model, self.cfg = model, cfg
        self.opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=lr, weight_decay=weight_decay)
        self.gen = torch.Generator().manual_seed(cfg.seed)
        self.step_count = 0

    def train_step(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> dict:
        c = self.cfg
        t = max(float(torch.rand((), generator=self.gen)), c.min_noise_level)
        targets = input_ids if labels is None else labels
        eligible = (labels != c.ignore_index) if (c.sft_mode and labels is not None) else None
        x_t, mask = forward_process(input_ids, t, c.mask_token_id, self.gen, eligible)
        logits = self.model(x_t)
        loss = diffusion_loss(logits, torch.where(targets == c.ignore_index, input_ids, targets) if not c.sft_mode else targets,
                              mask, t, c.use_elbo_loss, c.ignore_index)
        self.opt.zero_grad()
        loss.backward()
        self.opt.step()
        self.step_count += 1
        return {"loss": float(loss.detach()), "t": t, "masked": int(mask.sum()), "mask_ratio": float(mask.float().mean())}

    @torch.no_grad()
    def evaluate(self, batches: Sequence[torch.Tensor], t: float = 0.5) -> dict:
        tot, n = 0.0, 0
        for ids in batches:
            x_t, mask = forward_process(ids, t, self.cfg.mask_token_id, self.gen)
            tot += float(diffusion_loss(self.model(x_t), ids, mask, t, False, self.cfg.ignore_index)) * int(mask.sum())
            n += int(mask.sum())
        loss = tot / max(n, 1)
        return {"loss": loss, "perplexity": math.exp(min(loss, 50.0))}


class DiffusionSampler:
    def __init__(self, cfg: DiffusionConfig):
        self.cfg = cfg
        self.gen = torch.Generator().manual_seed(cfg.seed)

    @torch.no_grad()
    def sample(self, model: nn.Module, prompt: Sequence[int], max_new_tokens: int, num_steps: Optional[int] = None) -> List[int]:
        c = self.cfg
        steps = num_steps or c.num_inference_steps
        dev = next(model.parameters()).device
        P = len(prompt)
        tokens = torch.tensor(list(prompt) + [c.mask_token_id] * max_new_tokens, device=dev)
        masked = torch.zeros(P + max_new_tokens, dtype=torch.bool, device=dev)
        masked[P:] = True
        for step in range(steps):
            t, s = 1.0 - step / steps, 1.0 - (step + 1) / steps
            logits = model(tokens[None])[0].float()
            if abs(c.sampling_temperature - 1.0) > 1e-6:
                logits = logits / c.sampling_temperature
            conf, pred = torch.softmax(logits, -1).max(-1)
            tokens = torch.where(masked, pred, tokens)
            conf = torch.where(masked, conf, torch.ones_like(conf))      # kept tokens are never re-masked first
            masked = torch.zeros_like(masked)
            if step < steps - 1:
                k = min(int(math.ceil(max_new_tokens * s / t)), max_new_tokens)
                span = torch.arange(P, P + max_new_tokens, device=dev)
                if c.remasking == "random":
                    idx = span[torch.randperm(max_new_tokens, generator=self.gen)[:k].to(dev)]
                elif c.remasking == "semi_autoregressive":
                    idx = span[(step + 1) * c.block_size:]
                else:
                    idx = span[torch.argsort(conf[P:], stable=True)[:k]]
                tokens[idx] = c.mask_token_id
                masked[idx] = True
        return tokens[P:].tolist()


# ------------------------------------------------------------------------------------------------ DFlash draft objective
def dflash_train_step(target, draft, tokens: torch.Tensor, block_start: int, block_size: Optional[int] = None) -> dict:
    """Loss of the draft on one masked block of ``tokens`` [1, T] (target frozen, ``GenericDecoderLM``). Returns
    {"loss": tensor with grad w.r.t. the draft, "accuracy": float, "block": (start, size)}."""
    c = draft.c
    B = min(block_size or c.block_size, c.block_size, tokens.shape[1] - block_start)
    if B < 2:
        raise ValueError("the block needs at least one position after the seed slot")
    ids = tokens.clone()
    ids[:, block_start:block_start + B] = c.mask_token_id
    ids[:, block_start] = tokens[:, block_start]                       # the seed slot keeps the verified token
    taps = {}
    hooks = [target.model.layers[i].register_forward_hook(lambda _m, _i, out, i=i: taps.__setitem__(i, out))
             for i in c.target_layer_ids]
    try:
        with torch.no_grad():
            target(ids[:, : block_start + B])
            hidden = torch.cat([taps[i] for i in c.target_layer_ids], -1)[:, :block_start]      # context before the block
            noise = target.model.embed_tokens(ids[:, block_start:block_start + B])
            if target.c.embed_scale != 1.0:
                noise = noise * target.c.embed_scale
    finally:
        for h in hooks:
            h.remove()
    if hidden.shape[1] == 0:
        raise ValueError("block_start must leave at least one context token")
    dh = draft(noise, hidden)
    logits = target.logits(dh[:, 1:]).float()
    gold = tokens[:, block_start + 1:block_start + B]
    loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), gold.reshape(-1))
    acc = float((logits.argmax(-1) == gold).float().mean())
    return {"loss": loss, "accuracy": acc, "block": (block_start, B)}


class DFlashDraftTrainer:
    """Optimises a draft on random blocks of token sequences."""

    def __init__(self, target, draft, lr: float = 1e-3, seed: int = 0):
        self.target, self.draft = target.eval(), draft
        for p in self.target.parameters():
            p.requires_grad_(False)
        self.opt = torch.optim.AdamW(draft.parameters(), lr=lr)
        self.gen = torch.Generator().manual_seed(seed)

    def train_step(self, tokens: torch.Tensor) -> dict:
        T = tokens.shape[1]
        B = self.draft.c.block_size
        start = int(torch.randint(1, max(T - 2, 2), (), generator=self.gen))
        out = dflash_train_step(self.target, self.draft, tokens, start, min(B, T - start))
        self.opt.zero_grad()
        out["loss"].backward()
        self.opt.step()
        return {"loss": float(out["loss"].detach()), "accuracy": out["accuracy"], "block": out["block"]}
