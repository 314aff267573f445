"""Token sampling.

Order of operations follows the reference sampler (crates/pmetal-models/src/generation.rs:796-1118):
penalties on the raw logits (repetition over prompt+output, frequency x count, flat presence) ->
greedy argmax when sampling is off -> log-softmax -> top-k (keep the k largest) -> top-p (ascending
sort, keep where the cumulative probability exceeds 1-p) -> min-p (keep logp >= max_logp + ln(min_p))
-> categorical over logp / T. Defaults: T 0.7, top-k 40, top-p 0.95, min-p 0.05, repetition 1.1,
256 new tokens (generation.rs:418-436). All steps are batched over rows and stay on the device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repetition_penalty: float = 1.1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    max_tokens: int = 256
    do_sample: bool = True
    seed: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)

    @classmethod
    def greedy(cls, max_tokens: int = 256) -> "SamplingParams":
        return cls(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0, max_tokens=max_tokens,
                   do_sample=False)

    @property
    def is_greedy(self) -> bool:
        return (not self.do_sample) or self.temperature <= 0.0


def apply_penalties(logits: torch.Tensor, token_counts: Optional[torch.Tensor], p: SamplingParams) -> torch.Tensor:
    """``token_counts`` [B, V]: occurrences of each id in prompt+output (dense; None = no history)."""
    if token_counts is None:
        return logits
    seen = token_counts > 0
    if p.repetition_penalty != 1.0:
        pen = torch.where(logits > 0, logits / p.repetition_penalty, logits * p.repetition_penalty)
        logits = torch.where(seen, pen, logits)
    if p.frequency_penalty != 0.0:
        logits = logits - p.frequency_penalty * token_counts.to(logits.dtype)
    if p.presence_penalty != 0.0:
        logits = logits - p.presence_penalty * seen.to(logits.dtype)
    return logits


def filtered_logprobs(logits: torch.Tensor, p: SamplingParams) -> torch.Tensor:
    """log-probabilities after top-k / top-p / min-p; masked entries are -inf. [B, V] fp32."""
    logp = torch.log_softmax(logits.float(), dim=-1)
    V = logp.shape[-1]
    if 0 < p.top_k < V:
        kth = torch.topk(logp, p.top_k, dim=-1).values[..., -1:]
        logp = logp.masked_fill(logp < kth, float("-inf"))
    if 0.0 < p.top_p < 1.0:
        srt, idx = torch.sort(logp, dim=-1, descending=False)
        cum = torch.cumsum(srt.exp(), dim=-1)
        total = cum[..., -1:]
        keep = cum > (1.0 - p.top_p) * total
        keep[..., -1] = True
        srt = srt.masked_fill(~keep, float("-inf"))
        logp = torch.full_like(logp, float("-inf")).scatter(-1, idx, srt)
    if p.min_p > 0.0:
        mx = logp.max(dim=-1, keepdim=True).values
        logp = logp.masked_fill(logp < mx + math.log(p.min_p), float("-inf"))
    return logp


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None, device=None):
        self.params = params or SamplingParams()
        self.gen = None
        if self.params.seed is not None:
            self.gen = torch.Generator(device=device or "cpu").manual_seed(self.params.seed)

    def _native_sample(self, logits, token_counts, return_logprobs):
        """Fused sampling kernel (csrc/sampling.cu): one launch for penalties, filters and the draw."""
        from ..ops import native
        p = self.params
        B = logits.shape[0]
        key = (B, logits.device)
        if getattr(self, "_nat_key", None) != key:
            dev = logits.device
            f = lambda v: torch.full((B,), float(v), dtype=torch.float32, device=dev)      # noqa: E731
            self._nat = dict(temp=f(0.0 if p.is_greedy else p.temperature),
                             top_k=torch.full((B,), int(p.top_k), dtype=torch.int32, device=dev), top_p=f(p.top_p),
                             min_p=f(p.min_p), rep=f(p.repetition_penalty), freq=f(p.frequency_penalty),
                             pres=f(p.presence_penalty))
            base = p.seed if p.seed is not None else int(torch.empty((), dtype=torch.int64).random_().item())
            self._nat["seeds"] = (torch.arange(B, dtype=torch.int64, device=dev) * 0x9E3779B1 + base)
            self._nat_key, self._nat_step = key, 0
        n = self._nat
        self._nat_step += 1
        if logits.stride(-1) != 1:
            logits = logits.contiguous()
        ids, lp = native.sample(logits, n["temp"], n["top_k"], n["top_p"], n["min_p"], token_counts, n["rep"], n["freq"],
                                n["pres"], n["seeds"], self._nat_step, return_logprobs)
        ids = ids.long()
        return (ids, lp) if return_logprobs else ids

    def sample(self, logits: torch.Tensor, token_counts: Optional[torch.Tensor] = None,
               return_logprobs: bool = False):
        """logits [B, V] -> ids [B] (and the log-probability of each chosen id under the filtered distribution)."""
        p = self.params
        if logits.is_cuda and logits.dim() == 2 and logits.dtype in (torch.float32, torch.bfloat16) and \
                (token_counts is None or token_counts.dtype == torch.int32):
            from ..ops import functional as _ops
            if _ops.native_enabled(logits):
                return self._native_sample(logits, token_counts, return_logprobs)
        logits = apply_penalties(logits.float(), token_counts, p)
        if p.is_greedy:
            ids = logits.argmax(dim=-1)
            if return_logprobs:
                lp = torch.log_softmax(logits, -1).gather(-1, ids[:, None])[:, 0]
                return ids, lp
            return ids
        logp = filtered_logprobs(logits, p)
        probs = torch.softmax(logp / p.temperature, dim=-1)
        if self.gen is not None and self.gen.device != probs.device:
            self.gen = torch.Generator(device=probs.device).manual_seed(self.params.seed)
        ids = torch.multinomial(probs, 1, generator=self.gen)[:, 0]
        if return_logprobs:
            return ids, torch.log(probs.gather(-1, ids[:, None])[:, 0])
        return ids


PRESETS = {
    # generation.rs:469-550 (model-card recommendations)
    "qwen3-thinking": SamplingParams(temperature=0.6, top_p=0.95, top_k=20, min_p=0.0, repetition_penalty=1.0),
    "qwen3-non-thinking": SamplingParams(temperature=0.7, top_p=0.8, top_k=20, min_p=0.0, repetition_penalty=1.0),
    "llama": SamplingParams(temperature=0.6, top_p=0.9, top_k=0, min_p=0.0, repetition_penalty=1.0),
    "default": SamplingParams(),
}


def params_from_generation_config(model_dir: str, base: Optional[SamplingParams] = None) -> SamplingParams:
    """Override defaults with ``generation_config.json`` (generation.rs:553-620)."""
    import json
    import os
    p = base or SamplingParams()
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.exists(path):
        return p
    with open(path, "r", encoding="utf-8") as fh:
        g = json.load(fh)
    for k in ("temperature", "top_k", "top_p", "min_p", "repetition_penalty"):
        if g.get(k) is not None:
            setattr(p, k, type(getattr(p, k))(g[k]))
    if g.get("do_sample") is not None:
        p.do_sample = bool(g["do_sample"])
    eos = g.get("eos_token_id")
    if eos is not None:
        p.stop_token_ids = list(eos) if isinstance(eos, list) else [eos]
    return p
