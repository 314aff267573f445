"""Reward functions for RL fine-tuning (crates/pmetal-trainer/src/grpo.rs reward section, reward_model.rs):
XML format reward, answer-accuracy reward with extraction, length reward, weighted combination, and a model-based
reward that scores completions with a sequence-classification head."""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

RewardFn = Callable[[List[List[int]], List[List[int]]], List[float]]

_FORMAT_RE = re.compile(r"^\s*<think>.*?</think>\s*<answer>.*?</answer>\s*$", re.S)
_ANSWER_RE = re.compile(r"<answer>(.*?)</answer>", re.S)
_BOXED_RE = re.compile(r"\\boxed\{([^}]*)\}")
_NUM_RE = re.compile(r"-?\d+(?:\.\d+)?")


def xml_format_reward(text: str) -> float:
    """1.0 for exactly ``<think>...</think><answer>...</answer>``, partial credit (0.25 each) for present tags."""
    if _FORMAT_RE.match(text):
        return 1.0
    return 0.25 * sum(tag in text for tag in ("<think>", "</think>", "<answer>", "</answer>")) * 0.5


def extract_answer(text: str) -> Optional[str]:
    for rx in (_ANSWER_RE, _BOXED_RE):
        m = rx.findall(text)
        if m:
            return m[-1].strip()
    nums = _NUM_RE.findall(text)
    return nums[-1] if nums else None


def accuracy_reward(text: str, target: str) -> float:
    got = extract_answer(text)
    if got is None:
        return 0.0
    if got.strip() == target.strip():
        return 1.0
    try:
        return 1.0 if abs(float(got) - float(target)) < 1e-6 else 0.0
    except ValueError:
        return 0.0


def make_reward(kind: str, tokenizer, targets: Optional[Dict[str, str]] = None) -> RewardFn:
    """``targets`` maps the decoded prompt to its reference answer (accuracy reward)."""
    def fn(prompts, completions):
        out = []
        for p, c in zip(prompts, completions):
            text = tokenizer.decode(c)
            if kind == "format":
                out.append(xml_format_reward(text))
            elif kind == "length":
                out.append(min(len(c), 256) / 256.0)
            elif kind == "accuracy":
                tgt = (targets or {}).get(tokenizer.decode(p))
                out.append(accuracy_reward(text, tgt) if tgt is not None else xml_format_reward(text))
            else:
                raise ValueError(kind)
        return out
    return fn


def combined_reward(fns: Sequence[RewardFn], weights: Sequence[float]) -> RewardFn:
    def fn(prompts, completions):
        parts = [f(prompts, completions) for f in fns]
        return [sum(w * p[i] for w, p in zip(weights, parts)) for i in range(len(completions))]
    return fn


@dataclass
class RewardModelConfig:
    """How a reward model reads a prompt + completion (crates/pmetal-trainer/src/reward_model.rs:47-120)."""
    max_length: int = 2048             # longer inputs are cut from the right
    use_last_token: bool = True        # False: mean over all positions
    batch_size: int = 16               # sequences per packed forward
    template: Optional[str] = None     # "... {prompt} ... {completion} ..." applied on text (needs a tokenizer)


class ModelReward:
    """Scores prompt + completion with a frozen decoder. Strategies of the reference's ``MLRewardModel``: a scalar head
    on the pooled hidden state (``score.weight`` of sequence-classification checkpoints) or, without a head, the mean of
    the read-out logits at the pooled position. Sequences are scored several at a time: the fast decoder takes them as one
    packed token stream (documents do not see each other), the config-driven architectures one row each."""

    def __init__(self, model, head_weight=None, config: Optional[RewardModelConfig] = None, tokenizer=None):
        self.model, self.head = model, head_weight
        self.cfg = config or RewardModelConfig()
        self.tok = tokenizer
        if self.cfg.template and tokenizer is None:
            raise ValueError("a reward template works on text and needs the tokenizer")
        self.strategy = "score_head" if head_weight is not None else "mean_logits"

    def _sequences(self, prompts, completions) -> List[List[int]]:
        out = []
        for p, c in zip(prompts, completions):
            if self.cfg.template:
                text = self.cfg.template.replace("{prompt}", self.tok.decode(list(p))).replace("{completion}", self.tok.decode(list(c)))
                ids = self.tok.encode(text)
            else:
                ids = list(p) + list(c)
            out.append((ids or [0])[: self.cfg.max_length])
        return out

    def _score(self, pooled):
        import torch
        if self.head is not None:
            return pooled.float() @ self.head.float().reshape(-1)
        m = self.model
        logits = m.logits(pooled) if hasattr(m, "logits") else torch.nn.functional.linear(pooled, m.head_weight())
        return logits.float().mean(-1)

    def __call__(self, prompts, completions):
        import torch
        seqs = self._sequences(prompts, completions)
        dev = next(self.model.parameters()).device
        fast = hasattr(self.model, "fused_linears")
        out: List[float] = []
        with torch.no_grad():
            for b0 in range(0, len(seqs), max(self.cfg.batch_size, 1)):
                part = seqs[b0:b0 + self.cfg.batch_size]
                if fast:
                    lens = [len(s) for s in part]
                    ids = torch.tensor([t for s in part for t in s], dtype=torch.int64, device=dev)
                    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
                    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).to(dev)
                    start = torch.repeat_interleave(cu[:-1], torch.tensor(lens, device=dev)).to(torch.int32)
                    h = self.model.forward_hidden(ids, pos, cu, start)
                    ends = (cu[1:] - 1).long()
                    if self.cfg.use_last_token:
                        pooled = h[ends]
                    else:
                        pooled = torch.stack([h[int(cu[i]):int(cu[i + 1])].float().mean(0) for i in range(len(part))]).to(h.dtype)
                else:
                    rows = []
                    for s_ in part:
                        h = self.model.forward_hidden(torch.tensor([s_], device=dev))[0]
                        rows.append(h[-1] if self.cfg.use_last_token else h.float().mean(0).to(h.dtype))
                    pooled = torch.stack(rows)
                out.extend(float(x) for x in self._score(pooled))
        return out
