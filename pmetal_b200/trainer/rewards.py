"""Reward functions for RL fine-tuning (crates/pmetal-trainer/src/grpo.rs reward section, reward_model.rs):
XML format reward, answer-accuracy reward with extraction, length reward, weighted combination, and a model-based
reward that scores completions with a sequence-classification head."""
from __future__ import annotations

import re
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


class ModelReward:
    """Scores prompt+completion with a decoder whose last hidden state feeds a scalar head (reward model)."""

    def __init__(self, model, head_weight=None):
        import torch
        self.model = model
        dev = model.embed_tokens.device
        self.head = head_weight if head_weight is not None else torch.zeros(model.cfg.hidden_size, device=dev)

    def __call__(self, prompts, completions):
        import torch
        out = []
        dev = self.model.embed_tokens.device
        with torch.no_grad():
            for p, c in zip(prompts, completions):
                ids = torch.tensor(list(p) + list(c), dtype=torch.int64, device=dev)
                T = ids.numel()
                h = self.model.forward_hidden(ids, torch.arange(T, dtype=torch.int32, device=dev),
                                              torch.tensor([0, T], dtype=torch.int32, device=dev),
                                              torch.zeros(T, dtype=torch.int32, device=dev))
                out.append(float(h[-1].float() @ self.head.float()))
        return out
