"""PPO for language-model policies: GAE, clipped surrogate, clipped value loss, entropy bonus, adaptive KL.

Defaults and formulas follow crates/pmetal-trainer/src/ppo.rs:60-150,323-362 — clip 0.2, vf coef 0.5, entropy coef 0.01,
4 epochs, GAE lambda 0.95, gamma 1.0, normalised advantages, max grad norm 0.5; GAE recursion
``delta_t = r_t + gamma V_{t+1} (1 - done) - V_t``, ``A_t = delta_t + gamma lambda (1 - done) A_{t+1}``; the KL penalty
coefficient is scaled by 1.5 / (1/1.5) when the measured KL leaves [target/1.5, target*1.5]."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn

from .logprob_utils import packed_completion_logps


@dataclass
class PpoConfig:
    clip_range: float = 0.2
    clip_range_vf: Optional[float] = 0.2
    vf_coef: float = 0.5
    entropy_coef: float = 0.01
    ppo_epochs: int = 4
    gae_lambda: float = 0.95
    gamma: float = 1.0
    normalize_advantages: bool = True
    max_grad_norm: float = 0.5
    learning_rate: float = 1e-6
    kl_coef: float = 0.05
    target_kl: Optional[float] = 6.0
    adaptive_kl: bool = True
    max_completion_length: int = 256
    temperature: float = 1.0
    logprob_chunk: int = 4096


def compute_gae(rewards: torch.Tensor, values: torch.Tensor, dones: torch.Tensor, gamma: float, lam: float):
    """1-D tensors over time for one trajectory. Returns (advantages, returns)."""
    T = rewards.numel()
    adv = torch.zeros_like(rewards)
    last = 0.0
    for t in reversed(range(T)):
        nv = values[t + 1] if t + 1 < T else 0.0
        nd = 1.0 - dones[t]
        delta = rewards[t] + gamma * nv * nd - values[t]
        last = delta + gamma * lam * nd * last
        adv[t] = last
    return adv, adv + values


def ppo_policy_loss(logp, old_logp, adv, clip: float):
    ratio = torch.exp(logp - old_logp)
    return -torch.minimum(ratio * adv, torch.clamp(ratio, 1 - clip, 1 + clip) * adv).mean(), ratio


def ppo_value_loss(values, old_values, returns, clip: Optional[float]):
    if clip is None:
        return 0.5 * ((values - returns) ** 2).mean()
    vc = old_values + torch.clamp(values - old_values, -clip, clip)
    return 0.5 * torch.maximum((values - returns) ** 2, (vc - returns) ** 2).mean()


class AdaptiveKl:
    def __init__(self, coef: float, target: Optional[float]):
        self.coef, self.target = coef, target

    def update(self, kl: float) -> float:
        if self.target:
            if kl > self.target * 1.5:
                self.coef *= 1.5
            elif kl < self.target / 1.5:
                self.coef /= 1.5
        return self.coef


class ValueHead(nn.Module):
    def __init__(self, hidden: int, device=None):
        super().__init__()
        self.proj = nn.Linear(hidden, 1, device=device, dtype=torch.float32)
        nn.init.zeros_(self.proj.weight)
        nn.init.zeros_(self.proj.bias)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.proj(h.float()).squeeze(-1)


class PpoTrainer:
    """Rollouts with the paged generator, per-token KL-shaped rewards (sequence reward on the last token), PPO updates
    on packed streams."""

    def __init__(self, policy, cfg: PpoConfig, reward_fn: Callable[[List[List[int]], List[List[int]]], List[float]],
                 reference=None, eos_ids: Sequence[int] = (), kv_blocks: int = 4096):
        from ..models.generation import Generator
        from .optimizer import FlatAdamW, attach_shadows
        self.policy, self.ref, self.cfg, self.reward_fn, self.eos_ids = policy, reference, cfg, reward_fn, list(eos_ids)
        self.device = policy.embed_tokens.device
        self.value_head = ValueHead(policy.cfg.hidden_size, self.device)
        shadow = torch.bfloat16 if self.device.type == "cuda" else None
        named = list(policy.named_parameters()) + [("value_head." + n, p) for n, p in self.value_head.named_parameters()]
        self.opt = FlatAdamW(named, lr=cfg.learning_rate, weight_decay=0.0, max_grad_norm=cfg.max_grad_norm,
                             shadow_dtype=shadow)
        if shadow is not None:
            attach_shadows(policy, self.opt)
        self.gen = Generator(policy, num_blocks=kv_blocks)
        self.kl = AdaptiveKl(cfg.kl_coef, cfg.target_kl if cfg.adaptive_kl else None)

    def _forward(self, seqs, plens, grad):
        lp, idx, h = packed_completion_logps(self.policy, seqs, plens, grad, self.cfg.logprob_chunk, return_hidden=True)
        with (torch.enable_grad() if grad else torch.no_grad()):
            v = self.value_head(h)
        return lp.float(), idx, v

    def step(self, prompts: List[List[int]]) -> dict:
        from ..models.sampling import SamplingParams
        c = self.cfg
        sp = SamplingParams(temperature=c.temperature, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                            max_tokens=c.max_completion_length, do_sample=True)
        was = self.policy.training
        self.policy.eval()
        with torch.no_grad():
            res = self.gen.generate(prompts, sp, self.eos_ids, track_history=False)
        self.policy.train(was)
        scores = list(self.reward_fn(prompts, res.tokens))
        keep = [i for i, t in enumerate(res.tokens) if len(t) > 0]
        if not keep:
            return {"loss": 0.0, "mean_reward": 0.0}
        seqs = [prompts[i] + res.tokens[i] for i in keep]
        plens = [len(prompts[i]) for i in keep]
        old_lp, idx, old_v = self._forward(seqs, plens, False)
        ref_lp = old_lp
        if self.ref is not None:
            ref_lp, _ = packed_completion_logps(self.ref, seqs, plens, False, c.logprob_chunk)
            ref_lp = ref_lp.float()
        kl_tok = old_lp - ref_lp
        rewards = -self.kl.coef * kl_tok
        adv = torch.zeros_like(old_lp)
        ret = torch.zeros_like(old_lp)
        for j, i in enumerate(keep):
            m = (idx == j).nonzero(as_tuple=True)[0]
            r = rewards[m].clone()
            r[-1] += scores[i]
            d = torch.zeros_like(r)
            d[-1] = 1.0
            a, rt = compute_gae(r, old_v[m], d, c.gamma, c.gae_lambda)
            adv[m], ret[m] = a, rt
        if c.normalize_advantages and adv.numel() > 1:
            adv = (adv - adv.mean()) / (adv.std() + 1e-8)
        stats = {}
        for _ in range(c.ppo_epochs):
            self.opt.zero_grad()
            lp, _, v = self._forward(seqs, plens, True)
            pl, ratio = ppo_policy_loss(lp, old_lp, adv, c.clip_range)
            vl = ppo_value_loss(v, old_v, ret, c.clip_range_vf)
            ent = -lp.mean()                      # sampled-token entropy estimate
            loss = pl + c.vf_coef * vl - c.entropy_coef * ent
            loss.backward()
            self.opt.step(1.0)
            stats = {"loss": float(loss.detach()), "policy_loss": float(pl.detach()), "value_loss": float(vl.detach()),
                     "clip_frac": float(((ratio - 1).abs() > c.clip_range).float().mean())}
        kl_mean = float(kl_tok.mean())
        stats.update(kl=kl_mean, kl_coef=self.kl.update(abs(kl_mean) * 100), mean_reward=sum(scores) / len(scores))
        return stats
