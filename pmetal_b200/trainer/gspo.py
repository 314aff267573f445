"""GSPO, full DAPO objective and RLKD on top of the GRPO rollout machinery.

* GSPO (crates/pmetal-trainer/src/gspo.rs:81-160,436-535): baseline = group median (or mean / trimmed mean / EWMA 0.99),
  optional length-normalised rewards, advantages clipped to +-5 and whitened, token weighting equal / positional decay /
  per-sequence; loss  sum(mask * -logp * A * w) / sum(mask * w) + beta * KL.
* DAPO (crates/pmetal-trainer/src/dapo.rs:334-356,400-583): advantage (r - mean_g) / max(std_g(population), 1e-8), token
  loss  -clamp(ratio, eps_low, 1 + eps_high) * A  averaged over all tokens of the batch, optional entropy bonus.
* RLKD (crates/pmetal-trainer/src/rlkd.rs): policy-gradient loss plus alpha * per-token KL(teacher || student) estimated
  on the sampled tokens."""
from __future__ import annotations

import statistics
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .grpo import GrpoConfig, GrpoTrainer
from .logprob_utils import packed_completion_logps


@dataclass
class GspoConfig:
    num_generations: int = 8
    beta: float = 0.01
    baseline: str = "median"            # median | mean | trimmed_mean | ewma
    ewma_decay: float = 0.99
    trim_fraction: float = 0.1
    length_normalize_rewards: bool = True
    advantage_clip: float = 5.0
    whiten: bool = True
    token_weighting: str = "equal"      # equal | positional_decay | sequence
    positional_decay: float = 0.999


def gspo_advantages(rewards: Sequence[float], lengths: Sequence[int], G: int, cfg: GspoConfig,
                    ewma_state: Optional[List[float]] = None) -> List[float]:
    r = [x / max(n, 1) if cfg.length_normalize_rewards else x for x, n in zip(rewards, lengths)]
    out: List[float] = []
    for g in range(len(r) // G):
        grp = r[g * G:(g + 1) * G]
        if cfg.baseline == "median":
            b = statistics.median(grp)
        elif cfg.baseline == "trimmed_mean":
            k = int(len(grp) * cfg.trim_fraction)
            s = sorted(grp)[k:len(grp) - k] or grp
            b = sum(s) / len(s)
        elif cfg.baseline == "ewma" and ewma_state is not None:
            m = sum(grp) / len(grp)
            ewma_state[0] = m if ewma_state[0] is None else cfg.ewma_decay * ewma_state[0] + (1 - cfg.ewma_decay) * m
            b = ewma_state[0]
        else:
            b = sum(grp) / len(grp)
        out.extend(x - b for x in grp)
    out = [max(-cfg.advantage_clip, min(cfg.advantage_clip, a)) for a in out]
    if cfg.whiten and len(out) > 1:
        m = sum(out) / len(out)
        sd = (sum((a - m) ** 2 for a in out) / (len(out) - 1)) ** 0.5
        out = [(a - m) / max(sd, 1e-8) for a in out]
    return out


def gspo_loss(logps, advantages, seq_idx, n_seq: int, cfg: GspoConfig, ref_logps=None, positions=None):
    w = torch.ones_like(logps)
    if cfg.token_weighting == "positional_decay" and positions is not None:
        w = cfg.positional_decay ** positions.to(logps.dtype)
    elif cfg.token_weighting == "sequence":
        n = torch.zeros(n_seq, dtype=logps.dtype, device=logps.device).index_add(0, seq_idx, torch.ones_like(logps))
        w = 1.0 / n[seq_idx].clamp(min=1)
    pol = (-(logps * advantages) * w).sum() / w.sum().clamp(min=1e-8)
    kl = torch.zeros((), device=logps.device)
    if ref_logps is not None and cfg.beta > 0:
        r = ref_logps - logps
        kl = ((torch.exp(r) - 1 - r) * w).sum() / w.sum().clamp(min=1e-8)
    return pol + cfg.beta * kl, pol.detach(), kl.detach()


def dapo_advantages(rewards: Sequence[float], G: int) -> List[float]:
    out: List[float] = []
    for g in range(len(rewards) // G):
        grp = rewards[g * G:(g + 1) * G]
        m = sum(grp) / len(grp)
        sd = (sum((x - m) ** 2 for x in grp) / len(grp)) ** 0.5 if len(grp) >= 2 else 1.0
        out.extend((x - m) / max(sd, 1e-8) for x in grp)
    return out


def dapo_token_loss(logps, old_logps, advantages, eps_low: float = 0.0, eps_high: float = 0.28):
    ratio = torch.exp(logps - old_logps)
    return (-(torch.clamp(ratio, eps_low, 1.0 + eps_high) * advantages)).mean()


class GspoTrainer(GrpoTrainer):
    def __init__(self, policy, cfg: GspoConfig, reward_fn, reference=None, grpo_cfg: Optional[GrpoConfig] = None, **kw):
        g = grpo_cfg or GrpoConfig(num_generations=cfg.num_generations, beta=cfg.beta)
        super().__init__(policy, g, reward_fn, reference, **kw)
        self.gcfg = cfg
        self._ewma: List[Optional[float]] = [None]

    def step(self, prompts: List[List[int]]):
        c, g = self.cfg, self.gcfg
        res = self.generate(prompts)
        G = c.num_generations
        rep = [p[-c.max_prompt_length:] for p in prompts for _ in range(G)]
        rewards = list(self.reward_fn(rep, res.tokens))
        adv = gspo_advantages(rewards, [len(t) for t in res.tokens], G, g, self._ewma)
        keep = [i for i, t in enumerate(res.tokens) if len(t) > 0]
        seqs = [rep[i] + res.tokens[i] for i in keep]
        plens = [len(rep[i]) for i in keep]
        ref_lp = None
        if g.beta > 0 and self.ref is not None:
            ref_lp, _ = packed_completion_logps(self.ref, seqs, plens, False, c.logprob_chunk)
            ref_lp = ref_lp.float()
        self.opt.zero_grad()
        lp, idx = packed_completion_logps(self.policy, seqs, plens, True, c.logprob_chunk)
        adv_t = torch.tensor([adv[i] for i in keep], dtype=torch.float32, device=self.device)[idx]
        first = torch.zeros(len(seqs), dtype=torch.long, device=self.device)
        first[1:] = torch.cumsum(torch.bincount(idx, minlength=len(seqs)), 0)[:-1]
        positions = torch.arange(idx.numel(), device=self.device) - first[idx]
        loss, pol, kl = gspo_loss(lp.float(), adv_t, idx, len(seqs), g, ref_lp, positions)
        loss.backward()
        self.opt.step(1.0)
        self.step_count += 1
        return {"loss": float(loss.detach()), "policy_loss": float(pol), "kl": float(kl),
                "mean_reward": sum(rewards) / max(len(rewards), 1)}


class RlkdTrainer(GrpoTrainer):
    """GRPO whose loss adds alpha * KL(teacher || student) on the sampled completion tokens."""

    def __init__(self, policy, cfg: GrpoConfig, reward_fn, teacher, alpha: float = 0.5, **kw):
        super().__init__(policy, cfg, reward_fn, **kw)
        self.teacher, self.alpha = teacher, alpha

    def step(self, prompts: List[List[int]]):
        from .grpo import group_advantages, grpo_loss
        c = self.cfg
        res = self.generate(prompts)
        G = c.num_generations
        rep = [p[-c.max_prompt_length:] for p in prompts for _ in range(G)]
        rewards = list(self.reward_fn(rep, res.tokens))
        adv = group_advantages(rewards, len(prompts), c.whiten_advantages)
        keep = [i for i, t in enumerate(res.tokens) if len(t) > 0]
        seqs = [rep[i] + res.tokens[i] for i in keep]
        plens = [len(rep[i]) for i in keep]
        old_lp, idx = self._completion_logps(self.policy, seqs, plens, False)
        t_lp, _ = packed_completion_logps(self.teacher, seqs, plens, False, c.logprob_chunk)      # either model kind
        self.opt.zero_grad()
        lp, _ = self._completion_logps(self.policy, seqs, plens, True)
        adv_t = torch.tensor([adv[i] for i in keep], dtype=torch.float32, device=self.device)[idx]
        rl, kl, pol = grpo_loss(lp.float(), old_lp.float().detach(), None, adv_t, torch.ones_like(lp), idx, len(seqs), c)
        # on-policy samples x ~ student: KL(student || teacher) ~ E[log p_s - log p_t]; the teacher-forcing direction
        # uses the k3 estimator with r = log p_t - log p_s
        r = t_lp.float() - lp.float()
        kd = (torch.exp(r) - 1 - r).mean()
        loss = rl + self.alpha * kd
        loss.backward()
        self.opt.step(1.0)
        self.step_count += 1
        return {"loss": float(loss.detach()), "rl_loss": float(rl.detach()), "kd_loss": float(kd.detach()),
                "mean_reward": sum(rewards) / max(len(rewards), 1)}


def portable_rlkd_trainer(policy, cfg: GrpoConfig, reward_fn, teacher, alpha: float = 0.5, **kw):
    """RLKD for a config-driven policy (adapters from ``lora/portable.py``): the step above on top of the rollouts and
    log-probabilities of ``PortableGrpoTrainer``; the teacher may be of either kind."""
    from .grpo_portable import PortableGrpoTrainer

    class PortableRlkdTrainer(PortableGrpoTrainer):
        step = RlkdTrainer.step

    tr = PortableRlkdTrainer(policy, cfg, reward_fn, **kw)
    tr.teacher, tr.alpha = teacher, alpha
    return tr
