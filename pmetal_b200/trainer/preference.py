"""Preference optimisation: DPO (sigmoid / IPO / hinge / robust), SimPO, ORPO, KTO, and online DPO.

Loss definitions follow the reference trainers:
* DPO  crates/pmetal-trainer/src/dpo.rs:415-535 — logits = beta * ((pi_w - ref_w) - (pi_l - ref_l)); sigmoid with label
  smoothing, IPO (logits - 1/(2 beta))^2, hinge max(0, 1 - logits), robust softplus(-logits) + 0.5 max(0, 0.5 - logits);
  reference-free mode drops the reference terms.
* SimPO crates/pmetal-trainer/src/simpo.rs:71-131 — length-normalised log-probs, beta 2.5, margin gamma 0.5, no reference.
* ORPO crates/pmetal-trainer/src/orpo.rs:4-140 — L = NLL(chosen) + lambda * -log sigmoid(log odds_w - log odds_l) with
  odds from the length-normalised log-prob.
* KTO  crates/pmetal-trainer/src/kto.rs:687-742 — desirable: w_d * sigmoid(z_ref - beta_d r), undesirable:
  w_u * sigmoid(beta_u r - z_ref), r = log pi - log ref, z_ref = clamped batch-mean KL estimate (detached).
* Online DPO crates/pmetal-trainer/src/online_dpo.rs — sample two completions per prompt, rank them with a reward
  function, train the DPO loss on the resulting pairs.
Every trainer runs the policy (and the frozen reference) on packed varlen streams through the fused kernels."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .logprob_utils import packed_completion_logps, sequence_sums


@dataclass
class PreferencePair:
    prompt: List[int]
    chosen: List[int]
    rejected: List[int]


@dataclass
class KtoExample:
    prompt: List[int]
    completion: List[int]
    desirable: bool


@dataclass
class PreferenceConfig:
    loss_type: str = "sigmoid"        # sigmoid | ipo | hinge | robust | simpo | orpo
    beta: float = 0.1
    label_smoothing: float = 0.0
    reference_free: bool = False
    simpo_gamma: float = 0.5
    orpo_lambda: float = 0.1
    learning_rate: float = 5e-7
    max_grad_norm: float = 1.0
    max_length: int = 2048
    logprob_chunk: int = 4096

    @classmethod
    def simpo(cls, **kw):
        return cls(**{**dict(loss_type="simpo", beta=2.5, simpo_gamma=0.5, reference_free=True), **kw})

    @classmethod
    def orpo(cls, **kw):
        return cls(**{**dict(loss_type="orpo", orpo_lambda=0.1, reference_free=True), **kw})


def dpo_loss(pi_w, pi_l, ref_w, ref_l, cfg: PreferenceConfig):
    """Inputs are per-pair sequence log-probs. Returns (loss, chosen_rewards, rejected_rewards)."""
    simpo = cfg.loss_type == "simpo"
    ref_free = cfg.reference_free or simpo or ref_w is None
    rw = pi_w if ref_free else pi_w - ref_w
    rl = pi_l if ref_free else pi_l - ref_l
    logits = cfg.beta * (rw - rl)
    if simpo:
        logits = logits - cfg.simpo_gamma
    if cfg.loss_type in ("sigmoid", "simpo"):
        s = cfg.label_smoothing
        loss = F.softplus(-logits) * (1 - s) + F.softplus(logits) * s if s > 0 else F.softplus(-logits)
    elif cfg.loss_type == "ipo":
        loss = (logits - 1.0 / (2.0 * cfg.beta)) ** 2
    elif cfg.loss_type == "hinge":
        loss = torch.clamp(1.0 - logits, min=0)
    elif cfg.loss_type == "robust":
        loss = F.softplus(-logits) + 0.5 * torch.clamp(0.5 - logits, min=0)
    else:
        raise ValueError(f"unknown DPO loss type {cfg.loss_type!r}")
    return loss.mean(), cfg.beta * rw.detach(), cfg.beta * rl.detach()


def orpo_loss(avg_w, avg_l, lam: float):
    """avg_*: length-normalised sequence log-probs. Returns (total, sft, odds-ratio term)."""
    def log_odds(lp):
        lp = lp.clamp(max=-1e-6)
        return lp - torch.log1p(-torch.exp(lp))
    sft = -avg_w.mean()
    ratio = -F.logsigmoid(log_odds(avg_w) - log_odds(avg_l)).mean()
    return sft + lam * ratio, sft.detach(), ratio.detach()


def kto_loss(rewards, desirable, z_ref: float, beta_d: float, beta_u: float, w_d: float = 1.0, w_u: float = 1.0):
    """rewards = log pi - log ref per example; desirable: bool tensor."""
    d = desirable.to(rewards.dtype)
    ld = torch.sigmoid(z_ref - beta_d * rewards) * w_d * d
    lu = torch.sigmoid(beta_u * rewards - z_ref) * w_u * (1 - d)
    return (ld + lu).mean()


class PreferenceTrainer:
    """DPO-family trainer on (prompt, chosen, rejected) token triples."""

    def __init__(self, policy, cfg: PreferenceConfig, reference=None, optimizer=None, dist=None):
        from .optimizer import FlatAdamW, attach_shadows
        self.policy, self.ref, self.cfg, self.dist = policy, reference, cfg, dist
        from .logprob_utils import is_fast_decoder
        self.device = next(policy.parameters()).device
        shadow = torch.bfloat16 if (self.device.type == "cuda" and is_fast_decoder(policy)) else None
        self.opt = optimizer or FlatAdamW(policy.named_parameters(), lr=cfg.learning_rate, weight_decay=0.0,
                                          max_grad_norm=cfg.max_grad_norm, shadow_dtype=shadow)
        if dist is not None and getattr(dist, "fused", False):
            dist.bind_optimizer(self.opt)
        if shadow is not None:
            attach_shadows(policy, self.opt)
        self.step_count = 0

    def _seq_logps(self, model, seqs, plens, grad, average):
        lp, idx = packed_completion_logps(model, seqs, plens, grad, self.cfg.logprob_chunk)
        s, n = sequence_sums(lp.float(), idx, len(seqs))
        return s / n.clamp(min=1) if average else s

    def loss(self, pairs: Sequence[PreferencePair]):
        c = self.cfg
        L = c.max_length
        seqs = [(p.prompt + p.chosen)[:L] for p in pairs] + [(p.prompt + p.rejected)[:L] for p in pairs]
        plens = [min(len(p.prompt), L - 1) for p in pairs] * 2
        n = len(pairs)
        average = c.loss_type in ("simpo", "orpo", "ipo")
        pi = self._seq_logps(self.policy, seqs, plens, True, average)
        if c.loss_type == "orpo":
            total, sft, ratio = orpo_loss(pi[:n], pi[n:], c.orpo_lambda)
            return total, {"sft_loss": float(sft), "or_loss": float(ratio)}
        ref = None
        if not (c.reference_free or c.loss_type == "simpo") and self.ref is not None:
            ref = self._seq_logps(self.ref, seqs, plens, False, average).detach()
        loss, rw, rl = dpo_loss(pi[:n], pi[n:], None if ref is None else ref[:n], None if ref is None else ref[n:], c)
        return loss, {"reward_chosen": float(rw.mean()), "reward_rejected": float(rl.mean()),
                      "reward_accuracy": float((rw > rl).float().mean()), "reward_margin": float((rw - rl).mean())}

    def step(self, pairs: Sequence[PreferencePair]) -> dict:
        self.opt.zero_grad()
        loss, stats = self.loss(pairs)
        loss.backward()
        if self.dist is not None and self.dist.world_size > 1:
            gn = self.dist.reduce_and_step(self.opt, 1.0)
        else:
            gn = self.opt.step(1.0)
        self.step_count += 1
        stats.update(loss=float(loss.detach()), grad_norm=float(gn))
        return stats


@dataclass
class KtoConfig:
    beta: float = 0.1
    beta_desirable: Optional[float] = None
    beta_undesirable: Optional[float] = None
    desirable_weight: float = 1.0
    undesirable_weight: float = 1.0
    learning_rate: float = 5e-7
    max_grad_norm: float = 1.0
    max_length: int = 2048
    logprob_chunk: int = 4096


class KtoTrainer(PreferenceTrainer):
    def __init__(self, policy, cfg: KtoConfig, reference, **kw):
        pc = PreferenceConfig(beta=cfg.beta, learning_rate=cfg.learning_rate, max_grad_norm=cfg.max_grad_norm,
                              max_length=cfg.max_length, logprob_chunk=cfg.logprob_chunk)
        super().__init__(policy, pc, reference, **kw)
        self.kcfg = cfg

    def loss(self, examples: Sequence[KtoExample]):
        k = self.kcfg
        L = k.max_length
        seqs = [(e.prompt + e.completion)[:L] for e in examples]
        plens = [min(len(e.prompt), L - 1) for e in examples]
        pi = self._seq_logps(self.policy, seqs, plens, True, False)
        ref = self._seq_logps(self.ref, seqs, plens, False, False).detach()
        r = pi - ref
        z_ref = float(r.detach().mean().clamp(min=0))            # batch KL estimate, never negative
        des = torch.tensor([e.desirable for e in examples], device=r.device)
        bd = k.beta_desirable if k.beta_desirable is not None else k.beta
        bu = k.beta_undesirable if k.beta_undesirable is not None else k.beta
        loss = kto_loss(r, des, z_ref, bd, bu, k.desirable_weight, k.undesirable_weight)
        return loss, {"z_ref": z_ref, "reward_mean": float((k.beta * r.detach()).mean())}


class OnlineDpoTrainer(PreferenceTrainer):
    """Samples two completions per prompt with the current policy, ranks them with ``reward_fn`` and trains DPO."""

    def __init__(self, policy, cfg: PreferenceConfig, reward_fn: Callable[[List[List[int]], List[List[int]]], List[float]],
                 reference=None, eos_ids: Sequence[int] = (), max_new_tokens: int = 256, temperature: float = 0.9,
                 kv_blocks: int = 4096, **kw):
        super().__init__(policy, cfg, reference, **kw)
        from ..models.generation import Generator
        self.reward_fn, self.eos_ids = reward_fn, list(eos_ids)
        self.max_new_tokens, self.temperature = max_new_tokens, temperature
        self.gen = Generator(policy, num_blocks=kv_blocks)

    @torch.no_grad()
    def make_pairs(self, prompts: List[List[int]]) -> List[PreferencePair]:
        from ..models.sampling import SamplingParams
        sp = SamplingParams(temperature=self.temperature, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                            max_tokens=self.max_new_tokens, do_sample=True)
        was = self.policy.training
        self.policy.eval()
        res = self.gen.generate(prompts, sp, self.eos_ids, num_return_sequences=2, track_history=False)
        self.policy.train(was)
        rep = [p for p in prompts for _ in range(2)]
        rewards = list(self.reward_fn(rep, res.tokens))
        pairs = []
        for i, p in enumerate(prompts):
            a, b = res.tokens[2 * i], res.tokens[2 * i + 1]
            ra, rb = rewards[2 * i], rewards[2 * i + 1]
            if ra == rb or not a or not b:
                continue                                   # no preference signal
            pairs.append(PreferencePair(p, a, b) if ra > rb else PreferencePair(p, b, a))
        return pairs

    def step_online(self, prompts: List[List[int]]) -> dict:
        pairs = self.make_pairs(prompts)
        if not pairs:
            return {"loss": 0.0, "pairs": 0}
        out = self.step(pairs)
        out["pairs"] = len(pairs)
        return out
