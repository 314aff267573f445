"""Group-relative policy optimisation (GRPO) with DAPO / DR-GRPO / BNPO / REINFORCE reductions.

Semantics follow crates/pmetal-trainer/src/grpo.rs:76-1715:
* advantages: reward minus group mean, divided by the *sample* standard deviation of the group (floor
  1e-4) when whitening is on (:604-611);
* loss: PPO-clip surrogate on the ratio against the generation-time (old) log-probs with separate
  low/high epsilons; reductions — BNPO/DAPO/REINFORCE: mean over completion tokens of the batch,
  DR-GRPO: per-sequence token mean then batch mean (:714-735);
* KL to the frozen reference by the k3 estimator exp(r) - 1 - r with r = ref - pi, weight beta (:737-752);
* DAPO extras: -1 penalty on length-truncated completions, groups whose accuracy is 0 or 1 are dropped
  (dynamic sampling), eps_high 0.28 (:268-278, 623-664).

The reference generates the G completions of one prompt serially; here every prompt of the step is
prefilled once, its KV blocks are shared by its G samples and all rollouts decode as one batch on the
paged cache. Generation and policy-update phases are timed separately.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from ..models.generation import Generator
from ..models.sampling import SamplingParams
from ..ops import functional as ops


@dataclass
class GrpoConfig:
    num_generations: int = 8
    max_prompt_length: int = 512
    max_completion_length: int = 512
    beta: float = 0.1
    temperature: float = 1.0
    top_p: float = 0.95
    top_k: int = 40
    whiten_advantages: bool = True
    epsilon_low: float = 0.2
    epsilon_high: float = 0.2
    loss_type: str = "bnpo"              # bnpo | dr_grpo | dapo | reinforce
    entropy_coef: float = 0.0
    learning_rate: float = 1e-6
    max_grad_norm: float = 1.0
    dapo_overlong_penalty: float = -1.0
    dapo_min_group_size: int = 2
    dapo_dynamic_sampling: bool = True
    dapo_accuracy_reward_threshold: float = 0.5
    dapo_dynamic_sampling_min_accuracy: float = 0.01
    logprob_chunk: int = 4096
    rollout_merged: bool = True          # generate from W + s B A folded into one bf16 weight (adapter-free decode path)

    @classmethod
    def dapo(cls, **kw) -> "GrpoConfig":
        d = dict(num_generations=16, beta=0.0, epsilon_high=0.28, loss_type="dapo", top_p=0.95)
        d.update(kw)
        return cls(**d)


def group_advantages(rewards: Sequence[float], num_prompts: int, whiten: bool = True) -> List[float]:
    n = len(rewards) // max(num_prompts, 1)
    if n == 0 or n * num_prompts != len(rewards):
        raise ValueError("rewards must be num_prompts x group_size")
    out = [0.0] * len(rewards)
    for i in range(num_prompts):
        g = rewards[i * n:(i + 1) * n]
        mean = sum(g) / n
        if whiten and n > 1:
            std = max(math.sqrt(sum((r - mean) ** 2 for r in g) / (n - 1)), 1e-4)
            for j in range(n):
                out[i * n + j] = (g[j] - mean) / std
        else:
            for j in range(n):
                out[i * n + j] = g[j] - mean
    return out


def grpo_loss(logps: torch.Tensor, old_logps: torch.Tensor, ref_logps: Optional[torch.Tensor], advantages: torch.Tensor,
              mask: torch.Tensor, seq_index: torch.Tensor, n_seq: int, cfg: GrpoConfig):
    """All inputs are flat over completion tokens [N]; ``advantages`` is per token (already expanded),
    ``seq_index`` maps tokens to sequences. Returns (loss, kl_mean, policy_loss)."""
    ratio = torch.exp(logps - old_logps)
    clipped = ratio.clamp(1.0 - cfg.epsilon_low, 1.0 + cfg.epsilon_high)
    tok = -torch.minimum(ratio * advantages, clipped * advantages) * mask
    total = mask.sum().clamp(min=1.0)
    if cfg.loss_type == "dr_grpo":
        per_sum = torch.zeros(n_seq, dtype=tok.dtype, device=tok.device).index_add_(0, seq_index, tok)
        per_cnt = torch.zeros(n_seq, dtype=tok.dtype, device=tok.device).index_add_(0, seq_index, mask)
        policy = (per_sum / per_cnt.clamp(min=1.0)).mean()
    else:
        policy = tok.sum() / total
    kl = logps.new_zeros(())
    if ref_logps is not None:
        r = ref_logps - logps
        kl = ((torch.exp(r) - 1.0 - r) * mask).sum() / total
    return policy + cfg.beta * kl, kl, policy


RewardFn = Callable[[List[List[int]], List[List[int]]], List[float]]


def mod7_length_reward(prompts: List[List[int]], completions: List[List[int]]) -> List[float]:
    """Deterministic synthetic reward: fraction of generated ids divisible by 7 minus 0.001 per token."""
    return [(sum(1 for t in c if t % 7 == 0) / max(len(c), 1)) - 0.001 * len(c) for c in completions]


@dataclass
class GrpoStepStats:
    loss: float = 0.0
    kl: float = 0.0
    policy_loss: float = 0.0
    mean_reward: float = 0.0
    completion_tokens: int = 0
    generation_seconds: float = 0.0
    train_seconds: float = 0.0
    skipped_groups: int = 0

    @property
    def gen_tok_per_s(self) -> float:
        return self.completion_tokens / self.generation_seconds if self.generation_seconds > 0 else 0.0


class RolloutWeights:
    """Context manager for the generation phase: every adapted projection is replaced by one bf16 weight
    W + s B A (refreshed from the current factors on entry, in buffers that keep their address from step to step), and
    the factors are hidden, so that rollouts run on the adapter-free decode path (the whole-step kernel, the tensor-core
    mat-vec and the CUDA graphs captured over them) instead of the slower adapter-aware one. The training forward is
    untouched: on exit the base weights and the factors are back. Packed (quantised) bases are left alone."""

    def __init__(self, model):
        self.items = []
        for _, _, fl in model.fused_linears():
            if fl.lora_a is None or getattr(fl, "qweight", None) is not None or fl.weight.dtype != torch.bfloat16:
                continue
            self.items.append((fl, torch.empty_like(fl.weight.data)))
        self.saved = []

    @torch.no_grad()
    def __enter__(self):
        self.saved = []
        for fl, buf in self.items:
            buf.copy_(fl.weight.data)
            o = 0
            for i, sz in enumerate(fl.seg_sizes):
                if fl.active[i]:
                    a = fl.lora_a.detach()[i * fl.r:(i + 1) * fl.r].to(torch.bfloat16)
                    b = fl.lora_b.detach()[o:o + sz].to(torch.bfloat16)
                    buf[o:o + sz].addmm_(b, a, alpha=fl.scale)
                o += sz
            self.saved.append((fl.weight.data, fl.lora_a, fl.lora_b, getattr(fl, "lora_a_c", None), getattr(fl, "lora_b_c", None)))
            fl.weight.data = buf
            fl.lora_a = fl.lora_b = None
            fl.lora_a_c = fl.lora_b_c = None
        return self

    def __exit__(self, *exc):
        for (fl, _), (w, a, b, ac, bc) in zip(self.items, self.saved):
            fl.weight.data = w
            fl.lora_a, fl.lora_b = a, b
            fl.lora_a_c, fl.lora_b_c = ac, bc
        self.saved = []
        return False


class GrpoTrainer:
    def __init__(self, policy, cfg: GrpoConfig, reward_fn: RewardFn, reference=None, eos_ids: Sequence[int] = (),
                 kv_blocks: int = 8192, dist=None, optimizer=None):
        from .optimizer import FlatAdamW, attach_shadows
        self.policy, self.ref, self.cfg, self.reward_fn, self.eos_ids = policy, reference, cfg, reward_fn, list(eos_ids)
        self.dist = dist
        self.device = policy.embed_tokens.device
        shadow = torch.bfloat16 if self.device.type == "cuda" else None
        self.opt = optimizer or FlatAdamW(policy.named_parameters(), lr=cfg.learning_rate, weight_decay=0.0,
                                          max_grad_norm=cfg.max_grad_norm, shadow_dtype=shadow)
        if dist is not None and getattr(dist, "fused", False):
            dist.bind_optimizer(self.opt)
        if shadow is not None:
            attach_shadows(policy, self.opt)
        self.gen = Generator(policy, num_blocks=kv_blocks)
        self.rollout_weights = (RolloutWeights(policy) if self.device.type == "cuda" and getattr(cfg, "rollout_merged", True)
                                else None)
        self.step_count = 0

    # ------------------------------------------------------------------ rollout phase
    @torch.no_grad()
    def generate(self, prompts: List[List[int]]):
        c = self.cfg
        sp = SamplingParams(temperature=c.temperature, top_k=c.top_k, top_p=c.top_p, min_p=0.0,
                            repetition_penalty=1.0, max_tokens=c.max_completion_length, do_sample=True)
        was = self.policy.training
        self.policy.eval()
        import contextlib
        with (self.rollout_weights if self.rollout_weights is not None and self.rollout_weights.items
              else contextlib.nullcontext()):
            res = self.gen.generate([p[-c.max_prompt_length:] for p in prompts], sp, self.eos_ids,
                                    num_return_sequences=c.num_generations, track_history=False)
        self.policy.train(was)
        return res

    # ------------------------------------------------------------------ log-probs of completions
    def _completion_logps(self, model, seqs: List[List[int]], prompt_lens: List[int], grad: bool):
        """Packed forward over prompt+completion streams; returns flat per-token log-probs of completion tokens
        (and the sequence index of each)."""
        from ..data.packing import PackedBatch, collate_packs
        ids: List[int] = []
        pos: List[int] = []
        cu = [0]
        for s in seqs:
            ids.extend(s)
            pos.extend(range(len(s)))
            cu.append(cu[-1] + len(s))
        dev = self.device
        T = len(ids)
        cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
        seq_start = torch.repeat_interleave(cu_t[:-1], (cu_t[1:] - cu_t[:-1]).long()).to(torch.int32)
        inp = torch.tensor(ids, dtype=torch.int64, device=dev)
        post = torch.tensor(pos, dtype=torch.int32, device=dev)
        # position t predicts token t+1; completion tokens are those at index >= prompt_len within a sequence
        sel, seq_idx = [], []
        for i, (s, pl) in enumerate(zip(seqs, prompt_lens)):
            for t in range(max(pl, 1), len(s)):
                sel.append(cu[i] + t - 1)
                seq_idx.append(i)
        sel_t = torch.tensor(sel, dtype=torch.int64, device=dev)
        tgt = inp[sel_t + 1]
        ctx = torch.enable_grad() if grad else torch.no_grad()
        with ctx:
            h = model.forward_hidden(inp, post, cu_t, seq_start)
            lp = ops.token_logprobs(h[sel_t], model.head_weight(), tgt, self.cfg.logprob_chunk, model.head_t)
        return lp, torch.tensor(seq_idx, dtype=torch.int64, device=dev)

    # ------------------------------------------------------------------ one GRPO step
    def step(self, prompts: List[List[int]]) -> GrpoStepStats:
        c = self.cfg
        st = GrpoStepStats()
        t0 = time.perf_counter()
        res = self.generate(prompts)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        st.generation_seconds = time.perf_counter() - t0
        G = c.num_generations
        rep_prompts = [p[-c.max_prompt_length:] for p in prompts for _ in range(G)]
        rewards = list(self.reward_fn(rep_prompts, res.tokens))
        st.completion_tokens = sum(len(t) for t in res.tokens)
        st.mean_reward = sum(rewards) / max(len(rewards), 1)
        keep_groups = list(range(len(prompts)))
        if c.loss_type == "dapo":
            for i in range(len(rewards)):
                if res.finish_reasons[i] == "length":
                    rewards[i] += c.dapo_overlong_penalty
            if c.dapo_dynamic_sampling:
                keep_groups = []
                for g in range(len(prompts)):
                    grp = rewards[g * G:(g + 1) * G]
                    acc = sum(1 for r in grp if r > c.dapo_accuracy_reward_threshold) / G
                    lo = c.dapo_dynamic_sampling_min_accuracy
                    if lo < acc < 1.0 - lo and G >= c.dapo_min_group_size:
                        keep_groups.append(g)
                st.skipped_groups = len(prompts) - len(keep_groups)
        adv = group_advantages(rewards, len(prompts), c.whiten_advantages)
        idx = [g * G + j for g in keep_groups for j in range(G)]
        t1 = time.perf_counter()
        if idx:
            seqs = [rep_prompts[i] + res.tokens[i] for i in idx]
            plens = [len(rep_prompts[i]) for i in idx]
            old_lp, seq_idx = self._completion_logps(self.policy, seqs, plens, grad=False)
            ref_lp = None
            if c.beta > 0 and self.ref is not None:
                ref_lp, _ = self._completion_logps(self.ref, seqs, plens, grad=False)
            self.opt.zero_grad()
            lp, _ = self._completion_logps(self.policy, seqs, plens, grad=True)
            adv_t = torch.tensor([adv[i] for i in idx], dtype=torch.float32, device=self.device)[seq_idx]
            mask = torch.ones_like(lp)
            loss, kl, pol = grpo_loss(lp.float(), old_lp.float().detach(), None if ref_lp is None else ref_lp.float(),
                                      adv_t, mask, seq_idx, len(idx), c)
            loss.backward()
            if self.dist is not None and self.dist.world_size > 1:
                self.dist.reduce_and_step(self.opt, 1.0)
            else:
                self.opt.step(1.0)
            st.loss, st.kl, st.policy_loss = float(loss.detach()), float(kl.detach()), float(pol.detach())
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        st.train_seconds = time.perf_counter() - t1
        self.step_count += 1
        return st
