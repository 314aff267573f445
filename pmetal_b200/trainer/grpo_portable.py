"""GRPO / DAPO for the config-driven architectures (Gemma, Phi, Cohere, Granite, DeepSeek, GPT-OSS, Llama 4, ...).

The algorithm (group advantages, clipped ratio, KL to a reference, DAPO filtering and over-length penalty) is the one of
``GrpoTrainer``; what changes is how the model is driven. Rollouts run on the model's own contiguous cache with the
``num_generations`` copies of a prompt as one batch (identical prompts need no padding); log-probabilities come from a
right-padded batch through ``forward_hidden`` with the read-out applied to the completion positions only, so the
[sequences, tokens, vocabulary] logits are never formed. The policy carries portable LoRA adapters (``lora/portable.py``);
the reference policy is the same network with the adapters switched off, so no second copy of the weights is held.
Reference: crates/pmetal-trainer/src/grpo.rs (GRPO over any ``TrainableModel``)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..models.generation import GenerationResult
from ..models.sampling import Sampler, SamplingParams
from .grpo import GrpoConfig, GrpoTrainer, RewardFn


class _TorchOpt:
    """The two calls ``GrpoTrainer.step`` makes on its optimiser, on top of ``torch.optim.AdamW`` with global-norm clipping."""

    def __init__(self, params, lr: float, max_grad_norm: float):
        self.params = list(params)
        self.opt = torch.optim.AdamW(self.params, lr=lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
        self.max_grad_norm = max_grad_norm

    def zero_grad(self) -> None:
        self.opt.zero_grad(set_to_none=True)

    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        if grad_scale != 1.0:
            for p in self.params:
                if p.grad is not None:
                    p.grad.mul_(grad_scale)
        gn = torch.nn.utils.clip_grad_norm_(self.params, self.max_grad_norm or float("inf"))
        self.opt.step()
        return gn.reshape(1)


class _AdaptersOff:
    """Context in which every portable LoRA wrapper computes the base projection only (the frozen reference policy)."""

    def __init__(self, model):
        from ..lora.portable import lora_modules
        self.mods = list(lora_modules(model).values())

    def __enter__(self):
        self.saved = [m.scale for m in self.mods]
        for m in self.mods:
            m.scale = 0.0

    def __exit__(self, *exc):
        for m, s in zip(self.mods, self.saved):
            m.scale = s


class _ReferenceHandle:
    """Stands for "the policy without its adapters" where ``GrpoTrainer.step`` passes a reference model around."""


class PortableGrpoTrainer(GrpoTrainer):
    def __init__(self, policy, cfg: GrpoConfig, reward_fn: RewardFn, eos_ids: Sequence[int] = (), pad_id: int = 0,
                 logprob_batch: int = 8):
        self.policy, self.cfg, self.reward_fn, self.eos_ids = policy, cfg, reward_fn, list(eos_ids)
        self.dist = None
        self.device = next(policy.parameters()).device
        train = [p for p in policy.parameters() if p.requires_grad]
        if not train:
            raise ValueError("the policy has no trainable parameters (apply_lora_portable first)")
        self.opt = _TorchOpt(train, cfg.learning_rate, cfg.max_grad_norm)
        # the reference policy is this network with its adapters off: a handle that _completion_logps recognises
        self.ref = _ReferenceHandle() if cfg.beta > 0 else None
        self.pad_id, self.logprob_batch = pad_id, logprob_batch
        self.rollout_weights = None
        self.step_count = 0

    # ------------------------------------------------------------------ rollouts
    @torch.no_grad()
    def generate(self, prompts: List[List[int]]) -> GenerationResult:
        c = self.cfg
        sp = SamplingParams(temperature=c.temperature, top_k=c.top_k, top_p=c.top_p, min_p=0.0, repetition_penalty=1.0,
                            max_tokens=c.max_completion_length, do_sample=True)
        sampler = Sampler(sp, self.device)
        eos = set(self.eos_ids)
        was = self.policy.training
        self.policy.eval()
        G = c.num_generations
        tokens: List[List[int]] = []
        reasons: List[str] = []
        for p in prompts:
            p = p[-c.max_prompt_length:] or [self.pad_id]
            cache = self.policy.new_cache()
            cur = torch.tensor([p] * G, device=self.device)
            outs: List[List[int]] = [[] for _ in range(G)]
            done = [None] * G
            for _ in range(c.max_completion_length):
                logits = self.policy(cur, cache)[:, -1].float()
                nxt = sampler.sample(logits, None).tolist()
                for g in range(G):
                    if done[g] is None:
                        outs[g].append(int(nxt[g]))
                        if nxt[g] in eos:
                            done[g] = "stop"
                if all(d is not None for d in done):
                    break
                cur = torch.tensor([[t] for t in nxt], device=self.device)
            tokens.extend(outs)
            reasons.extend(d or "length" for d in done)
        self.policy.train(was)
        return GenerationResult(tokens=tokens, finish_reasons=reasons, prompt_tokens=sum(len(p) for p in prompts) * G)

    # ------------------------------------------------------------------ log-probabilities of the completion tokens
    def _completion_logps(self, model, seqs: List[List[int]], prompt_lens: List[int], grad: bool):
        """Flat log-probabilities of every completion token (position t predicts token t + 1) and the index of its
        sequence. The reference handle evaluates the policy with its adapters off."""
        import contextlib

        from .logprob_utils import padded_completion_logps
        is_ref = isinstance(model, _ReferenceHandle)
        with (_AdaptersOff(self.policy) if is_ref else contextlib.nullcontext()):
            return padded_completion_logps(self.policy if is_ref else model, seqs, prompt_lens, grad and not is_ref,
                                           self.logprob_batch, self.pad_id)
