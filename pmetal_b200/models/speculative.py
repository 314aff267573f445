"""Speculative decoding: draft proposes k tokens, the target verifies them in one forward.

Three pieces, matching the reference's split:

* accept/reject rules (crates/pmetal-mlx/src/speculative.rs:343-620): greedy — accept token i iff the
  target's argmax at position i equals it, at the first mismatch emit the target's argmax, if all k are
  accepted emit the bonus token; sampling — accept with probability min(1, p_t/p_d), on rejection sample
  from normalize(max(0, p_t - p_d)), which preserves the target distribution; adaptive k — after a round
  with acceptance > 0.8 grow k by one (max 2 k0), below 0.4 shrink by one (min 1) (speculative.rs:602-615).
* a two-model decoder (draft model + target model, both on paged caches); the reference ships only the
  verifier for this case (speculative.rs:28-32).
* layer-split self-speculation (crates/pmetal-models/src/speculative.rs:208-384): the draft is the first
  max(1, L/3) layers of the target followed by the shared final norm and output head.

Rejected draft tokens are rolled back by truncating the paged sequences.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .generation import Generator
from .sampling import SamplingParams


@dataclass
class SpeculativeConfig:
    num_draft_tokens: int = 5
    temperature: float = 0.0
    min_acceptance_rate: float = 0.5
    adaptive_k: bool = True


@dataclass
class SpecStats:
    rounds: int = 0
    proposed: int = 0
    accepted: int = 0
    emitted: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_round(self) -> float:
        return self.emitted / self.rounds if self.rounds else 0.0


def verify_greedy(target_logits: torch.Tensor, draft: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """target_logits [B, k+1, V], draft [B, k] -> (n_accepted [B], next_token [B])."""
    tgt = target_logits.argmax(-1)                                   # [B, k+1]
    match = (tgt[:, :-1] == draft).to(torch.int32)
    n_acc = torch.cumprod(match, dim=1).sum(dim=1)                   # leading matches
    nxt = tgt.gather(1, n_acc[:, None].long())[:, 0]                  # correction, or bonus when all accepted
    return n_acc, nxt


def verify_sampling(target_logits: torch.Tensor, draft: torch.Tensor, draft_probs: torch.Tensor,
                    temperature: float, generator: Optional[torch.Generator] = None):
    """Rejection sampling. draft_probs [B, k, V] are the distributions the draft sampled from."""
    B, k1, V = target_logits.shape
    k = k1 - 1
    pt = torch.softmax(target_logits.float() / max(temperature, 1e-6), dim=-1)
    u = torch.rand(B, k, device=draft.device, generator=generator)
    ptx = pt[:, :k].gather(-1, draft[..., None])[..., 0]
    pdx = draft_probs.gather(-1, draft[..., None])[..., 0]
    ok = (u < torch.clamp(ptx / pdx.clamp_min(1e-20), max=1.0)).to(torch.int32)
    n_acc = torch.cumprod(ok, dim=1).sum(dim=1)
    idx = n_acc.clamp(max=k)[:, None, None].expand(B, 1, V).long()
    p_next = pt.gather(1, idx)[:, 0]
    pd_pad = torch.cat([draft_probs, torch.zeros(B, 1, V, device=draft.device, dtype=draft_probs.dtype)], 1)
    resid = torch.clamp(p_next - pd_pad.gather(1, idx)[:, 0], min=0.0)
    z = resid.sum(-1, keepdim=True)
    resid = torch.where(z > 0, resid / z.clamp_min(1e-20), p_next)
    nxt = torch.multinomial(resid, 1, generator=generator)[:, 0]
    return n_acc, nxt


def adjust_k(k: int, k0: int, round_acceptance: float) -> int:
    if round_acceptance > 0.8:
        return min(k + 1, 2 * k0)
    if round_acceptance < 0.4:
        return max(k - 1, 1)
    return k


def optimal_k(target_latency: float, draft_latency: float) -> int:
    return int(min(max(round(math.sqrt(target_latency / max(draft_latency, 1e-9))), 2), 10))


def is_speculative_beneficial(t_target: float, t_draft: float, k: int, acceptance: float) -> bool:
    return t_target / ((k * t_draft + t_target) / (1 + k * acceptance)) > 1.0


class SpeculativeDecoder:
    """Two-model speculative decoding over a batch of sequences (greedy or sampling verification)."""

    def __init__(self, target, draft, cfg: Optional[SpeculativeConfig] = None, target_blocks: int = 4096,
                 draft_blocks: int = 4096, cuda_graphs: Optional[bool] = None):
        self.cfg = cfg or SpeculativeConfig()
        self.t = Generator(target, num_blocks=target_blocks, cuda_graphs=cuda_graphs)
        self.d = Generator(draft, num_blocks=draft_blocks, cuda_graphs=cuda_graphs)
        self.stats = SpecStats()

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256, eos_ids: Sequence[int] = ()):
        cfg = self.cfg
        dev = self.t.device
        B = len(prompts)
        ts = [self.t.new_seq() for _ in range(B)]
        ds = [self.d.new_seq() for _ in range(B)]
        t_logits = self.t.prefill(ts, prompts)
        self.d.prefill(ds, prompts)
        greedy = cfg.temperature <= 0
        nxt = t_logits.argmax(-1) if greedy else torch.multinomial(torch.softmax(t_logits.float() / cfg.temperature, -1), 1)[:, 0]
        out: List[List[int]] = [[int(x)] for x in nxt.tolist()]
        done = [out[i][-1] in eos_ids for i in range(B)]
        k, k0 = cfg.num_draft_tokens, cfg.num_draft_tokens
        while not all(done) and max(len(o) for o in out) < max_new_tokens:
            live = [i for i in range(B) if not done[i]]
            cur = torch.tensor([out[i][-1] for i in live], device=dev)
            # ---- draft proposes k tokens (its cache receives cur + k-1 drafts)
            drafts, dprobs = [], []
            tok = cur
            for _ in range(k):
                dl = self.d.decode_step([ds[i] for i in live], tok)
                if greedy:
                    tok = dl.argmax(-1)
                else:
                    pr = torch.softmax(dl.float() / cfg.temperature, -1)
                    tok = torch.multinomial(pr, 1)[:, 0]
                    dprobs.append(pr)
                drafts.append(tok)
            draft = torch.stack(drafts, 1)                                    # [b, k]
            # ---- target verifies cur + k drafts in one forward of k+1 tokens per sequence
            ver_in = torch.cat([cur[:, None], draft], 1).reshape(-1)
            meta = self.t.cache.prepare([ts[i] for i in live], [k + 1] * len(live))
            tl = self.t.model.forward_paged(ver_in, self.t.cache, meta, all_logits=True).view(len(live), k + 1, -1)
            if greedy:
                from ..ops import functional as _ops
                if _ops.native_enabled(tl):          # accept / correct / bonus decided on the device (csrc/sampling.cu)
                    from ..ops import native as _nat
                    n_acc, new = _nat.spec_verify(tl.float().contiguous(), None, draft.to(torch.int32), 0.0)
                else:
                    n_acc, new = verify_greedy(tl, draft)
            else:
                n_acc, new = verify_sampling(tl, draft, torch.stack(dprobs, 1), cfg.temperature)
            n_l, new_l, dr_l = n_acc.tolist(), new.tolist(), draft.tolist()
            self.stats.rounds += 1
            self.stats.proposed += k * len(live)
            self.stats.accepted += sum(n_l)
            for j, i in enumerate(live):
                acc = n_l[j]
                emit = dr_l[j][:acc] + [new_l[j]]
                # roll both caches back to "everything before the newest emitted token"
                base_t = self.t.cache.length(ts[i]) - (k + 1)
                self.t.cache.truncate(ts[i], base_t + 1 + acc)
                base_d = self.d.cache.length(ds[i]) - k
                self.d.cache.truncate(ds[i], min(base_d + 1 + acc, base_d + k))
                for tkn in emit:
                    out[i].append(tkn)
                    self.stats.emitted += 1
                    if tkn in eos_ids or len(out[i]) >= max_new_tokens:
                        done[i] = True
                        break
                if acc == k and not done[i]:
                    # all drafts accepted: the draft cache has not seen its own last proposal yet
                    self.d.decode_step([ds[i]], torch.tensor([dr_l[j][-1]], device=dev))
            if cfg.adaptive_k:
                k = adjust_k(k, k0, sum(n_l) / max(k * len(live), 1))
        for s in ts:
            self.t.cache.free_sequence(s)
        for s in ds:
            self.d.cache.free_sequence(s)
        return [o[:max_new_tokens] for o in out]


class LayerSplitDraft(torch.nn.Module):
    """Self-speculation draft: the first max(1, L/3) layers of the target plus its final norm and head."""

    def __init__(self, target, num_layers: Optional[int] = None):
        super().__init__()
        import copy
        n = num_layers or max(1, len(target.layers) // 3)
        self.cfg = copy.copy(target.cfg)
        self.cfg.num_hidden_layers = n
        self.embed_tokens = target.embed_tokens
        self.layers = torch.nn.ModuleList(list(target.layers[:n]))
        self.norm = target.norm
        self.lm_head = target.lm_head
        self._target = [target]
        self._rope_schedule = None

    def head_weight(self):
        return self._target[0].head_weight()

    def logits(self, h):
        return self._target[0].logits(h)

    def new_cache(self, num_blocks, dtype=None, device=None):
        from .kv_cache import PagedKVCache
        p = self.embed_tokens
        return PagedKVCache(len(self.layers), self.cfg.num_key_value_heads, self.cfg.head_dim, num_blocks,
                            dtype or p.dtype, device or p.device)

    forward_paged = None   # bound below


def _bind_layer_split():
    from .decoder import DecoderLM
    LayerSplitDraft.forward_paged = DecoderLM.forward_paged
    LayerSplitDraft._paged_attention_reference = DecoderLM._paged_attention_reference
    LayerSplitDraft.rope = DecoderLM.rope


_bind_layer_split()
