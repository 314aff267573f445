"""Two-model speculative decoding for the config-driven architectures.

A small draft proposes ``k`` tokens one by one on its own contiguous cache; the target scores the last accepted token
and the ``k`` proposals in one forward of ``k + 1`` tokens, keeps the longest prefix it agrees with (greedy) or accepts
each proposal with probability min(1, p_target / p_draft) and resamples the first rejected position from the positive
part of p_target - p_draft (sampling), and both caches are cut back to the accepted length. The output distribution is
that of the target alone; with greedy decoding the text is identical token for token. Accept / reject rules:
crates/pmetal-mlx/src/speculative.rs:411-615 (``verify_greedy``, ``verify_logits``, ``adjust_k``). Any pair of models with
the same vocabulary works, attention-only stacks (caches of recurrent layers cannot be rolled back)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .generic import KVCache


def truncate_cache(cache: KVCache, length: int) -> None:
    """Forget everything after the first ``length`` positions (plain contiguous caches only)."""
    if type(cache) is not KVCache:
        raise TypeError("speculative decoding needs the plain contiguous cache (no quantised cache)")
    if cache.state:
        raise TypeError("recurrent layers keep a state that cannot be rolled back")
    for i, k in enumerate(cache.k):
        if k is not None and k.shape[2] > length:
            cache.k[i] = k[:, :, :length]
            cache.v[i] = cache.v[i][:, :, :length]


@dataclass
class SpeculativeStats:
    rounds: int = 0
    proposed: int = 0
    accepted: int = 0
    tokens: List[int] = field(default_factory=list)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0


@torch.no_grad()
def speculative_generate(target, draft, prompt: Sequence[int], max_tokens: int, k: int = 4, eos_ids: Sequence[int] = (),
                         temperature: float = 0.0, generator: Optional[torch.Generator] = None,
                         adaptive: bool = True) -> SpeculativeStats:
    """Generate up to ``max_tokens`` tokens after ``prompt`` (one sequence). ``temperature`` 0 = greedy. With
    ``adaptive`` the number of proposals grows by one after a round in which all were accepted and shrinks by one after a
    round in which none was (between 1 and 2 k)."""
    dev = next(target.parameters()).device
    eos = set(eos_ids)
    st = SpeculativeStats()
    tc, dc = target.new_cache(), draft.new_cache()
    ids = torch.tensor([list(prompt)], device=dev)
    t_logits = target(ids, tc)[:, -1].float()
    draft(ids, dc)
    k_now, k_max = max(1, k), max(2 * k, 1)

    def probs(lg):
        return torch.softmax(lg / temperature, -1)

    def pick(lg):
        if temperature <= 0:
            return int(lg.argmax(-1))
        return int(torch.multinomial(probs(lg), 1, generator=generator))

    nxt = pick(t_logits[0])
    st.tokens.append(nxt)
    while len(st.tokens) < max_tokens and nxt not in eos:
        base = tc.length()                          # positions held by both caches before this round
        # --- draft proposes
        prop, q_rows = [], []
        cur = nxt
        for _ in range(min(k_now, max_tokens - len(st.tokens))):
            lg = draft(torch.tensor([[cur]], device=dev), dc)[:, -1].float()[0]
            q_rows.append(lg)
            cur = pick(lg)
            prop.append(cur)
        # --- target scores the accepted token and all proposals at once
        block = torch.tensor([[nxt] + prop], device=dev)
        lg_t = target(block, tc)[0].float()          # row i: distribution after block[:i + 1]
        n_ok = 0
        bonus = None
        for i, tok in enumerate(prop):
            if temperature <= 0:
                want = int(lg_t[i].argmax(-1))
                if want != tok:
                    bonus = want
                    break
            else:
                p, q = probs(lg_t[i]), probs(q_rows[i])
                u = torch.rand((), device=dev, generator=generator)
                if float(u) * float(q[tok]) > float(p[tok]):
                    resid = (p - q).clamp(min=0)
                    resid = resid / resid.sum().clamp(min=1e-20)
                    bonus = int(torch.multinomial(resid, 1, generator=generator))
                    break
            n_ok += 1
            if tok in eos:
                break
        st.rounds += 1
        st.proposed += len(prop)
        st.accepted += n_ok
        out = prop[:n_ok]
        if bonus is None and not (out and out[-1] in eos):
            bonus = pick(lg_t[n_ok])                 # every proposal accepted: one more token from the target for free
        if bonus is not None:
            out = out + [bonus]
        room = max_tokens - len(st.tokens)
        out = out[:room]
        for t_ in out:
            st.tokens.append(t_)
            if t_ in eos:
                break
        nxt = st.tokens[-1]
        # both caches keep the prompt, everything emitted before this round, the round's first token and the accepted
        # proposals; the bonus token enters the caches at the start of the next round
        keep = base + 1 + n_ok
        truncate_cache(tc, keep)
        if dc.length() < keep:                       # the draft never saw its last proposal: feed it
            draft(torch.tensor([[prop[n_ok - 1]]], device=dev), dc)
        truncate_cache(dc, keep)
        if adaptive and prop:
            if n_ok == len(prop):
                k_now = min(k_now + 1, k_max)
            elif n_ok == 0:
                k_now = max(k_now - 1, 1)
    return st
