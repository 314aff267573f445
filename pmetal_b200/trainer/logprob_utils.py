"""Per-token and per-sequence log-probabilities of completions, computed on packed streams.

All sequences of a call are concatenated into one varlen stream (per-sequence causal attention), the hidden states
of the positions that predict completion tokens are selected, and the chunked fused linear + log-softmax op returns
log p(token) without materialising logits for the whole stream. Counterpart of the reference's padded-batch helpers
(crates/pmetal-trainer/src/logprob_utils.rs)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from ..ops import functional as ops


def is_fast_decoder(model) -> bool:
    """The hand-written decoder (flat packed token streams) as opposed to a config-driven architecture ([batch, tokens])."""
    return hasattr(model, "fused_linears") and hasattr(model, "head_weight")


def padded_completion_logps(model, seqs: Sequence[Sequence[int]], prompt_lens: Sequence[int], grad: bool,
                            batch: int = 8, pad_id: int = 0, return_hidden: bool = False):
    """The same contract for a config-driven architecture: right-padded batches through ``forward_hidden`` and the model's
    own read-out (logit scale, soft cap) on the completion positions only."""
    dev = next(model.parameters()).device
    lps, idx, hid = [], [], []
    with (torch.enable_grad() if grad else torch.no_grad()):
        for b0 in range(0, len(seqs), batch):
            part = seqs[b0:b0 + batch]
            L = max(len(s) for s in part)
            ids = torch.full((len(part), L), pad_id, dtype=torch.int64, device=dev)
            rows, cols, tgt = [], [], []
            for i, s in enumerate(part):
                ids[i, :len(s)] = torch.tensor(list(s), device=dev)
                for t in range(max(prompt_lens[b0 + i], 1), len(s)):
                    rows.append(i)
                    cols.append(t - 1)
                    tgt.append(s[t])
                    idx.append(b0 + i)
            if not rows:
                continue
            h = model.forward_hidden(ids)
            sel = h[torch.tensor(rows, device=dev), torch.tensor(cols, device=dev)]
            lg = model.logits(sel).float()
            lps.append(torch.log_softmax(lg, -1).gather(-1, torch.tensor(tgt, device=dev)[:, None])[:, 0])
            hid.append(sel)
    lp = torch.cat(lps) if lps else torch.zeros(0, device=dev)
    idx_t = torch.tensor(idx, dtype=torch.int64, device=dev)
    if return_hidden:
        return lp, idx_t, (torch.cat(hid) if hid else torch.zeros(0, device=dev))
    return lp, idx_t


def packed_completion_logps(model, seqs: Sequence[Sequence[int]], prompt_lens: Sequence[int], grad: bool,
                            chunk: int = 4096, return_hidden: bool = False):
    """Returns (logps [n_completion_tokens], seq_idx [n_completion_tokens][, hidden of the selected positions])."""
    if not is_fast_decoder(model):
        return padded_completion_logps(model, seqs, prompt_lens, grad, return_hidden=return_hidden)
    dev = model.embed_tokens.device
    ids: List[int] = []
    pos: List[int] = []
    cu = [0]
    for s in seqs:
        ids.extend(s)
        pos.extend(range(len(s)))
        cu.append(cu[-1] + len(s))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    seq_start = torch.repeat_interleave(cu_t[:-1], (cu_t[1:] - cu_t[:-1]).long()).to(torch.int32)
    inp = torch.tensor(ids, dtype=torch.int64, device=dev)
    post = torch.tensor(pos, dtype=torch.int32, device=dev)
    sel, seq_idx = [], []
    for i, (s, pl) in enumerate(zip(seqs, prompt_lens)):
        for t in range(max(pl, 1), len(s)):          # position t-1 predicts token t
            sel.append(cu[i] + t - 1)
            seq_idx.append(i)
    sel_t = torch.tensor(sel, dtype=torch.int64, device=dev)
    tgt = inp[sel_t + 1]
    with (torch.enable_grad() if grad else torch.no_grad()):
        h = model.forward_hidden(inp, post, cu_t, seq_start)
        hs = h[sel_t]
        lp = ops.token_logprobs(hs, model.head_weight(), tgt, chunk, getattr(model, "head_t", None))
    idx_t = torch.tensor(seq_idx, dtype=torch.int64, device=dev)
    return (lp, idx_t, hs) if return_hidden else (lp, idx_t)


def sequence_sums(values: torch.Tensor, seq_idx: torch.Tensor, n_seq: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(sum per sequence, token count per sequence)."""
    s = torch.zeros(n_seq, dtype=values.dtype, device=values.device).index_add(0, seq_idx, values)
    n = torch.zeros(n_seq, dtype=values.dtype, device=values.device).index_add(0, seq_idx, torch.ones_like(values))
    return s, n


def sequence_logps(model, seqs, prompt_lens, grad: bool, chunk: int = 4096, average: bool = False) -> torch.Tensor:
    lp, idx = packed_completion_logps(model, seqs, prompt_lens, grad, chunk)
    s, n = sequence_sums(lp.float(), idx, len(seqs))
    return s / n.clamp(min=1) if average else s
