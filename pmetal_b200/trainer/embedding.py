"""Embedding-model fine-tuning: pooling and contrastive objectives.

Follows crates/pmetal-trainer/src/embedding_trainer.rs and contrastive_loss.rs: mean / last-token / CLS pooling over the
final hidden states, L2 normalisation, and InfoNCE (in-batch negatives, temperature 0.05), triplet (margin on cosine
distance) and CoSENT (pairwise ranking of cosine similarities against graded labels, scale 20) losses."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


def pool(hidden: torch.Tensor, cu: Sequence[int], mode: str = "mean", normalize: bool = True) -> torch.Tensor:
    """hidden [T, H] of a packed stream with boundaries ``cu`` -> [n_seq, H]."""
    outs = []
    for a, b in zip(cu[:-1], cu[1:]):
        h = hidden[a:b].float()
        outs.append(h.mean(0) if mode == "mean" else h[-1] if mode == "last" else h[0])
    e = torch.stack(outs)
    return F.normalize(e, dim=-1) if normalize else e


def info_nce(anchors: torch.Tensor, positives: torch.Tensor, temperature: float = 0.05,
             negatives: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In-batch negatives: row i's positive is column i; optional explicit hard negatives are appended as columns."""
    cand = positives if negatives is None else torch.cat([positives, negatives], 0)
    logits = anchors @ cand.t() / temperature
    return F.cross_entropy(logits, torch.arange(anchors.shape[0], device=anchors.device))


def triplet_loss(anchors, positives, negatives, margin: float = 0.5) -> torch.Tensor:
    dp = 1 - (anchors * positives).sum(-1)
    dn = 1 - (anchors * negatives).sum(-1)
    return F.relu(dp - dn + margin).mean()


def cosent_loss(a: torch.Tensor, b: torch.Tensor, labels: torch.Tensor, scale: float = 20.0) -> torch.Tensor:
    """log(1 + sum over pairs (i, j) with label_i < label_j of exp(scale * (cos_i - cos_j)))."""
    cos = (a * b).sum(-1) * scale
    diff = cos[:, None] - cos[None, :]
    mask = labels[:, None] < labels[None, :]
    diff = diff.masked_fill(~mask, float("-inf")).reshape(-1)
    return torch.logsumexp(torch.cat([diff.new_zeros(1), diff]), 0)


@dataclass
class EmbeddingConfig:
    loss: str = "infonce"            # infonce | triplet | cosent
    pooling: str = "mean"
    temperature: float = 0.05
    margin: float = 0.5
    learning_rate: float = 2e-5
    max_grad_norm: float = 1.0
    max_length: int = 512
    weight_decay: float = 0.0
    normalize: bool = True           # unit-length embeddings (cosine similarities in the losses)


class EmbeddingTrainer:
    def __init__(self, model, cfg: EmbeddingConfig = EmbeddingConfig(), optimizer=None):
        from .logprob_utils import is_fast_decoder
        from .optimizer import FlatAdamW, attach_shadows
        self.model, self.cfg = model, cfg
        self.device = next(model.parameters()).device
        self.fast = is_fast_decoder(model)
        shadow = torch.bfloat16 if (self.device.type == "cuda" and self.fast) else None
        self.opt = optimizer or FlatAdamW(model.named_parameters(), lr=cfg.learning_rate, weight_decay=cfg.weight_decay,
                                          max_grad_norm=cfg.max_grad_norm, shadow_dtype=shadow)
        if shadow is not None:
            attach_shadows(model, self.opt)

    def _encode_padded(self, seqs: Sequence[Sequence[int]], grad: bool) -> torch.Tensor:
        """Encoders (BERT family: ``forward(ids, attention_mask)`` + ``pool``) and config-driven decoders (``forward_hidden``
        on right-padded rows; causal attention keeps the padding out of the real positions): masked pooling."""
        rows = [list(s)[: self.cfg.max_length] or [0] for s in seqs]
        L = max(len(r) for r in rows)
        ids = torch.zeros(len(rows), L, dtype=torch.int64, device=self.device)
        mask = torch.zeros(len(rows), L, dtype=torch.int64, device=self.device)
        for i, r in enumerate(rows):
            ids[i, :len(r)] = torch.tensor(r, device=self.device)
            mask[i, :len(r)] = 1
        mode = self.cfg.pooling
        with (torch.enable_grad() if grad else torch.no_grad()):
            if hasattr(self.model, "pool") and not hasattr(self.model, "forward_hidden"):
                h = self.model(ids, mask)
                return self.model.pool(h, mask, {"first": "cls"}.get(mode, mode), self.cfg.normalize)
            h = self.model.forward_hidden(ids).float()
            m = mask[..., None].float()
            if mode == "last":
                e = h[torch.arange(len(rows), device=self.device), mask.sum(1) - 1]
            elif mode in ("first", "cls"):
                e = h[:, 0]
            else:
                e = (h * m).sum(1) / m.sum(1).clamp(min=1.0)
            return F.normalize(e, dim=-1) if self.cfg.normalize else e

    def encode(self, seqs: Sequence[Sequence[int]], grad: bool = False) -> torch.Tensor:
        if not self.fast:
            return self._encode_padded(seqs, grad)
        ids: List[int] = []
        pos: List[int] = []
        cu = [0]
        for s in seqs:
            s = list(s)[: self.cfg.max_length]
            ids.extend(s)
            pos.extend(range(len(s)))
            cu.append(cu[-1] + len(s))
        dev = self.device
        cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
        ss = torch.repeat_interleave(cu_t[:-1], (cu_t[1:] - cu_t[:-1]).long()).to(torch.int32)
        with (torch.enable_grad() if grad else torch.no_grad()):
            h = self.model.forward_hidden(torch.tensor(ids, dtype=torch.int64, device=dev),
                                          torch.tensor(pos, dtype=torch.int32, device=dev), cu_t, ss)
            return pool(h, cu, self.cfg.pooling, self.cfg.normalize)

    def step(self, anchors, positives, negatives=None, labels=None) -> dict:
        c = self.cfg
        self.opt.zero_grad()
        a, p = self.encode(anchors, True), self.encode(positives, True)
        if c.loss == "infonce":
            loss = info_nce(a, p, c.temperature, self.encode(negatives, True) if negatives else None)
        elif c.loss == "triplet":
            loss = triplet_loss(a, p, self.encode(negatives, True), c.margin)
        elif c.loss == "cosent":
            loss = cosent_loss(a, p, torch.as_tensor(labels, dtype=torch.float32, device=self.device))
        else:
            raise ValueError(c.loss)
        loss.backward()
        gn = self.opt.step(1.0)
        return {"loss": float(loss.detach()), "grad_norm": float(gn)}
