"""Vocabulary compaction: train only the embedding / classifier rows of tokens that occur in the dataset.

A scan of the training tokens yields the active ids; a two-way map (full id <-> compact id, compact ids in increasing
full-id order) lets the embedding table, the classifier GEMM and the optimiser state shrink to the active rows
(typically 3-4x for a narrow-domain corpus) and scatters the result back afterwards
(crates/pmetal-data/src/vocab_compact.rs:11-150)."""
from __future__ import annotations

from typing import Iterable, Sequence

import torch


class VocabCompactor:
    def __init__(self, active: torch.Tensor, full_vocab: int):
        self.full_vocab = int(full_vocab)
        self.compact_to_full = active.to(torch.int64)
        self.full_to_compact = torch.full((self.full_vocab,), -1, dtype=torch.int64)
        self.full_to_compact[self.compact_to_full] = torch.arange(len(self.compact_to_full))

    @classmethod
    def from_dataset(cls, samples: Iterable[Sequence[int]], full_vocab: int) -> "VocabCompactor":
        seen = torch.zeros(full_vocab, dtype=torch.bool)
        for s in samples:
            t = torch.as_tensor(s, dtype=torch.int64)
            t = t[(t >= 0) & (t < full_vocab)]          # ignore-index labels and out-of-range ids are skipped
            seen[t] = True
        return cls(torch.nonzero(seen).flatten(), full_vocab)

    @property
    def compact_vocab(self) -> int:
        return len(self.compact_to_full)

    def to_compact(self, ids: torch.Tensor, missing: int = 0) -> torch.Tensor:
        """Full ids -> compact ids; ids outside the active set (and negative ignore labels, kept as they are) map to
        ``missing``."""
        ids = torch.as_tensor(ids, dtype=torch.int64)
        neg = ids < 0
        c = self.full_to_compact[ids.clamp(0, self.full_vocab - 1)]
        c = torch.where(c < 0, torch.full_like(c, missing), c)
        return torch.where(neg, ids, c)

    def to_full(self, ids: torch.Tensor) -> torch.Tensor:
        return self.compact_to_full[torch.as_tensor(ids, dtype=torch.int64)]

    def extract_rows(self, full: torch.Tensor) -> torch.Tensor:
        """[full_vocab, d] -> [compact_vocab, d] (embedding or classifier weight)."""
        return full.index_select(0, self.compact_to_full.to(full.device))

    def scatter_gradients(self, full_grad: torch.Tensor, compact_grad: torch.Tensor) -> None:
        full_grad.index_add_(0, self.compact_to_full.to(full_grad.device), compact_grad.to(full_grad.dtype))

    def update_full(self, full: torch.Tensor, compact: torch.Tensor) -> None:
        full.index_copy_(0, self.compact_to_full.to(full.device), compact.to(full.dtype))
