"""Batch iterators.

* ``DataLoader`` — padded batches; shuffling uses one seed on every rank and each
  rank then takes ``indices[rank::world]`` (crates/pmetal-data/src/dataloader.rs:68-141);
  inputs are padded to the batch maximum with ``pad_token_id`` and labels with −100
  (dataloader.rs:224-340).
* ``PackedDataLoader`` — packs the whole dataset once, then yields groups of packs.
"""
from __future__ import annotations

import random
from typing import Iterator, List, Optional, Sequence

import torch

from .packing import (IGNORE_INDEX, PackedBatch, PackedTensors, PackerConfig, PackingStats, Sample, SequencePacker,
                      collate_packs)


class DataLoader:
    def __init__(self, samples: Sequence[Sample], batch_size: int, shuffle: bool = True, seed: int = 42,
                 pad_token_id: int = 0, max_seq_len: Optional[int] = None, rank: int = 0, world_size: int = 1,
                 drop_last: bool = False):
        self.samples, self.batch_size, self.shuffle, self.seed = samples, batch_size, shuffle, seed
        self.pad_token_id, self.max_seq_len = pad_token_id, max_seq_len
        self.rank, self.world_size, self.drop_last = rank, world_size, drop_last
        self.epoch = 0

    def _indices(self) -> List[int]:
        idx = list(range(len(self.samples)))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        return idx[self.rank::self.world_size]

    def __len__(self) -> int:
        n = len(self._indices())
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __iter__(self) -> Iterator[dict]:
        idx = self._indices()
        for s in range(0, len(idx), self.batch_size):
            chunk = idx[s:s + self.batch_size]
            if self.drop_last and len(chunk) < self.batch_size:
                break
            yield self.collate([self.samples[i] for i in chunk])

    def collate(self, batch: Sequence[Sample]) -> dict:
        m = max(len(s) for s in batch)
        if self.max_seq_len:
            m = min(m, self.max_seq_len)
        ids = torch.full((len(batch), m), self.pad_token_id, dtype=torch.int64)
        lab = torch.full((len(batch), m), IGNORE_INDEX, dtype=torch.int64)
        att = torch.zeros((len(batch), m), dtype=torch.int64)
        for i, s in enumerate(batch):
            n = min(len(s), m)
            ids[i, :n] = torch.tensor(s.input_ids[:n])
            lab[i, :n] = torch.tensor((s.labels if s.labels is not None else s.input_ids)[:n])
            att[i, :n] = 1
        return {"input_ids": ids, "labels": lab, "attention_mask": att, "tokens": int(att.sum())}


class PackedDataLoader:
    def __init__(self, samples: Sequence[Sample], pack_len: int, packs_per_batch: int = 1, shuffle: bool = True,
                 seed: int = 42, rank: int = 0, world_size: int = 1, pad_token_id: int = 0,
                 fixed_shape: bool = True, algorithm: str = "ffd"):
        cfg = PackerConfig(max_length=pack_len, algorithm=algorithm, max_seq_length=pack_len)
        self.packs: List[PackedBatch] = SequencePacker(cfg).pack(samples)
        self.stats = PackingStats.from_batches(self.packs, pack_len)
        self.pack_len, self.packs_per_batch = pack_len, packs_per_batch
        self.shuffle, self.seed, self.rank, self.world_size = shuffle, seed, rank, world_size
        self.pad_token_id, self.fixed_shape = pad_token_id, fixed_shape
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _indices(self) -> List[int]:
        idx = list(range(len(self.packs)))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        return idx[self.rank::self.world_size]

    def __len__(self) -> int:
        return -(-len(self._indices()) // self.packs_per_batch)

    def __iter__(self) -> Iterator[PackedTensors]:
        idx = self._indices()
        for s in range(0, len(idx), self.packs_per_batch):
            group = [self.packs[i] for i in idx[s:s + self.packs_per_batch]]
            yield collate_packs(group, self.pack_len if self.fixed_shape else None, self.pad_token_id)


def synthetic_documents(n_docs: int, min_len: int, max_len: int, vocab: int, seed: int = 0) -> List[Sample]:
    """Uniform-random documents (lengths uniform in [min_len, max_len], tokens uniform in [0, vocab))."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(min_len, max_len + 1, (n_docs,), generator=g).tolist()
    out = []
    for n in lens:
        ids = torch.randint(0, vocab, (n,), generator=g).tolist()
        out.append(Sample(ids, list(ids)))
    return out
