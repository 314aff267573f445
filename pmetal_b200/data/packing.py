"""Sequence packing: several documents per fixed-length token stream.

Semantics follow the reference packer (crates/pmetal-data/src/packing.rs:59-841):
greedy (order-preserving) or first-fit-decreasing bin packing, per-document position
ids restarting at 0, ``cu_seqlens`` boundaries, and — because the loss shifts labels
by one — the label of the *first* token of every non-first document is masked so the
last token of one document is never trained to predict the first of the next.
The reference then builds a dense [T,T] mask from the boundaries; here the
boundaries feed the varlen attention kernel directly.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence

import torch

IGNORE_INDEX = -100


@dataclass
class Sample:
    input_ids: List[int]
    labels: Optional[List[int]] = None
    attention_mask: Optional[List[int]] = None

    def __len__(self) -> int:
        return len(self.input_ids)


@dataclass
class PackedBatch:
    input_ids: List[int]
    position_ids: List[int]
    cu_seqlens: List[int]
    seq_lengths: List[int]
    max_seqlen: int
    num_sequences: int
    labels: Optional[List[int]] = None

    def total_tokens(self) -> int:
        return len(self.input_ids)

    def mask_label_boundaries(self, ignore_index: int = IGNORE_INDEX) -> None:
        if self.labels is None:
            return
        off = 0
        for i, n in enumerate(self.seq_lengths):
            if i > 0 and off < len(self.labels):
                self.labels[off] = ignore_index
            off += n

    def dense_mask(self) -> torch.Tensor:
        """[T,T] additive block-diagonal causal mask (what the reference feeds its attention)."""
        n = self.total_tokens()
        m = torch.full((n, n), float("-inf"))
        off = 0
        for ln in self.seq_lengths:
            blk = torch.triu(torch.full((ln, ln), float("-inf")), diagonal=1)
            m[off:off + ln, off:off + ln] = blk
            off += ln
        return m


@dataclass
class PackerConfig:
    max_length: int = 2048
    pad_to_multiple: int = 8
    mask_boundaries: bool = True
    algorithm: str = "ffd"          # "ffd" | "greedy"
    min_length: int = 1
    max_seq_length: Optional[int] = None


@dataclass
class PackingStats:
    total_tokens: int = 0
    total_capacity: int = 0
    num_batches: int = 0
    num_sequences: int = 0
    efficiency: float = 0.0
    avg_sequences_per_batch: float = 0.0
    max_sequences_per_batch: int = 0

    @classmethod
    def from_batches(cls, batches: Sequence[PackedBatch], max_length: int) -> "PackingStats":
        if not batches:
            return cls()
        tt = sum(b.total_tokens() for b in batches)
        ns = sum(b.num_sequences for b in batches)
        return cls(tt, len(batches) * max_length, len(batches), ns, tt / (len(batches) * max_length),
                   ns / len(batches), max(b.num_sequences for b in batches))

    def summary(self) -> str:
        return (f"{self.num_sequences} sequences -> {self.num_batches} packs, {self.efficiency * 100:.1f}% full, "
                f"{self.avg_sequences_per_batch:.1f} seq/pack (max {self.max_sequences_per_batch})")


class SequencePacker:
    def __init__(self, config: Optional[PackerConfig] = None):
        self.config = config or PackerConfig()

    def _prepare(self, s: Sample) -> Sample:
        m = self.config.max_seq_length
        if m is not None and len(s) > m:
            return Sample(s.input_ids[:m], s.labels[:m] if s.labels is not None else None,
                          s.attention_mask[:m] if s.attention_mask is not None else None)
        return s

    def pack(self, samples: Sequence[Sample]) -> List[PackedBatch]:
        if self.config.algorithm == "greedy":
            bins = self._bins_greedy(samples)
        else:
            bins = self._bins_ffd(samples)
        return [self._make(b) for b in bins if b]

    def _bins_greedy(self, samples) -> List[List[Sample]]:
        cfg, bins, cur, used = self.config, [], [], 0
        for s in samples:
            if len(s) < cfg.min_length:
                continue
            s = self._prepare(s)
            n = len(s)
            if n > cfg.max_length:
                continue
            if used + n > cfg.max_length and cur:
                bins.append(cur)
                cur, used = [], 0
            cur.append(s)
            used += n
        if cur:
            bins.append(cur)
        return bins

    def _bins_ffd(self, samples) -> List[List[Sample]]:
        """First-fit decreasing. The scan for the first bin with room uses a max-tree over remaining
        capacities, O(log n) per item, and returns the same bins as a linear first-fit scan."""
        cfg = self.config
        items = [self._prepare(s) for s in samples if len(s) >= cfg.min_length]
        items = [s for s in items if len(s) <= cfg.max_length]
        order = sorted(range(len(items)), key=lambda i: -len(items[i]))   # stable: ties keep input order
        cap = 1
        while cap < max(len(items), 1):
            cap *= 2
        tree = [0] * (2 * cap)            # remaining room per bin; unopened bins hold max_length
        for i in range(cap):
            tree[cap + i] = cfg.max_length
        for i in range(cap - 1, 0, -1):
            tree[i] = max(tree[2 * i], tree[2 * i + 1])
        bins: List[List[Sample]] = []
        for idx in order:
            s = items[idx]
            n = len(s)
            node = 1
            while node < cap:
                node = 2 * node if tree[2 * node] >= n else 2 * node + 1
            b = node - cap
            while len(bins) <= b:
                bins.append([])
            bins[b].append(s)
            tree[node] -= n
            node //= 2
            while node:
                tree[node] = max(tree[2 * node], tree[2 * node + 1])
                node //= 2
        return bins

    def _make(self, samples: List[Sample]) -> PackedBatch:
        ids: List[int] = []
        pos: List[int] = []
        cu = [0]
        lens = []
        for s in samples:
            ids.extend(s.input_ids)
            pos.extend(range(len(s)))
            lens.append(len(s))
            cu.append(cu[-1] + len(s))
        labels = None
        if all(s.labels is not None for s in samples):
            labels = []
            for s in samples:
                labels.extend(s.labels)
        b = PackedBatch(ids, pos, cu, lens, max(lens) if lens else 0, len(samples), labels)
        if self.config.mask_boundaries:
            b.mask_label_boundaries(IGNORE_INDEX)
        return b


def compute_pack_seq_len(sequence_lengths: Sequence[int], model_max_seq_len: int) -> int:
    """p99 length rounded up to a power of two, capped by the model maximum (packing.rs:826-841)."""
    if not sequence_lengths:
        return model_max_seq_len
    s = sorted(sequence_lengths)
    import math
    idx = math.ceil(len(s) * 0.99)
    p99 = s[min(max(idx - 1, 0), len(s) - 1)]
    pow2 = 1 << max(p99 - 1, 0).bit_length() if p99 > 1 else 1
    return min(pow2, model_max_seq_len)


@dataclass
class PackedTensors:
    """Device-ready view of one or more packs concatenated into a single token stream."""
    input_ids: torch.Tensor        # [T] int64
    labels: torch.Tensor           # [T] int64 (unshifted; boundary-masked)
    position_ids: torch.Tensor     # [T] int32
    cu_seqlens: torch.Tensor       # [n_docs+1] int32
    seq_start: torch.Tensor        # [T] int32: first token index of the token's document
    total_tokens: int = 0          # real (non-padding) tokens
    num_sequences: int = 0
    max_seqlen: int = 0

    def to(self, device, non_blocking: bool = True) -> "PackedTensors":
        return PackedTensors(*(t.to(device, non_blocking=non_blocking) for t in
                               (self.input_ids, self.labels, self.position_ids, self.cu_seqlens, self.seq_start)),
                             self.total_tokens, self.num_sequences, self.max_seqlen)

    def pin(self) -> "PackedTensors":
        return PackedTensors(*(t.pin_memory() for t in
                               (self.input_ids, self.labels, self.position_ids, self.cu_seqlens, self.seq_start)),
                             self.total_tokens, self.num_sequences, self.max_seqlen)


def collate_packs(packs: Sequence[PackedBatch], pack_len: Optional[int] = None, pad_id: int = 0) -> PackedTensors:
    """Concatenate packs into one stream. With ``pack_len`` each pack is right-padded to that length by a
    trailing pseudo-document of ignored tokens, so the stream has a fixed shape (CUDA-graph friendly)."""
    ids: List[int] = []
    lab: List[int] = []
    pos: List[int] = []
    cu = [0]
    real = nseq = mx = 0
    for p in packs:
        ids.extend(p.input_ids)
        lab.extend(p.labels if p.labels is not None else p.input_ids)
        if p.labels is None and len(cu) > 1:
            pass
        pos.extend(p.position_ids)
        base = cu[-1]
        cu.extend(base + c for c in p.cu_seqlens[1:])
        real += p.total_tokens()
        nseq += p.num_sequences
        mx = max(mx, p.max_seqlen)
        if pack_len is not None and p.total_tokens() < pack_len:
            padn = pack_len - p.total_tokens()
            ids.extend([pad_id] * padn)
            lab.extend([IGNORE_INDEX] * padn)
            pos.extend(range(padn))
            cu.append(cu[-1] + padn)
    # first token of each pack must not be predicted from the previous pack's last token
    off = 0
    for p in packs:
        if off > 0:
            lab[off] = IGNORE_INDEX
        off += max(p.total_tokens(), pack_len or 0)
    T = len(ids)
    cu_t = torch.tensor(cu, dtype=torch.int32)
    seq_start = torch.repeat_interleave(cu_t[:-1], (cu_t[1:] - cu_t[:-1]).to(torch.int64)).to(torch.int32)
    assert seq_start.numel() == T
    return PackedTensors(torch.tensor(ids, dtype=torch.int64), torch.tensor(lab, dtype=torch.int64),
                         torch.tensor(pos, dtype=torch.int32), cu_t, seq_start, real, nseq, mx)
