"""Native packing and collation (``csrc/host/runtime.cpp``).

:class:`TokenStore` keeps a tokenised dataset as two flat int32 arrays plus document offsets instead of Python lists;
:func:`pack_lengths` bins documents (first-fit decreasing or greedy) and :class:`FastPackedLoader` collates the packs of a
batch straight into reusable pinned host buffers with a few worker threads, so a training step's input costs one
host-to-device copy per tensor and no per-token Python work. The results are identical to
``packing.SequencePacker`` + ``packing.collate_packs`` (the semantics of the reference packer,
crates/pmetal-data/src/packing.rs:59-841); ``tests/test_fastpack.py`` checks that element by element."""
from __future__ import annotations

import ctypes
import random
from typing import Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..utils import hostlib
from .packing import PackedTensors, PackingStats, Sample

_I32P = ctypes.POINTER(ctypes.c_int32)
_I64P = ctypes.POINTER(ctypes.c_int64)
_READY = False


def _lib():
    global _READY
    L = hostlib.load()
    if not _READY:
        L.pm_pack_ffd.restype = ctypes.c_int64
        L.pm_pack_ffd.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
        L.pm_pack_greedy.restype = ctypes.c_int64
        L.pm_pack_greedy.argtypes = L.pm_pack_ffd.argtypes
        L.pm_collate_packs.restype = ctypes.c_int
        L.pm_collate_packs.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int] + \
            [ctypes.c_void_p] * 6 + [ctypes.c_int]
        _READY = True
    return L


class TokenStore:
    """Flat storage of a tokenised dataset: ``tokens``/``labels`` int32 [total], ``offsets`` int64 [n_docs + 1]."""

    def __init__(self, tokens: np.ndarray, offsets: np.ndarray, labels: Optional[np.ndarray] = None):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        self.offsets = np.ascontiguousarray(offsets, dtype=np.int64)
        self.labels = None if labels is None else np.ascontiguousarray(labels, dtype=np.int32)
        if self.labels is not None and self.labels.shape != self.tokens.shape:
            raise ValueError("labels and tokens differ in length")

    @classmethod
    def from_samples(cls, samples: Sequence[Sample]) -> "TokenStore":
        lens = np.fromiter((len(s) for s in samples), dtype=np.int64, count=len(samples))
        off = np.zeros(len(samples) + 1, dtype=np.int64)
        np.cumsum(lens, out=off[1:])
        tok = np.empty(int(off[-1]), dtype=np.int32)
        have_labels = all(s.labels is not None for s in samples) and len(samples) > 0
        lab = np.empty(int(off[-1]), dtype=np.int32) if have_labels else None
        for i, s in enumerate(samples):
            tok[off[i]:off[i + 1]] = s.input_ids
            if lab is not None:
                lab[off[i]:off[i + 1]] = s.labels
        return cls(tok, off, lab)

    def __len__(self) -> int:
        return len(self.offsets) - 1

    def lengths(self) -> np.ndarray:
        return (self.offsets[1:] - self.offsets[:-1]).astype(np.int64)


def pack_lengths(lengths: np.ndarray, capacity: int, algorithm: str = "ffd", min_length: int = 1) -> Tuple[np.ndarray, int]:
    """Bin index per document (-1 = dropped: shorter than ``min_length``) and the bin count. Lengths above ``capacity``
    are the caller's to clip (a clipped document occupies a whole pack)."""
    lens = np.ascontiguousarray(np.minimum(lengths, np.iinfo(np.int32).max), dtype=np.int32)
    out = np.empty(len(lens), dtype=np.int32)
    fn = _lib().pm_pack_ffd if algorithm == "ffd" else _lib().pm_pack_greedy
    n = fn(lens.ctypes.data, len(lens), int(capacity), int(min_length), out.ctypes.data)
    return out, int(n)


class FastPackedLoader:
    """Drop-in for ``dataloader.PackedDataLoader`` over a :class:`TokenStore`: same packs, same shuffling, same tensors.

    Batches are written into ``buffers`` rotating sets of pinned tensors (a batch stays valid until ``buffers - 1`` more
    have been produced), so the host-to-device copies of consecutive steps can overlap."""

    def __init__(self, store: TokenStore, pack_len: int, packs_per_batch: int = 1, shuffle: bool = True, seed: int = 42,
                 rank: int = 0, world_size: int = 1, pad_token_id: int = 0, algorithm: str = "ffd", threads: int = 4,
                 buffers: int = 3, pin: Optional[bool] = None):
        self.store, self.pack_len, self.packs_per_batch = store, int(pack_len), int(packs_per_batch)
        self.shuffle, self.seed, self.rank, self.world_size = shuffle, seed, rank, world_size
        self.pad_token_id, self.threads, self.epoch = int(pad_token_id), int(threads), 0
        self.doc_len = np.minimum(store.lengths(), self.pack_len).astype(np.int32)     # long documents are truncated
        bins, n_bins = pack_lengths(self.doc_len, self.pack_len, algorithm)
        # documents of a bin in placement order: FFD places by decreasing length (stable), greedy in input order
        keep = np.nonzero(bins >= 0)[0]
        if algorithm == "ffd":
            keep = keep[np.argsort(-self.doc_len[keep].astype(np.int64), kind="stable")]
        order = keep[np.argsort(bins[keep], kind="stable")]
        counts = np.bincount(bins[keep], minlength=n_bins).astype(np.int64)
        self.pack_docs = np.ascontiguousarray(order, dtype=np.int64)
        self.pack_off = np.zeros(n_bins + 1, dtype=np.int64)
        np.cumsum(counts, out=self.pack_off[1:])
        self.num_packs = n_bins
        tok = int(self.doc_len[keep].sum())
        self.stats = PackingStats(tok, n_bins * self.pack_len, n_bins, len(keep),
                                  tok / max(n_bins * self.pack_len, 1), len(keep) / max(n_bins, 1),
                                  int(counts.max()) if n_bins else 0)
        pin = torch.cuda.is_available() if pin is None else pin
        T = self.packs_per_batch * self.pack_len
        max_cu = self.packs_per_batch * ((int(counts.max()) if n_bins else 0) + 1) + 1
        self._bufs = []
        for _ in range(max(buffers, 1)):
            b = dict(ids=torch.empty(T, dtype=torch.int64), labels=torch.empty(T, dtype=torch.int64),
                     pos=torch.empty(T, dtype=torch.int32), start=torch.empty(T, dtype=torch.int32),
                     cu=torch.empty(max_cu, dtype=torch.int32))
            if pin:
                b = {k: v.pin_memory() for k, v in b.items()}
            self._bufs.append(b)
        self._next = 0
        self._pinned = bool(pin)
        self._handed = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _indices(self) -> List[int]:
        idx = list(range(self.num_packs))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        return idx[self.rank::self.world_size]

    def __len__(self) -> int:
        return -(-len(self._indices()) // self.packs_per_batch)

    def collate(self, packs: Sequence[int]) -> PackedTensors:
        docs = [self.pack_docs[self.pack_off[p]:self.pack_off[p + 1]] for p in packs]
        pd = np.ascontiguousarray(np.concatenate(docs) if docs else np.zeros(0, dtype=np.int64))
        po = np.zeros(len(packs) + 1, dtype=np.int64)
        np.cumsum([len(d) for d in docs], out=po[1:])
        b = self._bufs[self._next]
        self._next = (self._next + 1) % len(self._bufs)
        self._handed += 1
        if self._pinned and self._handed > len(self._bufs) and torch.cuda.is_initialized():
            # this buffer was handed out `buffers` batches ago; its asynchronous host-to-device copy (queued on the
            # current stream by the consumer) must have run before the buffer is overwritten
            torch.cuda.current_stream().synchronize()
        T = len(packs) * self.pack_len
        meta = np.zeros(5, dtype=np.int64)
        st = self.store
        rc = _lib().pm_collate_packs(st.tokens.ctypes.data, st.labels.ctypes.data if st.labels is not None else None,
                                     st.offsets.ctypes.data, self.doc_len.ctypes.data, pd.ctypes.data, po.ctypes.data,
                                     len(packs), self.pack_len, self.pad_token_id, 1, b["ids"].data_ptr(),
                                     b["labels"].data_ptr(), b["pos"].data_ptr(), b["start"].data_ptr(),
                                     b["cu"].data_ptr(), meta.ctypes.data, self.threads)
        if rc != 0:
            raise RuntimeError("a pack holds more tokens than pack_len")
        assert int(meta[0]) == T
        return PackedTensors(b["ids"][:T], b["labels"][:T], b["pos"][:T], b["cu"][:int(meta[1])], b["start"][:T],
                             int(meta[2]), int(meta[3]), int(meta[4]))

    def __iter__(self) -> Iterator[PackedTensors]:
        idx = self._indices()
        for s in range(0, len(idx), self.packs_per_batch):
            yield self.collate(idx[s:s + self.packs_per_batch])
