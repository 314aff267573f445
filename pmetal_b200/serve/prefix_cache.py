"""Serving prefix cache: finished prompts keep their KV blocks so that a later request with the same token prefix
forks them instead of recomputing the prefill.

Policy follows crates/pmetal-serve/src/prefix_cache.rs: at most ``max_entries`` (16) entries and ``max_bytes`` (2 GiB)
of KV, least-recently-used eviction, longest-prefix match on token ids. On the paged cache an entry is just a parked
sequence id whose blocks are reference-counted, so a hit costs one block-table copy."""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

from ..models.kv_cache import BLOCK, PagedKVCache


class PrefixCache:
    def __init__(self, cache: PagedKVCache, max_entries: int = 16, max_bytes: int = 2 << 30, min_tokens: int = BLOCK):
        self.cache, self.max_entries, self.max_bytes, self.min_tokens = cache, max_entries, max_bytes, min_tokens
        self.entries: "OrderedDict[int, Tuple[List[int], int]]" = OrderedDict()     # seq id -> (tokens, bytes)
        self.hits = self.misses = 0
        self._next = -1          # parked sequences use negative ids

    def _bytes_per_token(self) -> int:
        k = self.cache.k[0]
        return 2 * len(self.cache.k) * k.shape[2] * k.shape[3] * k.element_size()

    def total_bytes(self) -> int:
        return sum(b for _, b in self.entries.values())

    def lookup(self, tokens: Sequence[int]) -> Tuple[Optional[int], int]:
        """Longest cached prefix of ``tokens`` that leaves at least one token to prefill. Returns (entry id, length)."""
        best, best_len = None, 0
        for sid, (toks, _) in self.entries.items():
            n = 0
            lim = min(len(toks), len(tokens) - 1)
            while n < lim and toks[n] == tokens[n]:
                n += 1
            n = (n // BLOCK) * BLOCK           # whole blocks only: a forked sequence appends into fresh blocks
            if n > best_len:
                best, best_len = sid, n
        if best is None or best_len < self.min_tokens:
            self.misses += 1
            return None, 0
        self.hits += 1
        self.entries.move_to_end(best)
        return best, best_len

    def attach(self, entry: int, length: int, new_seq: int) -> None:
        """Make ``new_seq`` share the first ``length`` cached tokens of ``entry``."""
        self.cache.fork(entry, new_seq)
        self.cache.truncate(new_seq, length)

    def insert(self, seq_id: int, tokens: Sequence[int]) -> None:
        """Park a copy of ``seq_id``'s blocks (its first len(tokens) positions) under a new entry."""
        n = (len(tokens) // BLOCK) * BLOCK
        if n < self.min_tokens:
            return
        toks = list(tokens[:n])
        for _, (t, _) in self.entries.items():
            if len(t) >= n and t[:n] == toks:
                return
        sid = self._next
        self._next -= 1
        self.cache.fork(seq_id, sid)
        self.cache.truncate(sid, n)
        self.entries[sid] = (toks, n * self._bytes_per_token())
        while len(self.entries) > self.max_entries or self.total_bytes() > self.max_bytes:
            old, _ = self.entries.popitem(last=False)
            self.cache.free_sequence(old)

    def evict_for_blocks(self, needed: int) -> None:
        while self.entries and self.cache.num_free() < needed:
            old, _ = self.entries.popitem(last=False)
            self.cache.free_sequence(old)

    def clear(self) -> None:
        for sid in list(self.entries):
            self.cache.free_sequence(sid)
        self.entries.clear()
