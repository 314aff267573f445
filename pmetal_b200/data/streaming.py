"""Memory-mapped token shards for pre-training (crates/pmetal-data/src/streaming.rs:66-411).

A shard is a flat little-endian ``u32`` token file ``*.bin`` with an optional ``*.idx`` of ``u64`` document offsets
(in tokens). ``ShardWriter`` appends documents; ``TokenShardDataset`` memory-maps the shards and yields fixed-length
windows (or whole documents) sharded by ``rank`` / ``world`` with a seeded shuffle of window order per epoch."""
from __future__ import annotations

import glob
import os
from typing import Iterator, List, Optional, Sequence

import numpy as np


class ShardWriter:
    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "wb")
        self._offsets: List[int] = [0]

    def add_document(self, tokens: Sequence[int]) -> None:
        arr = np.asarray(tokens, dtype="<u4")
        self._fh.write(arr.tobytes())
        self._offsets.append(self._offsets[-1] + arr.size)

    def close(self) -> None:
        self._fh.close()
        np.asarray(self._offsets, dtype="<u8").tofile(os.path.splitext(self.path)[0] + ".idx")

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class TokenShardDataset:
    def __init__(self, pattern_or_paths, seq_len: int, rank: int = 0, world: int = 1, seed: int = 42,
                 shuffle: bool = True, drop_last: bool = True, loop: bool = False):
        paths = sorted(glob.glob(pattern_or_paths)) if isinstance(pattern_or_paths, str) else list(pattern_or_paths)
        if not paths:
            raise FileNotFoundError(f"no token shards match {pattern_or_paths!r}")
        self.shards = [np.memmap(p, dtype="<u4", mode="r") for p in paths]
        self.seq_len, self.rank, self.world, self.seed, self.shuffle, self.drop_last = seq_len, rank, world, seed, shuffle, drop_last
        self.index = []                    # (shard, start)
        for si, sh in enumerate(self.shards):
            n = sh.size // seq_len if drop_last else -(-sh.size // seq_len)
            self.index.extend((si, i * seq_len) for i in range(n))
        self.epoch = 0
        self.cursor = 0                    # windows of the current epoch already handed out (this rank)
        self.loop = loop                   # keep going into the next epoch (new shuffle) instead of stopping

    def state_dict(self) -> dict:
        """Exact position in the stream: resuming from it yields the windows an uninterrupted run would have seen next
        (the reference's ``StreamPosition``, crates/pmetal-data/src/streaming.rs:66-80,333)."""
        return {"epoch": int(self.epoch), "cursor": int(self.cursor), "seed": int(self.seed), "windows": len(self.index)}

    def load_state_dict(self, d: dict) -> None:
        if d.get("windows") not in (None, len(self.index)) or d.get("seed", self.seed) != self.seed:
            raise ValueError("stream position belongs to a different shard set, window length or seed")
        self.epoch, self.cursor = int(d["epoch"]), int(d["cursor"])

    def __len__(self) -> int:
        return len(self.index[self.rank::self.world])

    def total_tokens(self) -> int:
        return int(sum(s.size for s in self.shards))

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __iter__(self) -> Iterator[np.ndarray]:
        while True:
            order = np.arange(len(self.index))
            if self.shuffle:
                np.random.default_rng(self.seed + self.epoch).shuffle(order)
            mine = order[self.rank::self.world]
            for k in range(self.cursor, len(mine)):
                si, start = self.index[mine[k]]
                self.cursor = k + 1
                yield np.asarray(self.shards[si][start:start + self.seq_len], dtype=np.int64)
            self.cursor = 0
            if not self.loop or len(mine) == 0:
                return
            self.epoch += 1

    def documents(self, shard: int) -> Optional[np.ndarray]:
        idx = os.path.splitext(self.shards[shard].filename)[0] + ".idx"
        return np.fromfile(idx, dtype="<u8") if os.path.exists(idx) else None
